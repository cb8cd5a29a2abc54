"""Benchmark of the pair-representation trunk on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--tokens 512] [--blocks 48]
                    [--block pairformer|pairmixer] [--cp RxC] [--replicas] [--probe NAME]

A "step" is one forward of the 48-block Pairformer trunk over one pair tensor z[1, N, N, 128] and single
track s[1, N, 384] (fp32 residual streams, bf16 tensor-core arithmetic), N = 512 with the last 37 tokens
padded -- the configuration the headline metric (trunk ms/forward and pair-cells/s) is quoted on.  The
block is the benchmark's composite one (--block pairformer); --block pairmixer runs the reference trunk's
own attention-free block.  Inputs are synthetic (seeded N(0,1)), weights random-init (Kaiming-uniform
linears, LayerNorm 1/0).

One JSON line is printed by rank 0.

* 1 GPU: `value` is pair cells per second (N^2 / forward time), timed with CUDA events with z resident in HBM;
  `e2e` is the same through the public module call with pinned HOST buffers, host->device and device->host copies
  inside the timed region; `roofline` describes the dominant kernel; `parity` compares block 0 of the trunk, run on
  the bench's own inputs, with the CPU oracle; `cpu_baseline` is the CPU oracle timed on this host's cores on a
  bounded sample; `torch_gpu_baseline` is the same oracle code run on this GPU under bf16 autocast (plain torch
  kernels), outside the timed region; `ops` holds per-op times, including the outer product mean (1024 x 384 MSA)
  and the N = 1536 / 3072 sizes.
* N > 1 GPUs (torchrun): the SAME workload with ONE pair tensor tiled over an R x C grid (1x2, 2x2, 2x4) -- context
  parallelism with NCCL row / column collectives, strong scaling; `cp_parity_rel` is the sharded result against the
  single-GPU modules on a small case run first, `cp_config3` times triangle multiplication out/in + triangle attention
  start/end at N = 1536 on the same grid.  --replicas keeps the older mode (every rank its own pair tensor, no
  collective, weak scaling).
* --probe NAME runs one kernel family alone a few times (for profiler captures) and prints its time.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import torch  # noqa: E402

METRIC = "pairformer_trunk_pair_cells_per_s"
UNIT = "pair-cells/s"
GRIDS = {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4)}
PROBES = ("attention_core", "triatt", "trimul", "transition", "apb", "opm", "trunk_glue", "window_attention")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--blocks", type=int, default=48)
    ap.add_argument("--block", default="pairformer", choices=["pairformer", "pairmixer"],
                    help="pairformer: the benchmark's composite block (triangle multiplication, triangle attention, "
                         "pair transition, single-track pair-bias attention, single transition); "
                         "pairmixer: the reference trunk's own block (no attention)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the outer-product-mean, N=1536/3072 and torch-on-GPU legs of the 1-GPU run")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the kernels of the HBM-resident step one by one instead of replaying a CUDA graph")
    ap.add_argument("--cp", default=None, metavar="RxC",
                    help="grid for the context-parallel run (default: 1x2, 2x2, 2x4 for 2, 4, 8 ranks)")
    ap.add_argument("--replicas", action="store_true",
                    help="with --gpus N > 1: N independent replicas (weak scaling) instead of context parallelism")
    ap.add_argument("--config4", action="store_true",
                    help="the largest configuration, under torchrun on 4 or 8 ranks: context-parallel 48-block trunk at "
                         "N = 3072 (three chains of 1024 tokens, ragged padding) followed by 24 diffusion token blocks "
                         "(16 heads, width 768, pair bias from the trunk's pair tensor); --tokens / --blocks shrink it")
    ap.add_argument("--probe", default=None, choices=PROBES,
                    help="run one kernel family alone (--steps launches after --warmup) and print its time")
    return ap.parse_args()


def pad_tokens(tokens: int) -> int:
    return max(1, round(37 * tokens / 512))


def block_weights(gen, kind: str) -> dict:
    """Random-init weights of ONE block (Kaiming-uniform linears, LayerNorm 1/0, gate bias 1)."""
    import helpers as H

    if kind == "pairmixer":
        return H.pairmixer_layer_weights(gen, 128, perturbed=False)
    w = {}
    w.update(H.prefixed("tri_mul_out", H.trimul_weights(gen, 128, False)))
    w.update(H.prefixed("tri_mul_in", H.trimul_weights(gen, 128, False)))
    w.update(H.prefixed("tri_att_start", H.triatt_weights(gen, perturbed=False)))
    w.update(H.prefixed("tri_att_end", H.triatt_weights(gen, perturbed=False)))
    w.update(H.prefixed("transition_z", H.transition_weights(gen, 128, 512, True, False)))
    w.update(H.prefixed("attention", H.apb_weights(gen, 384, 128, 16, True, False)))
    w.update(H.prefixed("transition_s", H.transition_weights(gen, 384, 1536, True, False)))
    return w


def workload(tokens: int, blocks: int, kind: str, seed: int = 2):
    """Seeded synthetic trunk input: z, s ~ N(0,1), last 37 tokens padded (scaled for other sizes).  The inputs are
    drawn before the weights and the weights block by block, so neither depends on how many blocks are asked for."""
    import helpers as H

    g = torch.Generator().manual_seed(seed)
    z = torch.randn(1, tokens, tokens, 128, generator=g)
    s = torch.randn(1, tokens, 384, generator=g)
    tok = torch.ones(1, tokens, dtype=torch.bool)
    tok[0, tokens - pad_tokens(tokens):] = False
    w = {}
    for i in range(blocks):
        w.update(H.prefixed(f"layers.{i}", block_weights(g, kind)))
    return w, s, z, tok


def opm_workload():
    """Outer product mean on m[1, 1024, 384, 64] bf16 with a random 10 % of the MSA rows masked, seed 1."""
    import helpers as H

    g = torch.Generator().manual_seed(1)
    w = H.opm_weights(g, perturbed=False)
    m = torch.randn(1, 1024, 384, 64, generator=g).bfloat16()
    rows = torch.rand(1, 1024, generator=g) > 0.1
    mask = rows[:, :, None].expand(1, 1024, 384).contiguous()
    return w, m, mask


def block_flops(N: int, kind: str) -> dict:
    P = float(N) * N
    f = {
        "trimul": 256.0 * N ** 3 + 196608.0 * P,           # one direction
        "transition_z": 393216.0 * P,
        "triatt": 512.0 * N ** 3 + 164864.0 * P,            # one direction
        "apb": 10.0 * N * 384 ** 2 + 2.0 * P * 128 * 16 + 4.0 * P * 384,
        "transition_s": 6.0 * N * 384 * 1536,
    }
    if kind == "pairmixer":
        f["block"] = 2 * f["trimul"] + f["transition_z"]
    else:
        f["block"] = 2 * f["trimul"] + 2 * f["triatt"] + f["transition_z"] + f["apb"] + f["transition_s"]
    return f


def config_dict(args, impl_note: str, parallelism: str) -> dict:
    what = ("triangle multiplication out/in, triangle attention start/end (4x32), pair transition, single-track "
            "pair-bias attention (16x24), single transition" if args.block == "pairformer"
            else "triangle multiplication out/in + pair transition (the reference trunk's own block)")
    if "context parallel" in parallelism:
        launch = "eager launches (NCCL collectives between the kernels)"
    else:
        launch = "eager" if args.no_graph else ("CUDA graph replay of the step (value); trunk.graphed(...) - the public "
                                                "graph-captured call - around pinned-memory copies (e2e)")
    return {
        "workload": f"Pairformer trunk forward, {args.blocks} blocks ({what}), N={args.tokens}, c_z=128, c_s=384, "
                    f"batch 1, last {pad_tokens(args.tokens)} tokens padded, seed 2",
        "block": args.block,
        "tokens": args.tokens,
        "blocks": args.blocks,
        "z_stream": "fp32",
        "arithmetic": "bf16 tensor cores, fp32 accumulate",
        "cache": "inputs larger than L2: z is 134 MB fp32 at N=512 and every kernel streams >=200 MB of scratch",
        "launch": launch,
        "parallelism": parallelism,
        "note": impl_note,
    }


# ----------------------------------------------------------------------------------------- CPU oracle legs
def oracle_block_fn(tokens: int, kind: str, device: str = "cpu"):
    """A closure running ONE block of the trunk (block 0 of the seed-2 workload) with the oracle, on `device`."""
    from oracle import pair_ops as O

    w, s, z, tok = workload(tokens, 1, kind, seed=2)
    w = {k[len("layers.0."):]: v.to(device) for k, v in w.items()}
    s, z, tok = s.to(device), z.to(device), tok.to(device)
    pm = tok[:, :, None] & tok[:, None, :]
    if kind == "pairmixer":
        return lambda: (s, O.pairmixer_layer(z, pm, w))
    return lambda: O.pairformer_block(s, z, tok, w, row_chunk=32)


def time_oracle(fn, reps: int, sync=None):
    """Median of `reps` runs after one warm-up; returns (seconds, last result)."""
    times, out = [], None
    with torch.no_grad():
        for i in range(reps + 1):
            t0 = time.perf_counter()
            out = fn()
            if sync:
                sync()
            if i > 0:
                times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2], out


def run_reference(args) -> None:
    """--impl reference: the CPU port of the reference path on all host cores, each step a bounded sample (one block
    of the trunk at the same N); rank 0 alone runs it."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    fn = oracle_block_fn(args.tokens, args.block)
    steps, warm = max(1, args.steps), max(0, args.warmup)
    with torch.no_grad():
        for _ in range(warm):
            fn()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        dt = (time.perf_counter() - t0) / steps
    fwd = dt * args.blocks
    value = args.tokens ** 2 / fwd
    sample = (f"each step = 1 of the {args.blocks} blocks at N={args.tokens} (fp32 torch on CPU, {dt:.2f} s/block, mean of "
              f"{steps} steps after {warm} warm-up); forward time = {args.blocks} x block time")
    note = "CPU port of the reference modules (oracle/pair_ops.py)"
    if args.block == "pairformer":
        note += "; triangle attention is not in the reference and is timed from the oracle's own statement of it"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": fwd * 1e3, "higher_is_better": True,
        "scaling": "weak" if (args.replicas or args.gpus == 1) else "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(args, note, f"CPU, {cores} threads"),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------- clocks
class ClockSampler:
    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}",
                 "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
                 "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                 "clocks_event_reasons.sw_power_cap", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ----------------------------------------------------------------------------------------- GPU helpers
def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def event_time_ms(fn, iters: int) -> float:
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def attention_core_probe(N: int, dev):
    """Operands of one triangle-attention core launch (N rows x 4 heads x 32) built once; returns a closure that
    launches ``b200_attention_core_fwd`` alone, so the dominant kernel can be timed by itself."""
    import ctypes

    from bioemu2_b200 import _lib

    H, DH = 4, 32
    Nk = (N + 7) // 8 * 8
    g = torch.Generator(device=dev).manual_seed(7)
    qkg = torch.randn(N, N, 384, device=dev, generator=g).bfloat16()
    vT = torch.randn(N, H * DH, Nk, device=dev, generator=g).bfloat16()
    bias = torch.randn(H, N, Nk, device=dev, generator=g).bfloat16()
    mask = torch.ones(N, N, dtype=torch.uint8, device=dev)
    out = torch.empty(N, N, 128, dtype=torch.bfloat16, device=dev)
    a = _lib.AttentionCoreArgs(
        qkg.data_ptr(), 384, N * 384, 0, 128, vT.data_ptr(), Nk, bias.data_ptr(), Nk, 1, N, mask.data_ptr(), 1, N, 1,
        qkg.data_ptr(), N * 384, 384, 256, out.data_ptr(), N * 128, 128, 0, DH, 32, N, H, N)
    keep = (qkg, vT, bias, mask, out)

    def launch():
        _lib.check(_lib.lib.b200_attention_core_fwd(ctypes.byref(a), torch.cuda.current_stream().cuda_stream))

    return launch, keep


def pair_ops_at(N: int, dev, seed: int = 3):
    """The four pair ops of one block (seed-3 weights, full mask) on a fresh z[1, N, N, 128]: the workload of the
    N = 1536 configuration.  Returns (modules, z, mask)."""
    import bioemu2_b200 as b
    import helpers as H

    g = torch.Generator().manual_seed(seed)
    mods = {}
    for name, mode in (("trimul_out", "outgoing"), ("trimul_in", "incoming")):
        m = b.TriangleMultiplication(128, mode).eval()
        m.load_state_dict(H.trimul_weights(g, perturbed=False), strict=True)
        mods[name] = m.to(dev)
    for name, ending in (("triatt_start", False), ("triatt_end", True)):
        m = b.TriangleAttention(ending=ending).eval()
        m.load_state_dict(H.triatt_weights(g, perturbed=False), strict=True)
        mods[name] = m.to(dev)
    gd = torch.Generator(device=dev).manual_seed(seed)
    z = torch.randn(1, N, N, 128, device=dev, generator=gd)
    mask = torch.ones(1, N, N, dtype=torch.uint8, device=dev)
    return mods, z, mask


def run_probe(args) -> None:
    """One kernel family alone, for profiler captures: --warmup launches, then --steps timed ones."""
    import bioemu2_b200 as b

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    N = args.tokens
    with torch.no_grad():
        if args.probe == "attention_core":
            fn, keep = attention_core_probe(N, dev)
        elif args.probe in ("triatt", "trimul"):
            mods, z, mask = pair_ops_at(N, dev)
            key = "triatt_start" if args.probe == "triatt" else "trimul_out"
            fn = lambda: mods[key].forward_residual_(z, mask)  # noqa: E731
        elif args.probe == "transition":
            w, s, z, tok = workload(N, 1, "pairformer")
            blk = b.PairformerBlock().eval()
            blk.load_state_dict({k[len("layers.0."):]: v for k, v in w.items()}, strict=True)
            blk.to(dev)
            zd = z.to(dev)
            fn = lambda: blk.transition_z.forward_residual_(zd)  # noqa: E731
        elif args.probe == "apb":
            w, s, z, tok = workload(N, 1, "pairformer")
            blk = b.PairformerBlock().eval()
            blk.load_state_dict({k[len("layers.0."):]: v for k, v in w.items()}, strict=True)
            blk.to(dev)
            sd, zd, td = s.to(dev), z.to(dev), tok.to(dev)
            fn = lambda: blk.attention(sd, zd, td)  # noqa: E731
        elif args.probe == "trunk_glue":
            return run_trunk_glue_probe(args, dev)
        elif args.probe == "window_attention":
            return run_window_attention_probe(args, dev)
        else:
            w, m, mask = opm_workload()
            mod = b.OuterProductMean(64, 32, 128).eval()
            mod.load_state_dict(w, strict=True)
            mod.to(dev)
            md, kd = m.to(dev), mask.to(dev)
            fn = lambda: mod(md, kd)  # noqa: E731
        for _ in range(args.warmup):
            fn()
        ms = event_time_ms(fn, args.steps)
        status = b._lib.device_status()
    print(json.dumps({"probe": args.probe, "tokens": N, "ms_per_call": ms, "device_status": status}), flush=True)


def run_trunk_glue_probe(args, dev, emit: bool = True) -> dict:
    """The HBM-bound glue around the trunk blocks at --tokens: pair initialisation, the recycling update and pairwise
    conditioning, each timed alone with its algorithmic bytes (fp32 pair tensor, 512 B per pair)."""
    import bioemu2_b200 as b
    from bioemu2_b200 import functional as F

    N = args.tokens
    g = torch.Generator().manual_seed(6)
    pair_bytes = N * N * 128 * 4
    emb = b.PairMixerSequenceEmbedder(384, 128, 456, msa_blocks=0, num_blocks=0, use_unconditional_branch=True).eval().to(dev)
    cond = b.PairwiseConditioning(128, 128).eval().to(dev)
    s_inputs = torch.randn(1, N, 456, generator=g).to(dev)
    z = torch.randn(1, N, N, 128, generator=g).to(dev)
    rel = torch.randn(1, N, N, 128, generator=g).to(dev)
    feats = {"pair_init_terms": rel}
    a, c = torch.randn(1, N, 128, generator=g).to(dev), torch.randn(1, N, 128, generator=g).to(dev)
    z_init = emb.initial_embeddings(s_inputs, feats)[1]
    legs = {
        # min_bytes: the fp32 pair tensors (N*N*512 B each) a fully fused form would have to move - inputs read once,
        # the result written once, no intermediate.  The legs that are several kernels move more than this.
        "pair_outer_sum": (lambda: F.pair_outer_sum(a, c, rel), 2 * pair_bytes),                      # terms in, z_init out
        "initial_embeddings": (lambda: emb.initial_embeddings(s_inputs, feats), 2 * pair_bytes),
        "recycle_update_z": (lambda: emb._recycle(z, z_init, emb.z_norm, "z_recycle"), 3 * pair_bytes),  # z, z_init in
        "unconditional_branch": (lambda: emb(s_inputs, feats, unconditional=True), 4 * pair_bytes),  # + z_init round trip
        "pairwise_conditioning": (lambda: cond(z, rel), 3 * pair_bytes),                            # z, rel in; z out
    }
    peak = peaks()
    out = {"probe": "trunk_glue", "tokens": N, "hbm_peak_gbs": peak["hbm_gbs"], "legs": {}}
    for name, (fn, nbytes) in legs.items():
        for _ in range(args.warmup):
            fn()
        ms = event_time_ms(fn, args.steps)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out["legs"][name] = {"ms": ms, "min_bytes": nbytes, "gbs": gbs, "frac_of_hbm_peak": gbs / peak["hbm_gbs"]}
    out["device_status"] = b._lib.device_status()
    if emit:
        print(json.dumps(out), flush=True)
    return out


def run_window_attention_probe(args, dev, emit: bool = True) -> dict:
    """The atom transformer's sliding-window attention at 8 atoms per token of --tokens (windows of 32 queries, 128
    keys, 4 heads of 32, pair width 16), 8 samples sharing one pair tensor: the whole module and its two kernels."""
    import bioemu2_b200 as b
    from bioemu2_b200 import functional as F

    NW, W, Hk, c_s, c_z, heads, M = args.tokens * 8 // 32, 32, 128, 128, 16, 4, 8
    g = torch.Generator().manual_seed(7)
    mod = b.AttentionPairBiasSlidingWindow(c_s, c_z, heads).eval().to(dev)
    s = torch.randn(M * NW, W, c_s, generator=g).to(dev)
    z = torch.randn(1, NW, W, Hk, c_z, generator=g).to(dev)
    mask = torch.ones(NW, W, dtype=torch.bool, device=dev)
    w = mod.packed()
    sn = F.rows_to_bf16(s, w.ln_s_w, w.ln_s_b)
    qkv, gate = F.linear_bf16(sn, w.w_qkv, bias_f32=w.b_qkv), F.linear_bf16(sn, w.w_g)
    bias = torch.empty(1, NW, heads, W, Hk, dtype=torch.float32, device=dev)
    og = torch.empty(M * NW, W, c_s, dtype=torch.bfloat16, device=dev)
    m8 = mask.to(torch.uint8)
    lib = b._lib.lib
    st = torch.cuda.current_stream().cuda_stream
    legs = {
        "module": lambda: mod(s, z, mask, multiplicity=M),
        "window_bias_kernel": lambda: lib.b200_window_bias_fwd(z.data_ptr(), w.ln_z_w.data_ptr(), None, w.w_z.data_ptr(),
                                                               bias.data_ptr(), NW, W, Hk, c_z, heads, 0, st),
        "window_attention_kernel": lambda: lib.b200_window_attention_fwd(qkv.data_ptr(), gate.data_ptr(), bias.data_ptr(),
                                                                         m8.data_ptr(), og.data_ptr(), 1, M, NW, W, Hk,
                                                                         heads, c_s // heads, st),
    }
    peak = peaks()
    z_bytes, bias_bytes = z.numel() * 4, bias.numel() * 4
    flops = M * NW * heads * W * Hk * (c_s // heads) * 4
    out = {"probe": "window_attention", "atoms": NW * W, "samples": M, "legs": {}}
    for name, fn in legs.items():
        for _ in range(args.warmup):
            fn()
        out["legs"][name] = {"ms": event_time_ms(fn, args.steps)}
    kb = out["legs"]["window_bias_kernel"]
    kb["bytes"] = z_bytes + bias_bytes
    kb["frac_of_hbm_peak"] = kb["bytes"] / (kb["ms"] * 1e-3) / 1e9 / peak["hbm_gbs"]
    ka = out["legs"]["window_attention_kernel"]
    ka["fp32_tflops"] = flops / (ka["ms"] * 1e-3) / 1e12
    ka["bytes"] = qkv.numel() * 2 + gate.numel() * 2 + og.numel() * 2 + M * bias_bytes
    out["device_status"] = b._lib.device_status()
    if emit:
        print(json.dumps(out), flush=True)
    return out


def parity_stats(actual: torch.Tensor, expected: torch.Tensor) -> dict:
    a, e = actual.detach().double().cpu(), expected.detach().double().cpu()
    d = (a - e).abs()
    return {"rel_max": float(d.max() / e.abs().max().clamp_min(1e-30)),
            "elementwise_ok": bool((d <= 2e-2 + 2e-2 * e.abs()).all()), "nan": bool(torch.isnan(a).any())}


# ----------------------------------------------------------------------------------------- 1 GPU (or replicas)
def run_b200(args) -> None:
    import torch.distributed as dist

    import bioemu2_b200 as b

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    composite = args.block == "pairformer"
    w, s_host, z_host, tok = workload(args.tokens, args.blocks, args.block, seed=2 + rank)
    trunk = (b.PairformerModule(384, 128, args.blocks) if composite else b.PairMixerModule(384, 128, args.blocks)).eval()
    trunk.load_state_dict(w, strict=True)
    trunk.to(dev)
    del w
    N = args.tokens
    cells = N * N
    pair_mask = tok[:, :, None] & tok[:, None, :]
    z_pinned, s_pinned = z_host.pin_memory(), s_host.pin_memory()
    tok_pinned, pm_pinned = tok.pin_memory(), pair_mask.pin_memory()
    z_out_pinned, s_out_pinned = torch.empty_like(z_host).pin_memory(), torch.empty_like(s_host).pin_memory()
    z_dev, s_dev, tok_dev = z_host.to(dev), s_host.to(dev), tok.to(dev)
    z_work, s_work = torch.empty_like(z_dev), torch.empty_like(s_dev)
    mask8 = pair_mask.to(dev).to(torch.uint8)

    def step_resident():
        # restore the inputs (the trunk loop updates z and s in place): two copies, ~0.05 ms of the step
        z_work.copy_(z_dev)
        s_work.copy_(s_dev)
        if composite:
            trunk.forward_(s_work, z_work, tok_dev, mask8)
        else:
            for layer in trunk.layers:
                layer.forward_(z_work, mask8)

    def step_e2e():
        zd = z_pinned.to(dev, non_blocking=True)
        sd = s_pinned.to(dev, non_blocking=True)
        if composite:
            s_out, z_out = trunk(sd, zd, tok_pinned.to(dev, non_blocking=True))
        else:
            s_out, z_out = trunk(sd, zd, pm_pinned.to(dev, non_blocking=True))
        z_out_pinned.copy_(z_out, non_blocking=True)
        s_out_pinned.copy_(s_out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        n0 = b._lib.launch_count()
        step_resident()
        launches_per_step = b._lib.launch_count() - n0
        for _ in range(max(args.warmup, 3) - 1):
            step_resident()
        barrier()
        timed_step = step_resident
        graphed = False
        if not args.no_graph:
            # The step is a fixed sequence of ~1200 launches on fixed buffers: capture it once, replay it per step.
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    step_resident()
                graph.replay()
                torch.cuda.synchronize()
                timed_step, graphed = graph.replay, True
            except Exception as exc:  # keep the eager path if capture is refused
                print(f"CUDA graph capture failed ({exc}); timing eager launches", file=sys.stderr)
                torch.cuda.synchronize()
        for _ in range(3 if graphed else 0):
            timed_step()
        barrier()
        ms = event_time_ms(timed_step, args.steps)
        barrier()

        e2e_step, e2e_graphed = step_e2e, False
        if not args.no_graph:
            # the public form of the same idea: trunk.graphed(...) captures the block loop once; a call copies the
            # inputs in (here from pinned host memory), replays, and returns static output buffers
            try:
                g_trunk = trunk.graphed(s_dev, z_dev, tok_dev if composite else pair_mask.to(dev))
                mask_pin = tok_pinned if composite else pm_pinned

                def step_e2e_graphed():
                    s_out, z_out = g_trunk(s_pinned, z_pinned, mask_pin)
                    z_out_pinned.copy_(z_out, non_blocking=True)
                    s_out_pinned.copy_(s_out, non_blocking=True)
                    torch.cuda.current_stream().synchronize()

                e2e_step, e2e_graphed = step_e2e_graphed, True
            except Exception as exc:
                print(f"trunk.graphed failed ({exc}); end-to-end step stays eager", file=sys.stderr)
                torch.cuda.synchronize()
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        barrier()
        e2e_eager_ms = None
        if e2e_graphed:
            step_e2e()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(max(args.steps // 2, 2)):
                step_e2e()
            torch.cuda.synchronize()
            e2e_eager_ms = (time.perf_counter() - t0) * 1e3 / max(args.steps // 2, 2)
            del g_trunk
        clocks = sampler.stop() if rank == 0 else None

        # per-op timings on the same data (inputs > L2), for the rooflines
        L0 = trunk.layers[0]
        zt, st = z_dev.clone(), s_dev.clone()
        it = max(args.steps, 5) * 4
        t = {}
        t["transition_z"] = event_time_ms(lambda: L0.transition_z.forward_residual_(zt), it)
        zt.copy_(z_dev)
        t["trimul_out"] = event_time_ms(lambda: L0.tri_mul_out.forward_residual_(zt, mask8), it)
        zt.copy_(z_dev)
        t["trimul_in"] = event_time_ms(lambda: L0.tri_mul_in.forward_residual_(zt, mask8), it)
        if composite:
            zt.copy_(z_dev)
            t["triatt_start"] = event_time_ms(lambda: L0.tri_att_start.forward_residual_(zt, mask8), it)
            zt.copy_(z_dev)
            t["triatt_end"] = event_time_ms(lambda: L0.tri_att_end.forward_residual_(zt, mask8), it)
            zt.copy_(z_dev)
            t["apb"] = event_time_ms(lambda: L0.attention(st, zt, tok_dev), it)
            t["transition_s"] = event_time_ms(lambda: L0.transition_s.forward_residual_(st), it)
            core, keep = attention_core_probe(N, dev)
            t["attention_core"] = event_time_ms(core, it)
            del keep
        # block 0 of the trunk on the bench's own inputs, kept for the parity check against the oracle below
        if composite:
            s_blk, z_blk = L0(s_dev, z_dev, tok_dev)
        else:
            s_blk, z_blk = L0(s_dev, z_dev, mask8)
        s_blk, z_blk = s_blk.cpu(), z_blk.cpu()
        del zt, st
        extras = {}
        if rank == 0 and world == 1 and not args.no_extras:
            extras = extra_ops(args, dev, b)
        status = b._lib.device_status()

    if world > 1:
        tt = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(tt[0]), float(tt[1])

    if rank == 0:
        pk = peaks()
        P = float(cells)
        fl = block_flops(N, args.block)
        tf = lambda flops, t_ms: flops / (t_ms * 1e-3) / 1e12  # noqa: E731
        ops = {k + "_ms": v for k, v in t.items()}
        ops["transition_z_tflops"] = tf(fl["transition_z"], t["transition_z"])
        ops["transition_z_frac_of_bf16_burst"] = ops["transition_z_tflops"] / pk["bf16_tflops"]
        t_tm = 0.5 * (t["trimul_out"] + t["trimul_in"])
        ops["trimul_tflops"] = tf(fl["trimul"], t_tm)
        ops["trimul_hbm_gbs"] = 3072.0 * P / (t_tm * 1e-3) / 1e9
        ops["trimul_frac_of_hbm"] = ops["trimul_hbm_gbs"] / pk["hbm_gbs"]
        ops["trunk_tflops"] = tf(args.blocks * fl["block"], ms)
        ops.update(extras.get("ops", {}))
        if composite:
            core_flops = 4.0 * N ** 3 * 128
            ach = tf(core_flops, t["attention_core"])
            ex2_floor_ms = (float(N) ** 3 * 4) / (16.0 * 148 * (clocks["sm_mhz"] or 1965) * 1e6) * 1e3 if clocks else None
            # q, k, g (N^2 x 384 bf16), V^T (N^2 x 128 bf16) read once, the gated output (N^2 x 128 bf16) written once,
            # the 4-head bias (4 N^2 bf16) read from L2
            core_bytes = P * (384 + 128 + 128) * 2 + 4 * P * 2
            roofline = {
                "kernel": "flash_core_kernel<32,2> (triangle-attention core: QK^T + bias tile + online softmax + PV), "
                          "launched alone on N rows x 4 heads x 32",
                "bound": "tensor", "achieved": ach, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                "frac": ach / pk["bf16_tflops"], "peak_source": pk["source"] + " burst (kernel timed alone)",
                "algorithmic_flops_per_launch": core_flops, "algorithmic_bytes_per_launch": core_bytes,
                "ms_per_launch": t["attention_core"],
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch at N=512 (ncu capture summarised in
                # profiles/flash_core_triatt_n512.md); the operands scale with N^2, so other sizes are scaled from it
                "traffic": 323.3e6 * (N / 512.0) ** 2,
                "traffic_source": "ncu capture at N=512 (270.8 MB read + 52.5 MB written), scaled by (N/512)^2; the "
                                  "algorithmic bytes of the launch are 337.6 MB at N=512 (four 67.1 MB operands read, one "
                                  "67.1 MB result written, 2.1 MB of bias), so the kernel moves no byte twice",
                "note": "head dim 32 makes the core ex2-bound, not tensor-bound: N^3*4 exponentials at 16/clk/SM "
                        f"take {ex2_floor_ms:.3f} ms at the sampled clock; the tensor work alone would take "
                        f"{core_flops / (pk['bf16_tflops'] * 1e12) * 1e3:.3f} ms" if ex2_floor_ms else "",
            }
        else:
            roofline = {
                "kernel": "transition_kernel<fp32 stream> (fused LN + fc1|fc2 + SwiGLU + fc3 + residual)",
                "bound": "tensor", "achieved": ops["transition_z_tflops"], "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                "frac": ops["transition_z_frac_of_bf16_burst"], "peak_source": pk["source"] + " burst (kernel timed alone)",
                "algorithmic_flops_per_launch": fl["transition_z"], "ms_per_launch": t["transition_z"], "traffic": None,
            }
        h2d = z_host.numel() * 4 + s_host.numel() * 4 + (tok.numel() if composite else pair_mask.numel())
        par = f"{world} independent replicas (weak scaling, no data-path collective)" if world > 1 else "single GPU"
        line = {
            "metric": METRIC, "value": world * cells / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(args, "hand-written sm_100a kernels through the C ABI (libb200pair.so)", par),
            "clocks": clocks,
            "e2e": {"value": world * cells / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": z_host.numel() * 4 + s_host.numel() * 4,
                    "call": "trunk.graphed(s, z, mask)(s_pinned, z_pinned, mask_pinned)" if e2e_graphed
                            else "trunk(s, z, mask) (eager launches)",
                    "ms_per_step_eager_forward": e2e_eager_ms},
            "gpu_launches": int(args.steps * launches_per_step),
            "gpu_launches_per_step": int(launches_per_step),
            "roofline": roofline, "ops": ops, "device_status": status,
        }
        for k in ("torch_gpu_baseline", "larger_sizes", "trunk_glue", "atom_window_attention"):
            if k in extras:
                line[k] = extras[k]
        if not args.no_cpu_baseline and world == 1:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            t_block, (s_ref, z_ref) = time_oracle(oracle_block_fn(N, args.block), 3)
            line["cpu_baseline"] = {
                "value": cells / (t_block * args.blocks), "unit": UNIT, "cores": cores, "kind": "port",
                "sample": f"1 of {args.blocks} blocks at N={N}, median of 3 after 1 warm-up ({t_block:.2f} s/block), "
                          f"forward = {args.blocks} x block",
            }
            pz, ps = parity_stats(z_blk, z_ref), parity_stats(s_blk, s_ref)
            line["parity"] = {
                "what": f"block 0 of the trunk on the bench inputs (N={N}, all cells) against the fp32 CPU oracle",
                "rel_max": max(pz["rel_max"], ps["rel_max"]), "rel_max_z": pz["rel_max"], "rel_max_s": ps["rel_max"],
                "elementwise_ok": pz["elementwise_ok"] and ps["elementwise_ok"] and not (pz["nan"] or ps["nan"]),
                "bar": "|d| <= 2e-2 + 2e-2 |ref| for every element, and rel_max <= 2e-2",
            }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def extra_ops(args, dev, b) -> dict:
    """The legs of the 1-GPU run outside the headline: outer product mean (1024 x 384 MSA), the N = 1536 pair ops, a
    two-block trunk at N = 1536 and a one-block trunk at N = 3072 (scaled to 48 blocks, stated as such), and the
    oracle's torch code on this GPU under bf16 autocast as the same-box GPU baseline."""
    out = {"ops": {}}
    ops = out["ops"]
    pk = peaks()
    # outer product mean
    w, m, mask = opm_workload()
    mod = b.OuterProductMean(64, 32, 128).eval()
    mod.load_state_dict(w, strict=True)
    mod.to(dev)
    md, kd = m.to(dev), mask.to(dev)
    mod(md, kd)
    ops["opm_c1_ms"] = event_time_ms(lambda: mod(md, kd), 20)
    opm_flops = 2.0 * 1024 * 384 ** 2 * 32 ** 2 + 2.0 * 384 ** 2 * 1024 * 128 + 2.0 * 1024 * 384 * 64 * 64
    ops["opm_c1_tflops"] = opm_flops / (ops["opm_c1_ms"] * 1e-3) / 1e12
    ops["opm_c1_frac_of_bf16_burst"] = ops["opm_c1_tflops"] / pk["bf16_tflops"]
    del mod, md, kd
    # N = 1536 pair ops (one block's triangle multiplication out/in + triangle attention start/end)
    mods, z, mask = pair_ops_at(1536, dev)
    z0 = z.clone()
    for k in ("trimul_out", "trimul_in", "triatt_start", "triatt_end"):
        z.copy_(z0)
        mods[k].forward_residual_(z, mask)
        ops[k + "_n1536_ms"] = event_time_ms(lambda: mods[k].forward_residual_(z, mask), 5)

    def config3():
        z.copy_(z0)
        for k in ("trimul_out", "trimul_in", "triatt_start", "triatt_end"):
            mods[k].forward_residual_(z, mask)

    ops["config3_n1536_ms"] = event_time_ms(config3, 5)
    del mods, z, z0, mask
    torch.cuda.empty_cache()
    # larger trunks, fewer blocks
    larger = {}
    for n_tok, n_blk in ((1536, 2), (3072, 1)):
        wl, s, zz, tok = workload(n_tok, n_blk, args.block, seed=2)
        trunk = (b.PairformerModule(384, 128, n_blk) if args.block == "pairformer" else b.PairMixerModule(384, 128, n_blk)).eval()
        trunk.load_state_dict(wl, strict=True)
        trunk.to(dev)
        sd, zd, td = s.to(dev), zz.to(dev), tok.to(dev)
        pm8 = (td[:, :, None] & td[:, None, :]).to(torch.uint8)
        zw, sw = torch.empty_like(zd), torch.empty_like(sd)

        def step():
            zw.copy_(zd)
            sw.copy_(sd)
            for layer in trunk.layers:
                if args.block == "pairformer":
                    layer.forward_(sw, zw, td, pm8)
                else:
                    layer.forward_(zw, pm8)

        step()
        ms = event_time_ms(step, 3)
        larger[f"N{n_tok}"] = {
            "blocks_timed": n_blk, "ms_per_block": ms / n_blk, "ms_per_forward_48_blocks_extrapolated": ms / n_blk * 48,
            "pair_cells_per_s_extrapolated": n_tok ** 2 / (ms / n_blk * 48 * 1e-3),
            "trunk_tflops": block_flops(n_tok, args.block)["block"] * n_blk / (ms * 1e-3) / 1e12,
        }
        del trunk, sd, zd, td, pm8, zw, sw
        b.functional.release_workspaces()
        torch.cuda.empty_cache()
    out["larger_sizes"] = larger
    # the glue around the trunk blocks and the atom transformer's window attention (the rows after the trunk itself)
    try:
        import types

        pa = types.SimpleNamespace(tokens=args.tokens, steps=10, warmup=3)
        out["trunk_glue"] = run_trunk_glue_probe(pa, dev, emit=False)["legs"]
        torch.cuda.empty_cache()
        wa = run_window_attention_probe(pa, dev, emit=False)
        out["atom_window_attention"] = {"atoms": wa["atoms"], "samples": wa["samples"], **wa["legs"]}
    except Exception as exc:  # must not cost the headline
        out["trunk_glue"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    torch.cuda.empty_cache()
    # the oracle's plain torch code on this GPU under bf16 autocast (cuBLAS / eager kernels)
    try:
        fn = oracle_block_fn(args.tokens, args.block, device=str(dev))

        def run():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                return fn()

        t_blk, _ = time_oracle(run, 3, sync=torch.cuda.synchronize)
        out["torch_gpu_baseline"] = {
            "what": "the oracle's un-fused torch code (the reference's `full`/`vanilla`/einsum formulation) on this GPU "
                    "under torch.autocast(bfloat16): cuBLAS and eager kernels, one block, outside the timed region",
            "ms_per_block": t_blk * 1e3, "ms_per_forward_extrapolated": t_blk * 1e3 * args.blocks,
            "value": args.tokens ** 2 / (t_blk * args.blocks), "unit": UNIT,
        }
    except Exception as exc:  # an out-of-memory or missing kernel here must not cost the headline
        out["torch_gpu_baseline"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------------------- context parallel
def run_cp(args) -> None:
    """ONE pair tensor tiled over an R x C grid of the ranks (strong scaling): the same 48-block trunk on the same
    seeded inputs as the 1-GPU run, every rank holding its block of z and its rows of s."""
    import torch.distributed as dist

    import bioemu2_b200 as b
    from bioemu2_b200.context_parallel import (CPGrid, CPPairformerModule, CPPairMixerModule, CPTriangleAttention,
                                               CPTriangleMultiplication, kernel_shard_multiple)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    rows, cols = (int(v) for v in args.cp.lower().split("x")) if args.cp else GRIDS.get(world, (1, world))
    if rows * cols != world:
        raise SystemExit(f"grid {rows}x{cols} needs {rows * cols} ranks, got {world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    N = args.tokens
    mult = kernel_shard_multiple(rows, cols)
    if N % mult:
        raise SystemExit(f"--tokens must be a multiple of {mult} for a {rows}x{cols} grid")
    grid = CPGrid(rows, cols)
    composite = args.block == "pairformer"

    def shard_inputs(s, z, tok):
        n = z.shape[1]
        (r0, r1), (c0, c1) = grid.coords.my_rows(n), grid.coords.my_cols(n)
        return s[:, r0:r1].contiguous(), z[:, r0:r1, c0:c1].contiguous(), tok[:, r0:r1].contiguous(), tok[:, c0:c1].contiguous()

    def build(n_tok, n_blk, seed):
        w, s, z, tok = workload(n_tok, n_blk, args.block, seed=seed)  # same seed on every rank: replicated weights
        serial = (b.PairformerModule(384, 128, n_blk) if composite else b.PairMixerModule(384, 128, n_blk)).eval()
        serial.load_state_dict(w, strict=True)
        serial.to(dev)
        cp = CPPairformerModule(serial, grid) if composite else CPPairMixerModule(serial, grid)
        return serial, cp, s, z, tok

    def run_sharded(cp, s_blk, z_blk, tr, tc):
        if composite:
            return cp.forward_(s_blk, z_blk, tr, tc)
        pm = (tr[:, :, None] & tc[:, None, :]).to(torch.uint8)
        return s_blk, cp(z_blk, pm)

    with torch.no_grad():
        # -- correctness first: two blocks at N = 256, sharded against the single-GPU modules, on every rank
        serial, cp, s, z, tok = build(256, 2, seed=5)
        s_l, z_l, tr, tc = (t.to(dev) for t in shard_inputs(s, z, tok))
        s_cp, z_cp = run_sharded(cp, s_l.clone(), z_l.clone(), tr, tc)
        td = tok.to(dev)
        if composite:
            s_ref, z_ref = serial(s.to(dev), z.to(dev), td)
        else:
            s_ref, z_ref = serial(s.to(dev), z.to(dev), (td[:, :, None] & td[:, None, :]))
        s_ref_l, z_ref_l, _, _ = shard_inputs(s_ref, z_ref, td)
        rel = max(float((z_cp - z_ref_l).abs().max() / z_ref.abs().max()),
                  float((s_cp - s_ref_l).abs().max() / s_ref.abs().max()))
        rel_t = torch.tensor([rel], device=dev, dtype=torch.float64)
        dist.all_reduce(rel_t, op=dist.ReduceOp.MAX)
        cp_parity_rel = float(rel_t[0])
        del serial, cp, s_cp, z_cp, s_ref, z_ref
        torch.cuda.empty_cache()

        # -- the headline workload, sharded
        serial, cp, s, z, tok = build(N, args.blocks, seed=2)
        s_h, z_h, tr_h, tc_h = shard_inputs(s, z, tok)
        s_pin, z_pin = s_h.pin_memory(), z_h.pin_memory()
        s_out_pin, z_out_pin = torch.empty_like(s_h).pin_memory(), torch.empty_like(z_h).pin_memory()
        s_d, z_d, tr, tc = s_h.to(dev), z_h.to(dev), tr_h.to(dev), tc_h.to(dev)
        s_w, z_w = torch.empty_like(s_d), torch.empty_like(z_d)

        def step_resident():
            s_w.copy_(s_d)
            z_w.copy_(z_d)
            run_sharded(cp, s_w, z_w, tr, tc)

        def step_e2e():
            sd = s_pin.to(dev, non_blocking=True)
            zd = z_pin.to(dev, non_blocking=True)
            so, zo = run_sharded(cp, sd, zd, tr, tc)
            s_out_pin.copy_(so, non_blocking=True)
            z_out_pin.copy_(zo, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        def barrier():
            dist.barrier()
            torch.cuda.synchronize()

        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        n0 = b._lib.launch_count()
        step_resident()
        launches_per_step = b._lib.launch_count() - n0
        for _ in range(max(args.warmup, 3) - 1):
            step_resident()
        barrier()
        ms = event_time_ms(step_resident, args.steps)
        barrier()
        step_e2e()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step_e2e()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        del serial, cp, s_d, z_d, s_w, z_w
        torch.cuda.empty_cache()

        # -- triangle multiplication out/in + triangle attention start/end at N = 1536, full mask, seed 3
        n3 = 1536
        cfg3 = None
        if composite and n3 % mult == 0:
            mods, _, _ = pair_ops_at(8, dev)  # weights only (seed 3, same on every rank); z is built per block below
            ops3 = [CPTriangleMultiplication(mods["trimul_out"], grid), CPTriangleMultiplication(mods["trimul_in"], grid),
                    CPTriangleAttention(mods["triatt_start"], grid), CPTriangleAttention(mods["triatt_end"], grid)]
            (r0, r1), (c0, c1) = grid.coords.my_rows(n3), grid.coords.my_cols(n3)
            gd = torch.Generator(device=dev).manual_seed(300 + rank)
            z3 = torch.randn(1, r1 - r0, c1 - c0, 128, device=dev, generator=gd)
            z3w = torch.empty_like(z3)
            m3 = torch.ones(1, r1 - r0, c1 - c0, dtype=torch.uint8, device=dev)

            def step3():
                z3w.copy_(z3)
                for op in ops3:
                    op(z3w, m3)

            step3()
            step3()
            barrier()
            ms3 = event_time_ms(step3, 5)
            barrier()
            t3 = torch.tensor([ms3], device=dev, dtype=torch.float64)
            dist.all_reduce(t3, op=dist.ReduceOp.MAX)
            cfg3 = {"grid": f"{rows}x{cols}", "tokens": n3, "ms": float(t3[0]),
                    "what": "triangle multiplication out/in + triangle attention start/end, one block, full mask, seed 3"}
        status = b._lib.device_status()

    tt = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(tt[0]), float(tt[1])
    st = torch.tensor([status], device=dev, dtype=torch.int64)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    if rank == 0:
        fl = block_flops(N, args.block)
        per_rank_in = s_h.numel() * 4 + z_h.numel() * 4
        line = {
            "metric": METRIC, "value": N * N / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(args, "hand-written sm_100a kernels through the C ABI (libb200pair.so); NCCL collectives "
                                        "over the grid's row and column groups, eager launches",
                                  f"context parallel: one pair tensor tiled {rows}x{cols} "
                                  f"(block {z_h.shape[1]}x{z_h.shape[2]}), single track row-sharded"),
            "clocks": clocks,
            "e2e": {"value": N * N / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": world * per_rank_in, "d2h_bytes_per_step": world * per_rank_in},
            "gpu_launches": int(args.steps * launches_per_step), "gpu_launches_per_step": int(launches_per_step),
            "cp_parity_rel": cp_parity_rel,
            "cp_parity": "2 blocks at N=256 (seed 5, 18 tokens padded): sharded result against the single-GPU modules "
                         "on the same inputs, max over ranks of max|d| / max|ref| over every cell",
            "cp_config3": cfg3,
            "ops": {"trunk_tflops_aggregate": args.blocks * fl["block"] / (ms * 1e-3) / 1e12},
            "device_status": int(st[0]),
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def run_config4(args) -> None:
    """Context-parallel trunk at N = 3072 plus the 24 token blocks of the diffusion module on the same grid.

    Inputs: three chains of N/3 tokens, the last 5-15 % of each chain masked (fractions drawn from the seed-4
    generator), z and s ~ N(0,1); every rank draws its own block of z on the device (seed 400 + rank) -- at this size
    nothing is compared with the CPU oracle, the sharded arithmetic is the one `cp_parity_rel` checks at N = 256.
    Weights: seed 4, identical on all ranks."""
    import math

    import torch.distributed as dist

    import bioemu2_b200 as b
    from bioemu2_b200.context_parallel import (CPConditionedTransformerLayer, CPGrid, CPPairformerModule,
                                               kernel_shard_multiple)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    rows, cols = (int(v) for v in args.cp.lower().split("x")) if args.cp else GRIDS.get(world, (1, world))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29512")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    N = args.tokens if args.tokens != 512 else 3072
    n_blocks, n_token_layers, width = args.blocks, 24, 768
    mult = math.lcm(kernel_shard_multiple(rows, cols), 3)
    if N % mult:
        raise SystemExit(f"--tokens must be a multiple of {mult} for a {rows}x{cols} grid and three chains")
    grid = CPGrid(rows, cols)
    g4 = torch.Generator().manual_seed(4)
    fracs = (0.05 + 0.10 * torch.rand(3, generator=g4)).tolist()
    chain = N // 3
    tok = torch.ones(1, N, dtype=torch.bool)
    for i, f in enumerate(fracs):
        tok[0, (i + 1) * chain - int(round(f * chain)):(i + 1) * chain] = False
    import helpers as H

    w = {}
    for i in range(n_blocks):
        w.update(H.prefixed(f"layers.{i}", block_weights(g4, "pairformer")))
    serial = b.PairformerModule(384, 128, n_blocks).eval()
    serial.load_state_dict(w, strict=True)
    serial.to(dev)
    del w
    trunk = CPPairformerModule(serial, grid)
    (r0, r1), (c0, c1) = grid.coords.my_rows(N), grid.coords.my_cols(N)
    gd = torch.Generator(device=dev).manual_seed(400 + rank)
    z0 = torch.randn(1, r1 - r0, c1 - c0, 128, device=dev, generator=gd)
    gs = torch.Generator(device=dev).manual_seed(40 + grid.coords.r)   # s rows are replicated over grid columns
    s0 = torch.randn(1, r1 - r0, 384, device=dev, generator=gs)
    tr, tc = tok[:, r0:r1].to(dev), tok[:, c0:c1].to(dev)
    z, s = torch.empty_like(z0), torch.empty_like(s0)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def trunk_step():
        z.copy_(z0)
        s.copy_(s0)
        trunk.forward_(s, z, tr, tc)

    steps = max(1, min(args.steps, 3))
    with torch.no_grad():
        trunk_step()
        barrier()
        trunk_ms = event_time_ms(trunk_step, steps)
        barrier()
        # ---- 24 token blocks on the trunk's pair tensor (static for the whole denoising loop)
        torch.manual_seed(4)
        layers = []
        for l in range(n_token_layers):
            m = b.ConditionedTransformerLayer(dim=width, dim_pairwise=128, dim_cond=width, heads=16,
                                              transition_hidden=4 * width, lns_scale=1.0 / math.sqrt(l + 1)).eval().to(dev)
            layers.append(CPConditionedTransformerLayer(m, grid))
        ga = torch.Generator(device=dev).manual_seed(44 + grid.coords.r)
        a0 = torch.randn(1, r1 - r0, width, device=dev, generator=ga)
        c0_ = torch.randn(1, r1 - r0, width, device=dev, generator=ga)

        def denoise_step():
            a = a0
            for layer in layers:
                a = layer(a, z, c0_, tr, 1)
            return a

        denoise_step()
        barrier()
        per_layer_ms = event_time_ms(denoise_step, steps)
        barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for layer in layers:
            layer.attention.prepare_static(z)
        t1.record()
        torch.cuda.synchronize()
        prepare_ms = t0.elapsed_time(t1)
        denoise_step()
        barrier()
        hoisted_ms = event_time_ms(denoise_step, steps)
        barrier()
        status = b._lib.device_status()
    tt = torch.tensor([trunk_ms, per_layer_ms, hoisted_ms, prepare_ms, float(status)], device=dev, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    trunk_ms, per_layer_ms, hoisted_ms, prepare_ms, status = (float(v) for v in tt)
    if rank == 0:
        fl = block_flops(N, "pairformer")
        line = {
            "metric": METRIC, "value": N * N / (trunk_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": 1, "ms_per_step": trunk_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"context-parallel Pairformer trunk, {n_blocks} blocks, N={N} (three chains of {chain}, "
                                   f"last {', '.join(f'{100 * f:.1f}%' for f in fracs)} of the chains padded), seed 4, pair tensor tiled "
                                   f"{rows}x{cols}; then {n_token_layers} diffusion token blocks (16 heads, width {width}, pair bias "
                                   "from the trunk's pair tensor)",
                       "tokens": N, "blocks": n_blocks, "grid": f"{rows}x{cols}", "z_stream": "fp32",
                       "arithmetic": "bf16 tensor cores, fp32 accumulate", "launch": "eager"},
            "ops": {"trunk_tflops_aggregate": n_blocks * fl["block"] / (trunk_ms * 1e-3) / 1e12},
            "diffusion_token_blocks": {
                "layers": n_token_layers,
                "ms_per_denoise_step_bias_per_layer": per_layer_ms,
                "ms_per_denoise_step_bias_hoisted": hoisted_ms,
                "ms_one_time_bias_for_all_layers": prepare_ms,
                "note": "per_layer: every layer projects and all-gathers its pair bias on every step, as the reference does; "
                        "hoisted: the static pair tensor is projected once per context (prepare_static)",
            },
            "device_status": int(status),
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args)
    elif args.config4:
        run_config4(args)
    elif args.probe:
        run_probe(args)
    elif world > 1 and not args.replicas:
        run_cp(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
