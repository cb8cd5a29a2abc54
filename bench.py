"""Benchmark of the pair-representation trunk on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--tokens 512] [--blocks 48]
                    [--block pairformer|pairmixer]

A "step" is one forward of the 48-block Pairformer trunk over one pair tensor z[1, N, N, 128] and single
track s[1, N, 384] (fp32 residual streams, bf16 tensor-core arithmetic), N = 512 with the last 37 tokens
padded -- the configuration the headline metric (trunk ms/forward and pair-cells/s) is quoted on.  The
block is the benchmark's composite one (--block pairformer); --block pairmixer runs the reference trunk's
own attention-free block.  Inputs are synthetic
(seeded N(0,1)), weights random-init (Kaiming-uniform linears, LayerNorm 1/0).

One JSON line is printed by rank 0.  `value` is pair cells per second (N^2 / forward time, summed over
ranks), timed with CUDA events with z resident in HBM; `e2e` is the same through the public module call
with pinned HOST buffers, host->device and device->host copies inside the timed region; `roofline`
describes the dominant kernel; `cpu_baseline` is the CPU oracle timed on this host's cores on a bounded
sample.  With --gpus N > 1 (torchrun) every rank runs the same workload on its own pair tensor
(independent systems, no data-path collective): weak scaling.
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
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the kernels of the HBM-resident step one by one instead of replaying a CUDA graph")
    ap.add_argument("--cp", default=None, metavar="RxC",
                    help="context-parallel mode: ONE pair tensor tiled over an RxC grid of the --gpus ranks (strong "
                         "scaling) running the PairMixer blocks; the default without --cp is independent replicas")
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
    """Seeded synthetic trunk input: z, s ~ N(0,1), last 37 tokens padded (scaled for other sizes)."""
    import helpers as H

    g = torch.Generator().manual_seed(seed)
    w = {}
    for i in range(blocks):
        w.update(H.prefixed(f"layers.{i}", block_weights(g, kind)))
    z = torch.randn(1, tokens, tokens, 128, generator=g)
    s = torch.randn(1, tokens, 384, generator=g)
    tok = torch.ones(1, tokens, dtype=torch.bool)
    tok[0, tokens - pad_tokens(tokens):] = False
    return w, s, z, tok


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


def config_dict(args, impl_note: str) -> dict:
    what = ("triangle multiplication out/in, triangle attention start/end (4x32), pair transition, single-track "
            "pair-bias attention (16x24), single transition" if args.block == "pairformer"
            else "triangle multiplication out/in + pair transition (the reference trunk's own block)")
    return {
        "workload": f"Pairformer trunk forward, {args.blocks} blocks ({what}), N={args.tokens}, c_z=128, c_s=384, "
                    f"batch 1, last {pad_tokens(args.tokens)} tokens padded, seed 2",
        "block": args.block,
        "tokens": args.tokens,
        "blocks": args.blocks,
        "z_stream": "fp32",
        "arithmetic": "bf16 tensor cores, fp32 accumulate",
        "cache": "inputs larger than L2: z is 134 MB fp32 at N=512 and every kernel streams >=200 MB of scratch",
        "launch": "eager" if args.no_graph else "CUDA graph replay of the step (value); eager launches (e2e)",
        "parallelism": f"{args.gpus} independent replicas" if args.gpus > 1 else "single GPU",
        "note": impl_note,
    }


# ----------------------------------------------------------------------------------------- CPU oracle legs
def cpu_block_fn(tokens: int, kind: str):
    """Returns a closure running ONE block of the trunk with the CPU oracle, and the core count used."""
    from oracle import pair_ops as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(2)
    w = block_weights(g, kind)
    z = torch.randn(1, tokens, tokens, 128, generator=g)
    s = torch.randn(1, tokens, 384, generator=g)
    tok = torch.ones(1, tokens, dtype=torch.bool)
    tok[0, tokens - pad_tokens(tokens):] = False
    pm = tok[:, :, None] & tok[:, None, :]
    if kind == "pairmixer":
        return (lambda: O.pairmixer_layer(z, pm, w)), cores
    return (lambda: O.pairformer_block(s, z, tok, w, row_chunk=32)), cores


def time_cpu_oracle(tokens: int, kind: str, reps: int = 1):
    fn, cores = cpu_block_fn(tokens, kind)
    times = []
    with torch.no_grad():
        for _ in range(reps + 1):
            t0 = time.perf_counter()
            fn()
            times.append(time.perf_counter() - t0)
    times = sorted(times[1:])
    return times[len(times) // 2], cores


def run_reference(args) -> None:
    """--impl reference: the CPU port of the reference path, each step a bounded sample (one block)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    fn, cores = cpu_block_fn(args.tokens, args.block)
    steps = max(1, min(args.steps, 3))
    warm = min(args.warmup, 1)
    with torch.no_grad():
        for _ in range(warm):
            fn()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        dt = (time.perf_counter() - t0) / steps
    fwd = dt * args.blocks
    value = args.tokens ** 2 / fwd
    sample = (f"1 of {args.blocks} blocks per step at N={args.tokens} (fp32 torch on CPU, {dt:.2f} s/block), "
              f"forward time = {args.blocks} x block time")
    note = "CPU port of the reference modules (oracle/pair_ops.py)"
    if args.block == "pairformer":
        note += "; triangle attention is not in the reference and is timed from the oracle's own statement of it"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": fwd * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(args, note),
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


# ----------------------------------------------------------------------------------------- GPU arm
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
            for layer in trunk.layers:
                layer.forward_(s_work, z_work, tok_dev, mask8)
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
        for _ in range(max(args.warmup, 3)):
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

        step_e2e()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step_e2e()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        barrier()
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
        if composite:
            core_flops = 4.0 * N ** 3 * 128
            ach = tf(core_flops, t["attention_core"])
            ex2_floor_ms = (float(N) ** 3 * 4) / (16.0 * 148 * (clocks["sm_mhz"] or 1965) * 1e6) * 1e3 if clocks else None
            roofline = {
                "kernel": "flash_core_kernel<32,2> (triangle-attention core: QK^T + bias tile + online softmax + PV), "
                          "launched alone on N rows x 4 heads x 32",
                "bound": "tensor", "achieved": ach, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                "frac": ach / pk["bf16_tflops"], "peak_source": pk["source"] + " burst (kernel timed alone)",
                "algorithmic_flops_per_launch": core_flops, "ms_per_launch": t["attention_core"],
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch at N=512 (ncu capture summarised in
                # profiles/flash_core_triatt_n512.md); the operands scale with N^2, so other sizes are scaled from it
                "traffic": 323.5e6 * (N / 512.0) ** 2,
                "traffic_source": "ncu capture at N=512 (271.1 MB read + 52.4 MB written), scaled by (N/512)^2",
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
        launches_per_block = 25 if composite else 7
        h2d = z_host.numel() * 4 + s_host.numel() * 4 + (tok.numel() if composite else pair_mask.numel())
        line = {
            "metric": METRIC, "value": world * cells / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(args, "hand-written sm_100a kernels through the C ABI (libb200pair.so)"),
            "clocks": clocks,
            "e2e": {"value": world * cells / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": z_host.numel() * 4 + s_host.numel() * 4},
            "gpu_launches": args.steps * args.blocks * launches_per_block,
            "roofline": roofline, "ops": ops, "device_status": status,
        }
        if not args.no_cpu_baseline and world == 1:
            t_block, cores = time_cpu_oracle(N, args.block)
            line["cpu_baseline"] = {
                "value": cells / (t_block * args.blocks), "unit": UNIT, "cores": cores, "kind": "port",
                "sample": f"1 of {args.blocks} blocks at N={N} timed once after 1 warm-up ({t_block:.2f} s/block), "
                          f"forward = {args.blocks} x block",
            }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_cp(args) -> None:
    """One pair tensor sharded over an RxC grid: triangle multiplication exchanges b-operands (all-gather over the
    column / row group) and fp32 partial sums (reduce-scatter); everything else is local to the block."""
    import torch.distributed as dist

    import bioemu2_b200 as b
    from bioemu2_b200.context_parallel import CPGrid, CPPairMixerModule, kernel_shard_multiple

    rows, cols = (int(v) for v in args.cp.lower().split("x"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if rows * cols != world:
        raise SystemExit(f"--cp {args.cp} needs {rows * cols} ranks, got {world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    N = args.tokens
    if N % kernel_shard_multiple(rows, cols):
        raise SystemExit(f"--tokens must be a multiple of {kernel_shard_multiple(rows, cols)} for a {args.cp} grid")
    grid = CPGrid(rows, cols)
    torch.manual_seed(2)  # same seed on every rank: replicated weights
    tri = args.block == "pairformer"  # BASELINE config 3: triangle multiplication out/in + triangle attention start/end
    if tri:
        from bioemu2_b200.context_parallel import CPTriangleAttention, CPTriangleMultiplication

        blocks = [b.PairformerBlock().eval().to(dev) for _ in range(args.blocks)]
        ops = []
        for blk in blocks:
            ops += [CPTriangleMultiplication(blk.tri_mul_out, grid), CPTriangleMultiplication(blk.tri_mul_in, grid),
                    CPTriangleAttention(blk.tri_att_start, grid), CPTriangleAttention(blk.tri_att_end, grid)]

        def cp(zz, mm):
            for op in ops:
                op(zz, mm)
    else:
        serial = b.PairMixerModule(384, 128, args.blocks).eval().to(dev)
        cp = CPPairMixerModule(serial, grid)
    (r0, r1), (c0, c1) = grid.coords.my_rows(N), grid.coords.my_cols(N)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    z0 = torch.randn(1, r1 - r0, c1 - c0, 128, device=dev, generator=g)
    z = torch.empty_like(z0)
    mask = torch.ones(1, r1 - r0, c1 - c0, dtype=torch.uint8, device=dev)

    def step():
        z.copy_(z0)
        cp(z, mask)

    with torch.no_grad():
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        for _ in range(max(args.warmup, 3)):
            step()
        dist.barrier()
        torch.cuda.synchronize()
        ms = event_time_ms(step, args.steps)
        dist.barrier()
        torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else None
        status = b._lib.device_status()
    tt = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms = float(tt[0])
    if rank == 0:
        fl = block_flops(N, "pairmixer")
        if tri:
            fl["block"] = 2 * fl["trimul"] + 2 * block_flops(N, "pairformer")["triatt"]
        line = {
            "metric": METRIC, "value": N * N / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"context-parallel {'triangle multiplication out/in + triangle attention start/end' if tri else 'PairMixer trunk'}, {args.blocks} blocks, N={N}, one pair tensor tiled "
                                   f"{rows}x{cols} (block {r1 - r0}x{c1 - c0}), full mask", "grid": args.cp, "tokens": N,
                       "blocks": args.blocks, "z_stream": "fp32",
                       "exchange": "all-gather of the b operand + fp32 reduce-scatter of partial sums per direction (NCCL)"},
            "clocks": clocks, "gpu_launches": args.steps * args.blocks * (2 * (3 + rows + cols) + 1),
            "ops": {"trunk_tflops_aggregate": args.blocks * fl["block"] / (ms * 1e-3) / 1e12}, "device_status": status,
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.cp:
        run_cp(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
