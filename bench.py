"""Benchmark of the pair-representation trunk on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--tokens 512] [--blocks 48]

A "step" is one forward of the 48-block trunk over one pair tensor z[1, N, N, 128] (fp32 residual
stream, bf16 tensor-core arithmetic), N = 512 with the last 37 tokens padded -- the configuration the
headline metric (trunk ms/forward and pair-cells/s) is quoted on.  Inputs are synthetic
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
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def workload(tokens: int, blocks: int, seed: int = 2):
    """Seeded synthetic trunk input: z ~ N(0,1), last 37 tokens padded (scaled for other sizes)."""
    import helpers as H

    g = torch.Generator().manual_seed(seed)
    w = {}
    for i in range(blocks):
        w.update(H.prefixed(f"layers.{i}", H.pairmixer_layer_weights(g, 128, perturbed=False)))
    z = torch.randn(1, tokens, tokens, 128, generator=g)
    pad = max(1, round(37 * tokens / 512))
    tok = torch.ones(1, tokens, dtype=torch.bool)
    tok[0, tokens - pad:] = False
    pair_mask = tok[:, :, None] & tok[:, None, :]
    return w, z, pair_mask


def config_dict(args, impl_note: str) -> dict:
    return {
        "workload": f"PairMixer trunk forward, {args.blocks} blocks (triangle multiplication out/in + pair transition), "
                    f"N={args.tokens}, c_z=128, batch 1, last {max(1, round(37 * args.tokens / 512))} tokens padded",
        "tokens": args.tokens,
        "blocks": args.blocks,
        "z_stream": "fp32",
        "arithmetic": "bf16 tensor cores, fp32 accumulate",
        "cache": "inputs larger than L2: z is 134 MB fp32 and every kernel streams >=200 MB of scratch",
        "parallelism": f"{args.gpus} independent replicas" if args.gpus > 1 else "single GPU",
        "note": impl_note,
    }


# ----------------------------------------------------------------------------------------- CPU oracle legs
def time_cpu_oracle(tokens: int, reps: int = 2):
    """Times ONE block of the trunk with the CPU oracle on all host cores; returns seconds per block."""
    import helpers as H
    from oracle import pair_ops as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(2)
    w = H.pairmixer_layer_weights(g, 128, perturbed=False)
    z = torch.randn(1, tokens, tokens, 128, generator=g)
    tok = torch.ones(1, tokens, dtype=torch.bool)
    pm = tok[:, :, None] & tok[:, None, :]
    times = []
    with torch.no_grad():
        for _ in range(reps + 1):
            t0 = time.perf_counter()
            O.pairmixer_layer(z, pm, w)
            times.append(time.perf_counter() - t0)
    times = sorted(times[1:])
    return times[len(times) // 2], cores


def run_reference(args) -> None:
    """--impl reference: the CPU port of the reference path, each step a bounded sample (one block)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import helpers as H
    from oracle import pair_ops as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(2)
    w = H.pairmixer_layer_weights(g, 128, perturbed=False)
    z = torch.randn(1, args.tokens, args.tokens, 128, generator=g)
    tok = torch.ones(1, args.tokens, dtype=torch.bool)
    pm = tok[:, :, None] & tok[:, None, :]
    steps = min(args.steps, 4)
    warm = min(args.warmup, 1)
    with torch.no_grad():
        for _ in range(warm):
            O.pairmixer_layer(z, pm, w)
        t0 = time.perf_counter()
        for _ in range(steps):
            O.pairmixer_layer(z, pm, w)
        dt = (time.perf_counter() - t0) / steps
    fwd = dt * args.blocks
    value = args.tokens ** 2 / fwd
    sample = f"1 of {args.blocks} blocks per step at N={args.tokens} (fp32 torch on CPU), forward time = {args.blocks} x block time"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": fwd * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(args, "CPU port of the reference modules (oracle/pair_ops.py)"),
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

    w, z_host, pair_mask = workload(args.tokens, args.blocks, seed=2 + rank)
    trunk = b.PairMixerModule(384, 128, args.blocks).eval()
    trunk.load_state_dict(w, strict=True)
    trunk.to(dev)
    N = args.tokens
    cells = N * N
    z_pinned = z_host.pin_memory()
    mask_pinned = pair_mask.pin_memory()
    out_pinned = torch.empty_like(z_host).pin_memory()
    s_dummy = torch.zeros(1, N, 384, device=dev)
    z_dev = z_host.to(dev)
    z_work = torch.empty_like(z_dev)
    mask8 = pair_mask.to(dev).to(torch.uint8)

    def step_resident():
        z_work.copy_(z_dev)  # restore the input (the trunk loop updates z in place); 0.04 ms of a ~20 ms step
        for layer in trunk.layers:
            layer.forward_(z_work, mask8)

    def step_e2e():
        zd = z_pinned.to(dev, non_blocking=True)
        md = mask_pinned.to(dev, non_blocking=True)
        _, out = trunk(s_dummy, zd, md)
        out_pinned.copy_(out, non_blocking=True)
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

        # per-op timings on the same data (inputs > L2), for the roofline of the dominant kernel
        layer0 = trunk.layers[0]
        zt = z_dev.clone()
        it = max(args.steps, 5) * 4
        t_transition = event_time_ms(lambda: layer0.transition_z.forward_residual_(zt), it)
        zt.copy_(z_dev)
        t_trimul_out = event_time_ms(lambda: layer0.tri_mul_out.forward_residual_(zt, mask8), it)
        zt.copy_(z_dev)
        t_trimul_in = event_time_ms(lambda: layer0.tri_mul_in.forward_residual_(zt, mask8), it)
        Np = (N + 127) // 128 * 128
        a = torch.randn(128, Np, Np, device=dev).bfloat16()
        bb = torch.randn(128, Np, Np, device=dev).bfloat16()
        t_bmm = event_time_ms(lambda: b.functional.bmm_nt(a, bb), it)
        status = b._lib.device_status()

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        pk = peaks()
        P = float(cells)
        flops_transition = 393216.0 * P
        flops_trimul = 256.0 * N ** 3 + 196608.0 * P
        flops_block = 2 * flops_trimul + flops_transition
        tf = flops_transition / (t_transition * 1e-3) / 1e12
        roofline = {
            "kernel": "transition_kernel<fp32 stream> (fused LN + fc1|fc2 + SwiGLU + fc3 + residual)",
            "bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
            "frac": tf / pk["bf16_tflops"], "peak_source": pk["source"] + " burst (kernel timed alone)",
            "algorithmic_flops_per_launch": flops_transition, "ms_per_launch": t_transition,
            "traffic": None,
        }
        ops = {
            "transition_ms": t_transition, "transition_tflops": tf,
            "transition_hbm_gbs": 1024.0 * P / (t_transition * 1e-3) / 1e9,
            "trimul_outgoing_ms": t_trimul_out, "trimul_incoming_ms": t_trimul_in,
            "trimul_tflops": flops_trimul / (0.5 * (t_trimul_out + t_trimul_in) * 1e-3) / 1e12,
            "trimul_hbm_gbs": 3072.0 * P / (0.5 * (t_trimul_out + t_trimul_in) * 1e-3) / 1e9,
            "bmm_ms": t_bmm, "bmm_tflops": 256.0 * Np ** 3 / (t_bmm * 1e-3) / 1e12,
            "trunk_tflops": args.blocks * flops_block / (ms * 1e-3) / 1e12,
        }
        line = {
            "metric": METRIC, "value": world * cells / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(args, "hand-written sm_100a kernels through the C ABI (libb200pair.so)"),
            "clocks": clocks,
            "e2e": {"value": world * cells / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": z_host.numel() * 4 + pair_mask.numel(),
                    "d2h_bytes_per_step": z_host.numel() * 4},
            "gpu_launches": args.steps * args.blocks * 7,
            "roofline": roofline, "ops": ops, "device_status": status,
        }
        if not args.no_cpu_baseline and world == 1:
            t_block, cores = time_cpu_oracle(N)
            line["cpu_baseline"] = {
                "value": cells / (t_block * args.blocks), "unit": UNIT, "cores": cores, "kind": "port",
                "sample": f"1 of {args.blocks} blocks at N={N} timed (median of 2 after 1 warm-up, {t_block:.2f} s/block), "
                          f"forward = {args.blocks} x block",
            }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
