"""Helpers for the GPU parity tests: tolerance, a results log, device-status check."""
from __future__ import annotations

import json
import os

import torch

# The stated bars: max|actual - expected| / max|expected|.
BF16_REL = 2e-2   # bf16 tensor-core path against the fp32/fp64 oracle
LOG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gpurun_out", "parity.jsonl")


def errors(actual: torch.Tensor, expected: torch.Tensor) -> dict:
    a = actual.detach().double().cpu()
    e = expected.detach().double().cpu()
    diff = (a - e).abs()
    idx = int(diff.argmax())
    return {
        "rel_max": float(diff.max() / e.abs().max().clamp_min(1e-30)),
        "rel_rms": float(diff.pow(2).mean().sqrt() / e.pow(2).mean().sqrt().clamp_min(1e-30)),
        "abs_max": float(diff.max()),
        "ref_absmax": float(e.abs().max()),
        "argmax": idx,
        "nan": bool(torch.isnan(a).any()),
    }


def record(name: str, stats: dict) -> None:
    try:
        os.makedirs(os.path.dirname(LOG), exist_ok=True)
        with open(LOG, "a") as f:
            f.write(json.dumps({"case": name, **stats}) + "\n")
    except OSError:
        pass


def assert_close(name: str, actual: torch.Tensor, expected: torch.Tensor, rel: float = BF16_REL) -> dict:
    import bioemu2_b200._lib as L

    status = L.device_status()
    st = errors(actual, expected)
    st["device_status"] = status
    record(name, st)
    assert status == 0, f"{name}: device status {status:#x} (a bounded wait ran out)"
    assert not st["nan"], f"{name}: NaN in output"
    assert st["rel_max"] <= rel, f"{name}: rel_max {st['rel_max']:.4g} > {rel} ({st})"
    return st
