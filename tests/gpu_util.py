"""Helpers for the GPU parity tests: tolerance, a results log, device-status check."""
from __future__ import annotations

import json
import os
import tempfile

import torch

# The bf16 bar, in the reference's own form (tests/biomoa/ops/test_triangle_multiplication.py:50-77 in the
# reference): every element must satisfy |actual - expected| <= ATOL + RTOL * |expected|.  On top of that the
# normalised maximum max|actual - expected| / max|expected| must stay under BF16_REL, which is the stricter of the
# two for outputs of small magnitude.
BF16_ATOL = 2e-2
BF16_RTOL = 2e-2
BF16_REL = 2e-2
# One JSON line per checked case; BIOEMU2_B200_PARITY_LOG names the file, the default sits in the temp directory.
LOG = os.environ.get("BIOEMU2_B200_PARITY_LOG") or os.path.join(tempfile.gettempdir(), "bioemu2_b200_parity.jsonl")


def errors(actual: torch.Tensor, expected: torch.Tensor, atol: float = BF16_ATOL, rtol: float = BF16_RTOL) -> dict:
    a = actual.detach().double().cpu()
    e = expected.detach().double().cpu()
    diff = (a - e).abs()
    idx = int(diff.argmax())
    excess = diff - (atol + rtol * e.abs())
    return {
        "rel_max": float(diff.max() / e.abs().max().clamp_min(1e-30)),
        "rel_rms": float(diff.pow(2).mean().sqrt() / e.pow(2).mean().sqrt().clamp_min(1e-30)),
        "abs_max": float(diff.max()),
        "ref_absmax": float(e.abs().max()),
        "argmax": idx,
        "elementwise_violations": int((excess > 0).sum()),
        "elementwise_worst_excess": float(excess.max()),
        "nan": bool(torch.isnan(a).any()),
    }


def record(name: str, stats: dict) -> None:
    try:
        with open(LOG, "a") as f:
            f.write(json.dumps({"case": name, **stats}) + "\n")
    except OSError:
        pass


def assert_close(name: str, actual: torch.Tensor, expected: torch.Tensor, rel: float = BF16_REL,
                 atol: float = BF16_ATOL, rtol: float = BF16_RTOL) -> dict:
    import bioemu2_b200._lib as L

    status = L.device_status()
    st = errors(actual, expected, atol, rtol)
    st["device_status"] = status
    record(name, st)
    assert status == 0, f"{name}: device status {status:#x} (a bounded wait ran out)"
    assert not st["nan"], f"{name}: NaN in output"
    assert st["elementwise_violations"] == 0, (
        f"{name}: {st['elementwise_violations']} elements outside |d| <= {atol} + {rtol}|ref| ({st})")
    assert st["rel_max"] <= rel, f"{name}: rel_max {st['rel_max']:.4g} > {rel} ({st})"
    return st
