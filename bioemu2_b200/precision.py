"""Which arithmetic the modules use for fp32 inputs.

``"bf16"`` (default): bf16 tensor-core operands, fp32 accumulation -- the reference's ``bf16-mixed`` trunk precision
(src/bioemu2/precision.py:9-26), held to the reference's bf16 bar (2e-2).  ``"ieee"``: the fp32-accurate split-operand
forms of ``bioemu2_b200.ieee`` for the pinned ops (triangle multiplication, transition, pair-bias attention, outer
product mean), held to 1e-4; the reference's ``32-true`` precision and its always-fp32 denoiser
(src/bioemu2/precision.py:29-47) are the counterpart.  A module constructed with ``matmul_precision="ieee"`` (the
keyword of the reference's kernel variants) uses the accurate form whatever the global setting.
"""
from __future__ import annotations

import contextlib

_MODE = "bf16"


def set_matmul_precision(mode: str) -> None:
    global _MODE
    if mode not in ("bf16", "ieee"):
        raise ValueError(f"matmul precision must be 'bf16' or 'ieee', got {mode!r}")
    _MODE = mode


def get_matmul_precision() -> str:
    return _MODE


@contextlib.contextmanager
def matmul_precision(mode: str):
    old = _MODE
    set_matmul_precision(mode)
    try:
        yield
    finally:
        set_matmul_precision(old)


def use_ieee(module_setting, *tensors) -> bool:
    """The accurate form applies to fp32 inputs when the module or the global setting asks for it."""
    if module_setting != "ieee" and _MODE != "ieee":
        return False
    import torch

    return all(t.dtype == torch.float32 for t in tensors)
