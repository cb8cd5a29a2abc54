"""ctypes binding of ``libb200pair.so`` (the C ABI declared in ``include/b200pair.h``).

There is no fallback: if the library has not been built, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int64, c_size_t, c_ulonglong, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
# BIOEMU2_B200_LIB points at an alternative build of the same library (profiling or experimental builds).
LIB_PATH = os.environ.get("BIOEMU2_B200_LIB") or os.path.join(HERE, "libb200pair.so")

OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_CUDA = 2
ERR_UNSUPPORTED_DEVICE = 3
ERR_WORKSPACE = 4
ERR_DEVICE_WAIT = 5

DTYPE_BF16 = 0
DTYPE_F32 = 1


class TriMulWeights(Structure):
    _fields_ = [
        ("w_in", c_void_p),
        ("w_out", c_void_p),
        ("ln_in_w", c_void_p),
        ("ln_in_b", c_void_p),
        ("ln_out_w", c_void_p),
        ("ln_out_b", c_void_p),
    ]


class OpmWeights(Structure):
    _fields_ = [("w_ab", c_void_p), ("w_o", c_void_p), ("ln_w", c_void_p), ("ln_b", c_void_p), ("bias_o", c_void_p)]


class ApbWeights(Structure):
    _fields_ = [("w_qkg", c_void_p), ("b_qkg", c_void_p), ("w_v", c_void_p), ("w_z", c_void_p), ("ln_z_w", c_void_p),
                ("ln_z_b", c_void_p), ("ln_s_w", c_void_p), ("ln_s_b", c_void_p), ("w_o", c_void_p)]


class TriAttWeights(Structure):
    _fields_ = [("w_qkgv", c_void_p), ("g_bias", c_void_p), ("w_b", c_void_p), ("w_o", c_void_p), ("ln_w", c_void_p),
                ("ln_b", c_void_p)]


class AttentionCoreArgs(Structure):
    _fields_ = [
        ("qk", c_void_p), ("qk_width", c_int64), ("qk_batch_stride", c_int64), ("q_col0", c_int), ("k_col0", c_int),
        ("vT", c_void_p), ("v_pitch", c_int64), ("bias", c_void_p), ("bias_pitch", c_int64), ("bias_groups", c_int),
        ("bias_div", c_int), ("mask", c_void_p), ("mask_div", c_int), ("mask_row_stride", c_int64),
        ("mask_key_stride", c_int64), ("gate", c_void_p), ("gate_batch_stride", c_int64), ("gate_pitch", c_int),
        ("gate_col0", c_int), ("out", c_void_p), ("out_batch_stride", c_int64), ("out_pitch", c_int),
        ("out_col0", c_int), ("head_dim_padded", c_int), ("head_dim_out", c_int), ("N", c_int), ("H", c_int),
        ("batch", c_int),
    ]


# name -> (restype, argtypes); mirrors include/b200pair.h one to one
SIGNATURES = {
    "b200_version": (c_int, []),
    "b200_last_error": (c_char_p, []),
    "b200_check_device": (c_int, []),
    "b200_device_status": (c_int, [POINTER(c_int)]),
    "b200_peek_status": (c_int, [POINTER(c_int)]),
    "b200_launch_count": (c_ulonglong, []),
    "b200_layernorm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p]),
    "b200_bmm_nt_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64,
                                 c_int64, c_int64, c_int64, c_int64, c_float, c_void_p]),
    "b200_trimul_workspace_bytes": (c_size_t, [c_int]),
    "b200_trimul_fwd": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(TriMulWeights), c_int, c_int, c_int, c_int,
                                c_int, c_void_p, c_size_t, c_void_p]),
    "b200_trimul_project": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, POINTER(TriMulWeights), c_int, c_int, c_int64,
                                    c_int64, c_int, c_int, c_int, c_void_p]),
    "b200_trimul_output": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(TriMulWeights), c_int, c_int, c_int64, c_int,
                                   c_int, c_int, c_int, c_void_p]),
    "b200_bmm_nt": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int64,
                            c_int64, c_int64, c_float, c_int, c_void_p]),
    "b200_trimul_fwd_static": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(TriMulWeights), c_int, c_int, c_int,
                                       c_int, c_int, c_void_p]),
    "b200_transition_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                    c_int, c_int, c_void_p]),
    "b200_opm_workspace_bytes": (c_size_t, [c_int, c_int]),
    "b200_opm_fwd": (c_int, [c_void_p, c_void_p, c_int, c_void_p, POINTER(OpmWeights), c_int, c_int, c_int, c_int,
                             c_int, c_void_p, c_size_t, c_void_p]),
    "b200_attention_core_fwd": (c_int, [POINTER(AttentionCoreArgs), c_void_p]),
    "b200_opm_cols_fwd": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(OpmWeights), c_int, c_int, c_int, c_int, c_void_p,
                                  c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "b200_apb_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "b200_apb_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, POINTER(ApbWeights), c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "b200_triatt_workspace_bytes": (c_size_t, [c_int]),
    "b200_triatt_fwd": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(TriAttWeights), c_int, c_int, c_int, c_int,
                                c_int, c_void_p, c_size_t, c_void_p]),
    "b200_pair_bias_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64,
                                   c_int64, c_int, c_int, c_int, c_void_p]),
    "b200_apb_fwd_bias": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, POINTER(ApbWeights), c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "b200_triatt_slab_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "b200_triatt_slab_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, POINTER(TriAttWeights), c_int,
                                     c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "b200_rows_to_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_linear_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int,
                                 c_void_p]),
    "b200_swiglu_fwd": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "b200_adaln_fwd": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int64, c_int, c_int,
                               c_void_p]),
    "b200_split_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_int, c_int, c_void_p]),
    "b200_gate_rows_f32": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int,
                                   c_void_p]),
    "b200_softmax_bias_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "b200_masked_softmax_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_pwa_gate": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200_gated_residual_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_int,
                                        c_void_p]),
    "b200_window_bias_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                                     c_int, c_void_p]),
    "b200_window_attention_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_int, c_int, c_int, c_void_p]),
    "b200_pair_outer_sum": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200_add_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p]),
    "b200_rows2_to_bf16": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                   c_void_p]),
}

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: the CUDA library has not been built "
        "(run `python __graft_entry__.py` at the repository root). There is no CPU or PyTorch fallback."
    )

lib = ctypes.CDLL(LIB_PATH)
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return (lib.b200_last_error() or b"").decode()


class DeviceWaitError(RuntimeError):
    """A kernel gave up one of its bounded waits: its results, and those of the kernels queued behind it, are invalid."""


def decode_status(word: int) -> str:
    """Readable form of the device status word: low byte = kind (1: a bounded wait ran out), bits 8.. = wait site."""
    if word == 0:
        return "ok"
    kind = {1: "bounded wait ran out"}.get(word & 0xFF, f"unknown kind {word & 0xFF}")
    return f"{kind} at wait site {word >> 8} (status {word:#x})"


def check(status: int) -> None:
    """Turn a status code into the exception the reference modules would raise."""
    if status == OK:
        return
    msg = last_error()
    if status in (ERR_INVALID_ARGUMENT, ERR_WORKSPACE):
        raise ValueError(f"b200pair: {msg}")
    if status == ERR_DEVICE_WAIT:
        raise DeviceWaitError(f"b200pair: {msg}")
    raise RuntimeError(f"b200pair (status {status}): {msg}")


def device_status() -> int:
    """Synchronises the device, reads and clears the status word."""
    out = c_int(0)
    check(lib.b200_device_status(ctypes.byref(out)))
    return out.value


def peek_status() -> int:
    """The status word as written by kernels that have finished; no synchronisation."""
    out = c_int(0)
    check(lib.b200_peek_status(ctypes.byref(out)))
    return out.value


def raise_if_device_wait() -> None:
    """Poll at a natural synchronisation point (end of a forward, before a collective or a device-to-host copy):
    raises ``DeviceWaitError`` when a finished kernel reported a wait that ran out.  Costs one host memory read."""
    word = peek_status()
    if word != 0:
        raise DeviceWaitError(f"b200pair: {decode_status(word)}; results since then are invalid "
                              "(device_status() clears the condition)")


def launch_count() -> int:
    return int(lib.b200_launch_count())
