"""Triangle multiplication modules with the reference's constructor / forward / state_dict contract.

Reference: ``_TriMulBase`` and ``TriangleMultiplicationFull`` in
src/bioemu2/biomoa/ops/triangle_multiplication.py:62-99, wrappers :370-395.  The parameters are the
same ``nn.LayerNorm`` / ``nn.Linear`` submodules under the same names, so checkpoints load unchanged;
the forward runs the sm_100a kernels (LayerNorm + gated projection, per-channel tcgen05 contraction,
LayerNorm + gated output projection).
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from . import functional as F
from . import ieee, precision


class PackedWeightsMixin:
    """Caches the bf16 kernel-layout copy of a module's parameters until one of them changes."""

    _packed = None
    _packed_key = None

    def _pack_key(self):
        return tuple((p.data_ptr(), p._version, str(p.device)) for p in self.parameters())

    def packed(self):
        key = self._pack_key()
        if self._packed is None or key != self._packed_key:
            with torch.no_grad():
                self._packed = self._build_packed()
            self._packed_key = key
        return self._packed

    _split = None
    _split_key = None

    def split_weights(self):
        """The (hi | lo | hi) split copies of the projection weights used by the fp32-accurate forms."""
        key = tuple((p.data_ptr(), p._version, str(p.device)) for p in self.parameters())
        if self._split is None or key != self._split_key:
            with torch.no_grad():
                self._split = self._build_split()
            self._split_key = key
        return self._split


class TriangleMultiplication(PackedWeightsMixin, nn.Module):
    """``TriangleMultiplication(dim, mode)``; registry kwargs of the reference's variants are accepted.

    ``tile_size`` selects among the reference's backends (triangle_multiplication.py:170-198) and is ignored.
    ``matmul_precision="ieee"`` (triangle_multiplication.py:119-136) selects the fp32-accurate form for fp32 inputs,
    as does ``bioemu2_b200.precision.set_matmul_precision("ieee")``; the default is the bf16 tensor-core path.
    """

    def __init__(self, dim: int = 128, mode: str = "outgoing", tile_size: int | None = None,
                 matmul_precision: str | None = None, **kwargs) -> None:
        super().__init__()
        assert mode in ("outgoing", "incoming")
        if dim != 128:
            raise ValueError("bioemu2_b200 triangle multiplication is built for dim=128")
        self.mode = mode
        self.dim = dim
        self.matmul_precision = matmul_precision
        self.norm_in = nn.LayerNorm(dim, eps=1e-5)
        self.p_in = nn.Linear(dim, 2 * dim, bias=False)
        self.g_in = nn.Linear(dim, 2 * dim, bias=False)
        self.norm_out = nn.LayerNorm(dim)
        self.p_out = nn.Linear(dim, dim, bias=False)
        self.g_out = nn.Linear(dim, dim, bias=False)

    def _build_packed(self):
        return F.TriMulPacked(self.norm_in.weight, self.norm_in.bias, self.p_in.weight, self.g_in.weight,
                              self.norm_out.weight, self.norm_out.bias, self.p_out.weight, self.g_out.weight)

    def _build_split(self):
        return ieee.SplitWeights(w_in=torch.cat([self.p_in.weight, self.g_in.weight], dim=0),
                                 w_p_out=self.p_out.weight, w_g_out=self.g_out.weight)

    def forward(self, x: Tensor, mask: Tensor) -> Tensor:
        """``x[B,N,N,dim]``, ``mask[B,N,N]`` -> update ``[B,N,N,dim]`` (no residual, like the reference)."""
        if precision.use_ieee(self.matmul_precision, x):
            return ieee.triangle_multiplication(x, mask, self, self.split_weights())
        return F.trimul(x, mask, self.packed(), incoming=self.mode == "incoming")

    def forward_residual_(self, x: Tensor, mask: Tensor) -> Tensor:
        """``x += forward(x, mask)`` in place with the add fused into the output kernel; returns ``x``."""
        if precision.use_ieee(self.matmul_precision, x):
            return x.add_(ieee.triangle_multiplication(x, mask, self, self.split_weights()))
        return F.trimul(x, mask, self.packed(), incoming=self.mode == "incoming", add_residual=True, out=x)


class TriangleMultiplicationOutgoing(TriangleMultiplication):
    def __init__(self, dim: int = 128) -> None:
        super().__init__(dim=dim, mode="outgoing")


class TriangleMultiplicationIncoming(TriangleMultiplication):
    def __init__(self, dim: int = 128) -> None:
        super().__init__(dim=dim, mode="incoming")
