"""Outer product mean with the reference's contract
(src/bioemu2/biomoa/ops/outer_product_mean.py:32-152: ``_OPMBase`` weights, ``forward(m, mask)``).

Both reference variants (``vanilla`` and ``triton_memory_saving``) compute the same function; there is
one implementation here, so both class names map to it and ``tile_size`` / ``matmul_precision`` are
accepted and ignored.  The kernels never build the ``[N, N, c_hidden^2]`` fp32 intermediate of the
vanilla variant: the MSA-depth contraction runs as a tcgen05 GEMM whose epilogue writes bf16 outer
products pair-contiguously, and ``proj_o`` is a second GEMM over them.
"""
from __future__ import annotations

import torch.nn as nn
from torch import Tensor

from . import functional as F
from . import ieee, precision
from .triangle_multiplication import PackedWeightsMixin


class OuterProductMean(PackedWeightsMixin, nn.Module):
    def __init__(self, c_in: int, c_hidden: int, c_out: int, tile_size: int | None = None,
                 matmul_precision: str | None = None) -> None:
        super().__init__()
        if matmul_precision not in (None, "ieee", "tf32", "tf32x3"):
            raise ValueError(f"matmul_precision must be in {{'ieee','tf32','tf32x3'}}; got {matmul_precision!r}.")
        # "ieee" selects the fp32-accurate contraction for fp32 inputs (the reference's default for its fp32 einsum,
        # outer_product_mean.py:66-74); None -- the default here -- and the tf32 settings take the bf16 tensor-core path.
        self.matmul_precision = matmul_precision
        if (c_in, c_hidden, c_out) != (64, 32, 128):
            raise ValueError("bioemu2_b200.OuterProductMean is built for c_in=64, c_hidden=32, c_out=128")
        self.c_hidden = c_hidden
        self.tile_size = 256 if tile_size is None else tile_size
        self.norm = nn.LayerNorm(c_in)
        self.proj_ab = nn.Linear(c_in, 2 * c_hidden, bias=False)
        self.proj_o = nn.Linear(c_hidden * c_hidden, c_out)

    def _build_packed(self):
        return F.OpmPacked(self.norm.weight, self.norm.bias, self.proj_ab.weight, self.proj_o.weight,
                           self.proj_o.bias)

    def _build_split(self):
        return ieee.SplitWeights(w_ab=self.proj_ab.weight, w_o=self.proj_o.weight)

    def forward(self, m: Tensor, mask: Tensor) -> Tensor:
        """``m[B,S,N,c_in]``, ``mask[B,S,N]`` or ``[B,N]`` -> ``[B,N,N,c_out]``."""
        if precision.use_ieee(self.matmul_precision, m):
            return ieee.outer_product_mean(m, mask, self, self.split_weights())
        return F.outer_product_mean(m, mask, self.packed())


OuterProductMeanVanilla = OuterProductMean
OuterProductMeanTritonMemorySaving = OuterProductMean
