"""Pair-weighted averaging with the reference's contract
(``PairWeightedAveraging``, src/bioemu2/biomoa/ops/pair_weighted_averaging.py:6-153): same constructor arguments,
parameter names (``norm_m``, ``norm_z``, ``proj_m``, ``proj_g``, ``proj_z``, ``proj_o``) and
``forward(m, z, mask, chunk_heads=False)``.

``chunk_heads`` selects the reference's head-by-head evaluation, which exists to bound the memory of the einsum path;
the result is the same function, and the composition here never builds more than one head-stack of weights, so the
flag is accepted and ignored.
"""
from __future__ import annotations

import torch.nn as nn
from torch import Tensor

from . import functional as F
from .triangle_multiplication import PackedWeightsMixin


class PairWeightedAveraging(PackedWeightsMixin, nn.Module):
    def __init__(self, c_m: int, c_z: int, c_h: int, num_heads: int, inf: float = 1e6,
                 use_bias_in_layer_norm: bool = True) -> None:
        super().__init__()
        if c_h != 32 or c_z != 128 or num_heads > 16 or c_m % 8:
            raise ValueError("bioemu2_b200.PairWeightedAveraging is built for c_h=32, c_z=128, at most 16 heads")
        if inf != 1e6:
            raise ValueError("the kernel's masked-logit constant is the reference default inf=1e6")
        self.c_m, self.c_z, self.c_h, self.num_heads, self.inf = c_m, c_z, c_h, num_heads, inf
        self.use_bias_in_layer_norm = use_bias_in_layer_norm
        self.norm_m = nn.LayerNorm(c_m)
        self.norm_z = nn.LayerNorm(c_z, bias=use_bias_in_layer_norm)
        self.proj_m = nn.Linear(c_m, c_h * num_heads, bias=False)
        self.proj_g = nn.Linear(c_m, c_h * num_heads, bias=False)
        self.proj_z = nn.Linear(c_z, num_heads, bias=False)
        self.proj_o = nn.Linear(c_h * num_heads, c_m, bias=False)

    def _build_packed(self):
        return F.PwaPacked(self.norm_m.weight, self.norm_m.bias, self.norm_z.weight, self.norm_z.bias, self.proj_m.weight,
                           self.proj_g.weight, self.proj_z.weight, self.proj_o.weight, self.num_heads)

    def forward(self, m: Tensor, z: Tensor, mask: Tensor, chunk_heads: bool = False) -> Tensor:
        """``m[B,S,N,c_m]``, ``z[B,N,N,c_z]``, ``mask[B,N,N]`` -> update ``[B,S,N,c_m]`` (no residual)."""
        return F.pair_weighted_averaging(m, z, mask, self.packed())

    def forward_residual(self, m: Tensor, z: Tensor, mask: Tensor) -> Tensor:
        """``m + forward(m, z, mask)`` with the add fused into the output projection."""
        return F.pair_weighted_averaging(m, z, mask, self.packed(), add_residual=True)
