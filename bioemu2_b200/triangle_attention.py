"""Triangle self-attention around the starting / ending node (4 heads x 32 on a 128-channel pair tensor).

The reference does not contain this op -- its trunk deliberately drops triangle attention
(src/bioemu2/biomoa/modules/pairmixer.py:459-462) -- but the benchmark's Pairformer block names it, so it
is provided here as the AlphaFold-2 algorithm written with the reference's pair-bias-attention conventions
(bias-free projections, LayerNorm eps 1e-5, masked logits replaced by -1e6) plus a gating projection with a
bias initialised to 1.  Parameter names: ``layer_norm``, ``linear_q/k/v`` (no bias), ``linear_b`` (pair
bias, no bias), ``linear_g`` (with bias), ``linear_o`` (no bias).  ``forward(x, mask)`` returns the update
without the residual, like the reference's triangle multiplication does.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from . import functional as F
from .triangle_multiplication import PackedWeightsMixin


class TriangleAttention(PackedWeightsMixin, nn.Module):
    def __init__(self, dim: int = 128, num_heads: int = 4, head_dim: int = 32, ending: bool = False,
                 inf: float = 1e6) -> None:
        super().__init__()
        if (dim, num_heads, head_dim) != (128, 4, 32):
            raise ValueError("bioemu2_b200 triangle attention is built for dim=128, 4 heads of 32")
        if inf != 1e6:
            raise ValueError("the kernel's masked-logit constant is inf=1e6")
        self.dim, self.num_heads, self.head_dim, self.ending, self.inf = dim, num_heads, head_dim, ending, inf
        hd = num_heads * head_dim
        self.layer_norm = nn.LayerNorm(dim, eps=1e-5)
        self.linear_q = nn.Linear(dim, hd, bias=False)
        self.linear_k = nn.Linear(dim, hd, bias=False)
        self.linear_v = nn.Linear(dim, hd, bias=False)
        self.linear_b = nn.Linear(dim, num_heads, bias=False)
        self.linear_g = nn.Linear(dim, hd, bias=True)
        self.linear_o = nn.Linear(hd, dim, bias=False)
        with torch.no_grad():
            self.linear_g.bias.fill_(1.0)

    def _build_packed(self):
        return F.TriAttPacked(self.layer_norm.weight, self.layer_norm.bias, self.linear_q.weight, self.linear_k.weight,
                              self.linear_v.weight, self.linear_b.weight, self.linear_g.weight, self.linear_g.bias,
                              self.linear_o.weight)

    def forward(self, x: Tensor, mask: Tensor) -> Tensor:
        """``x[B,N,N,dim]``, ``mask[B,N,N]`` -> update ``[B,N,N,dim]`` (no residual)."""
        return F.triangle_attention(x, mask, self.packed(), self.ending)

    def forward_residual_(self, x: Tensor, mask: Tensor) -> Tensor:
        """``x += forward(x, mask)`` in place (the add is fused into the output projection); returns ``x``."""
        return F.triangle_attention(x, mask, self.packed(), self.ending, add_residual=True, out=x)


class TriangleAttentionStartingNode(TriangleAttention):
    def __init__(self, dim: int = 128, num_heads: int = 4, head_dim: int = 32) -> None:
        super().__init__(dim, num_heads, head_dim, ending=False)


class TriangleAttentionEndingNode(TriangleAttention):
    def __init__(self, dim: int = 128, num_heads: int = 4, head_dim: int = 32) -> None:
        super().__init__(dim, num_heads, head_dim, ending=True)
