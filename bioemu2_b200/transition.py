"""SwiGLU transition with the reference's contract (src/bioemu2/biomoa/ops/transition.py:17-91).

``fc3(silu(fc1(norm(x))) * fc2(norm(x)))``.  ``chunk_size`` exists in the reference to bound the
memory of the hidden activations; the fused kernel never materialises them, so it is accepted and
ignored.  The pair transition (dim 128, hidden up to 512) runs as one fused kernel; other widths (the single
track: 384 -> 1536, 768 -> 4*768) run as LayerNorm, two tcgen05 GEMMs and a SwiGLU kernel.
"""
from __future__ import annotations

import torch.nn as nn
from torch import Tensor

from . import functional as F
from . import ieee, precision
from .triangle_multiplication import PackedWeightsMixin


class Transition(PackedWeightsMixin, nn.Module):
    def __init__(self, dim: int, hidden: int, out_dim: int | None = None, use_norm: bool = True,
                 chunk_size: int | None = None) -> None:
        super().__init__()
        out_dim = out_dim or dim
        self.use_norm = use_norm
        self.chunk_size = chunk_size
        if use_norm:
            self.norm = nn.LayerNorm(dim, eps=1e-5)
        self.fc1 = nn.Linear(dim, hidden, bias=False)
        self.fc2 = nn.Linear(dim, hidden, bias=False)
        self.fc3 = nn.Linear(hidden, out_dim, bias=False)
        self.hidden = hidden
        self._fused = (dim, out_dim) == (128, 128) and hidden <= 512 and hidden % 8 == 0
        if not self._fused and (dim % 8 or hidden % 8 or out_dim % 8 or dim > 1024):
            raise ValueError("bioemu2_b200.Transition needs widths that are multiples of 8 and dim <= 1024")

    def _build_packed(self):
        cls = F.TransitionPacked if self._fused else F.TransitionGenericPacked
        return cls(self.norm.weight if self.use_norm else None, self.norm.bias if self.use_norm else None,
                   self.fc1.weight, self.fc2.weight, self.fc3.weight)

    def _build_split(self):
        import torch

        return ieee.SplitWeights(w12=torch.cat([self.fc1.weight, self.fc2.weight], dim=0), w3=self.fc3.weight)

    def _ieee(self, x: Tensor, add_residual: bool) -> Tensor:
        return ieee.transition(x, self.norm if self.use_norm else None, self.fc1, self.fc2, self.fc3, self.split_weights(),
                               add_residual)

    def forward(self, x: Tensor) -> Tensor:
        if precision.use_ieee(None, x):
            return self._ieee(x, False)
        if self._fused:
            return F.transition(x, self.packed())
        return F.transition_generic(x, self.packed())

    def forward_residual_(self, x: Tensor) -> Tensor:
        """``x += forward(x)`` in place, fused into the kernel's final store; returns ``x``."""
        if precision.use_ieee(None, x):
            return x.copy_(self._ieee(x, True))
        if self._fused:
            return F.transition(x, self.packed(), add_residual=True, out=x)
        return F.transition_generic(x, self.packed(), add_residual=True, out=x)
