"""PairMixer trunk blocks with the reference's contract (src/bioemu2/biomoa/modules/pairmixer.py:301-456).

``PairMixerLayer``: ``z += tri_mul_out(z); z += tri_mul_in(z); z += transition_z(z)``; ``s`` passes
through.  Constructor keywords that pick among the reference's kernel variants are accepted and
ignored.  Inference only: dropout is the identity in eval mode, which is the only mode supported.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from . import _lib
from .transition import Transition
from .triangle_multiplication import TriangleMultiplication


class PairMixerLayer(nn.Module):
    def __init__(self, token_s: int, token_z: int, dropout: float = 0.25, trimul_variant=None,
                 trimul_tile_size: int | None = None, transition_chunk_size: int | None = None,
                 trimul_matmul_precision: str | None = None) -> None:
        super().__init__()
        self.token_z = token_z
        self.dropout = dropout
        self.tri_mul_out = TriangleMultiplication(dim=token_z, mode="outgoing")
        self.tri_mul_in = TriangleMultiplication(dim=token_z, mode="incoming")
        self.transition_z = Transition(dim=token_z, hidden=token_z * 4, chunk_size=transition_chunk_size)

    def forward(self, s: Tensor, z: Tensor, pair_mask: Tensor) -> tuple[Tensor, Tensor]:
        if self.training:
            raise RuntimeError("bioemu2_b200 modules are inference-only: call .eval()")
        z = z.clone()  # the reference returns a new tensor; the three updates then run in place on the copy
        return s, self.forward_(z, pair_mask)

    def forward_(self, z: Tensor, pair_mask: Tensor) -> Tensor:
        """In-place form used by the trunk loop: updates and returns ``z``."""
        self.tri_mul_out.forward_residual_(z, pair_mask)
        self.tri_mul_in.forward_residual_(z, pair_mask)
        self.transition_z.forward_residual_(z)
        return z


class PairMixerModule(nn.Module):
    def __init__(self, token_s: int, token_z: int, num_blocks: int, dropout: float = 0.25, trimul_variant=None,
                 trimul_tile_size: int | None = None, transition_chunk_size: int | None = None,
                 trimul_matmul_precision: str | None = None) -> None:
        super().__init__()
        self.token_z = token_z
        self.num_blocks = num_blocks
        self.dropout = dropout
        self.layers = nn.ModuleList(
            [PairMixerLayer(token_s, token_z, dropout, transition_chunk_size=transition_chunk_size)
             for _ in range(num_blocks)])

    def forward(self, s: Tensor, z: Tensor, pair_mask: Tensor) -> tuple[Tensor, Tensor]:
        if self.training:
            raise RuntimeError("bioemu2_b200 modules are inference-only: call .eval()")
        z = z.clone()
        mask8 = pair_mask.to(torch.uint8).contiguous()  # converted once for all layers
        for layer in self.layers:
            layer.forward_(z, mask8)
        _lib.raise_if_device_wait()  # a kernel whose bounded wait ran out earlier in the stack invalidates the result
        return s, z
