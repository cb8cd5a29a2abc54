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
from . import functional as F
from .outer_product_mean import OuterProductMean
from .pair_weighted_averaging import PairWeightedAveraging
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

    def graphed(self, s: Tensor, z: Tensor, pair_mask: Tensor):
        """The block loop captured in a CUDA graph for inputs of these shapes: ``g = trunk.graphed(s, z, pair_mask)``
        once, then ``s_out, z_out = g(s, z[, pair_mask])`` per forward (see ``bioemu2_b200.graph``)."""
        from .graph import GraphedTrunk

        return GraphedTrunk(self, s, z, pair_mask)


class PairMixerMSALayer(nn.Module):
    """The MSA block of the PairMixer trunk (src/bioemu2/biomoa/modules/pairmixer.py:614-757):

        m += PairWeightedAveraging(m, z);  m += Transition(m);  z += OuterProductMean(m);
        z += TriMul_out(z);  z += TriMul_in(z);  z += Transition(z)

    Same sub-module names (``msa_transition``, ``pair_weighted_averaging``, ``tri_mul_out``, ``tri_mul_in``,
    ``z_transition``, ``outer_product_mean``), so the reference's state_dict loads unchanged.  The kernel-variant and
    tile-size keywords pick among the reference's backends and are accepted and ignored; dropout is the identity in
    eval mode, the only mode supported.
    """

    def __init__(self, token_s: int, msa_s: int, token_z: int, msa_dropout: float = 0.0, z_dropout: float = 0.0,
                 trimul_variant=None, trimul_tile_size: int | None = None, transition_chunk_size: int | None = None,
                 opm_variant=None, opm_tile_size: int | None = None, opm_matmul_precision: str | None = None,
                 trimul_matmul_precision: str | None = None) -> None:
        super().__init__()
        self.msa_dropout, self.z_dropout = msa_dropout, z_dropout
        self.msa_transition = Transition(dim=msa_s, hidden=msa_s * 4, chunk_size=transition_chunk_size)
        self.pair_weighted_averaging = PairWeightedAveraging(c_m=msa_s, c_z=token_z, c_h=32, num_heads=8)
        self.tri_mul_out = TriangleMultiplication(dim=token_z, mode="outgoing")
        self.tri_mul_in = TriangleMultiplication(dim=token_z, mode="incoming")
        self.z_transition = Transition(dim=token_z, hidden=token_z * 4, chunk_size=transition_chunk_size)
        self.outer_product_mean = OuterProductMean(c_in=msa_s, c_hidden=32, c_out=token_z, tile_size=opm_tile_size)

    def forward(self, s: Tensor, z: Tensor, m: Tensor, token_mask: Tensor, msa_mask: Tensor,
                chunk_heads_pwa: bool = False) -> tuple[Tensor, Tensor, Tensor]:
        """``s[B,T,token_s]``, ``z[B,T,T,token_z]``, ``m[B,S,T,msa_s]``, ``token_mask[B,T,T]`` (pair mask), ``msa_mask[B,S,T]``
        -> ``(s, z, m)``; the inputs are not modified."""
        if self.training:
            raise RuntimeError("bioemu2_b200 modules are inference-only: call .eval()")
        m = self.pair_weighted_averaging.forward_residual(m, z, token_mask)      # a new tensor
        self.msa_transition.forward_residual_(m)
        upd = self.outer_product_mean(m, msa_mask)
        z = F.add_rows(z.contiguous(), upd) if z.dtype == torch.float32 else z + upd.to(z.dtype)  # a new tensor
        mask8 = token_mask.to(torch.uint8).contiguous()
        self.tri_mul_out.forward_residual_(z, mask8)
        self.tri_mul_in.forward_residual_(z, mask8)
        self.z_transition.forward_residual_(z)
        return s, z, m
