"""Pairwise conditioning of the diffusion module with the reference's contract
(src/bioemu2/biomoa/modules/diffusion.py:464-534).

``z = Linear(LayerNorm(cat(z_trunk, token_rel_pos_feats)))`` followed by ``z = Transition(z) + z`` per transition.
No pair talks to another pair: the module is three HBM-bound passes over the pair tensor.  The concatenation is never
materialised (the LayerNorm kernel reads the two sources), the projection is one tcgen05 GEMM writing fp32, and every
transition adds its residual in its final store.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from . import functional as F
from .transition import Transition


class PairwiseConditioning(nn.Module):
    def __init__(self, token_z: int, dim_token_rel_pos_feats: int, a_z: int | None = None, num_transitions: int = 2,
                 transition_expansion_factor: int = 2, transition_chunk_size: int | None = None) -> None:
        super().__init__()
        a_z = a_z if a_z is not None else token_z
        width = token_z + dim_token_rel_pos_feats
        if token_z % 8 or dim_token_rel_pos_feats % 8 or a_z % 8 or width > 1024:
            raise ValueError("bioemu2_b200.PairwiseConditioning needs widths that are multiples of 8 and "
                             "token_z + dim_token_rel_pos_feats <= 1024")
        self.token_z, self.dim_token_rel_pos_feats, self.a_z = token_z, dim_token_rel_pos_feats, a_z
        # same layout as the reference: index 0 is the LayerNorm, index 1 the bias-free projection
        self.dim_pairwise_init_proj = nn.Sequential(nn.LayerNorm(width), nn.Linear(width, a_z, bias=False))
        self.transitions = nn.ModuleList(
            [Transition(dim=a_z, hidden=transition_expansion_factor * a_z, chunk_size=transition_chunk_size)
             for _ in range(num_transitions)])
        self._w_bf16: Tensor | None = None
        self._w_version = -1

    def _weight(self) -> Tensor:
        w = self.dim_pairwise_init_proj[1].weight
        if self._w_bf16 is None or self._w_version != w._version or self._w_bf16.device != w.device:
            self._w_bf16 = w.detach().to(torch.bfloat16).contiguous()
            self._w_version = w._version
        return self._w_bf16

    def forward(self, z_trunk: Tensor, token_rel_pos_feats: Tensor) -> Tensor:
        """``z_trunk[B, N, N, token_z]``, ``token_rel_pos_feats[B, N, N, rel]`` -> fp32 ``[B, N, N, a_z]``."""
        if self.training:
            raise RuntimeError("bioemu2_b200 modules are inference-only: call .eval()")
        if z_trunk.shape[:-1] != token_rel_pos_feats.shape[:-1]:
            raise ValueError("z_trunk and token_rel_pos_feats must agree in every axis but the last")
        if z_trunk.shape[-1] != self.token_z or token_rel_pos_feats.shape[-1] != self.dim_token_rel_pos_feats:
            raise ValueError(f"expected widths {self.token_z} and {self.dim_token_rel_pos_feats}, got "
                             f"{z_trunk.shape[-1]} and {token_rel_pos_feats.shape[-1]}")
        if token_rel_pos_feats.dtype != z_trunk.dtype:
            token_rel_pos_feats = token_rel_pos_feats.to(z_trunk.dtype)
        ln = self.dim_pairwise_init_proj[0]
        zn = F.rows2_to_bf16(z_trunk, token_rel_pos_feats, ln.weight, ln.bias)
        z = F.linear_bf16(zn, self._weight(), out_dtype=torch.float32)
        for t in self.transitions:
            t.forward_residual_(z)
        return z
