"""Single-track attention with pair bias, reference contract of ``AttentionPairBias``
(src/bioemu2/biomoa/ops/attention_pair_bias.py:42-225): same constructor arguments, parameter names
(``norm_s``, ``proj_qkv``, ``proj_q_bias``, ``proj_g``, ``norm_z``, ``proj_z``, ``proj_o``) and
``forward(s, z, mask, multiplicity=1)``.

``tile_size`` bounds the logits tile of the reference's einsum path and ``use_efficient_fusion``
selects its conv2d formulation of the bias projection; the flash kernel needs neither, so both are
accepted and ignored (the results are the ones of the default, batch-invariant path).
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from . import functional as F
from .triangle_multiplication import PackedWeightsMixin


class AttentionPairBias(PackedWeightsMixin, nn.Module):
    def __init__(self, c_s: int, c_z: int, num_heads: int, inf: float = 1e6, initial_norm: bool = True,
                 tile_size: int | None = 512, zero_init_output: bool = False,
                 use_bias_in_layer_norm: bool = False, use_efficient_fusion: bool = False) -> None:
        super().__init__()
        assert c_s % num_heads == 0
        if use_efficient_fusion and use_bias_in_layer_norm:
            raise ValueError(
                "use_efficient_fusion=True is incompatible with use_bias_in_layer_norm=True: "
                "the LayerNorm+Linear fold cannot absorb a LayerNorm bias."
            )
        if inf != 1e6:
            raise ValueError("the kernel's masked-logit constant is the reference default inf=1e6")
        self.c_s, self.c_z, self.num_heads = c_s, c_z, num_heads
        self.head_dim = c_s // num_heads
        self.inf = inf
        self.tile_size = tile_size
        self.use_bias_in_layer_norm = use_bias_in_layer_norm
        self.use_efficient_fusion = use_efficient_fusion
        self.initial_norm = initial_norm
        if initial_norm:
            self.norm_s = nn.LayerNorm(c_s)
        self.proj_qkv = nn.Linear(c_s, 3 * c_s, bias=False)
        self.proj_q_bias = nn.Parameter(torch.zeros(c_s))
        self.proj_g = nn.Linear(c_s, c_s, bias=False)
        self.norm_z = nn.LayerNorm(c_z, bias=use_bias_in_layer_norm)
        self.proj_z = nn.Linear(c_z, num_heads, bias=False)
        self.proj_o = nn.Linear(c_s, c_s, bias=False)
        if zero_init_output:
            nn.init.zeros_(self.proj_o.weight)

    def _build_packed(self):
        return F.ApbPacked(
            self.c_s, self.c_z, self.num_heads, self.proj_qkv.weight, self.proj_q_bias, self.proj_g.weight,
            self.norm_z.weight, self.norm_z.bias, self.proj_z.weight, self.proj_o.weight,
            self.norm_s.weight if self.initial_norm else None, self.norm_s.bias if self.initial_norm else None)

    def forward(self, s: Tensor, z: Tensor, mask: Tensor, multiplicity: int = 1) -> Tensor:
        """``s[B*M,N,c_s]``, ``z[B,N,N,c_z]``, ``mask[B,N]`` bool -> ``[B*M,N,c_s]``."""
        assert s.ndim == 3 and z.ndim == 4 and mask.ndim == 2, f"{s.shape}, {z.shape}, {mask.shape}"
        assert s.shape[0] == z.shape[0] * multiplicity, f"{s.shape}, {z.shape}, multiplicity={multiplicity}"
        return F.attention_pair_bias(s, z, mask, self.packed(), multiplicity)
