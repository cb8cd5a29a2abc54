"""Token block of the diffusion module: ``ConditionedTransformerLayer`` with full attention
(src/bioemu2/biomoa/modules/transformer.py:231-353, ``ada_ln`` :26-41, ``AttentionLayer`` :54-135).

    alpha1, beta1, gamma1, alpha2, beta2, gamma2 = cond(c).chunk(6)        cond = LayerNorm -> SiLU -> Linear
    x += gamma1 * APB(lns * ((1 + alpha1) * LN(x) + beta1), pairs, mask)
    x += gamma2 * Transition(lns * ((1 + alpha2) * LN(x) + beta2))         Transition without its own norm

Same sub-module names as the reference (``cond.0``, ``cond.2``, ``attention.pair_bias_attn``, ``transition``),
so its state_dict loads unchanged.  With ``is_sliding_window=True`` the attention is the atom transformer's windowed
one (``SlidingWindowAttentionLayer`` :147-229 around ``AttentionPairBiasSlidingWindow``): same block, atoms in place of
tokens, the pair tensor pre-windowed ``[B, NW, W, H, dim_pairwise]``.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from . import functional as F
from .attention_pair_bias import AttentionPairBias, AttentionPairBiasSlidingWindow
from .transition import Transition
from .triangle_multiplication import PackedWeightsMixin


class AttentionLayer(nn.Module):
    def __init__(self, heads: int, dim: int = 384, dim_pairwise: int = 128,
                 attn_pair_bias_tile_size: int | None = None, is_sliding_window: bool = False,
                 window_queries: int | None = None, window_keys: int | None = None,
                 zero_init_output: bool = False) -> None:
        super().__init__()
        if is_sliding_window:
            assert window_queries is not None and window_keys is not None, (
                "sliding-window AttentionLayer requires window_queries / window_keys.")
            self.pair_bias_attn = AttentionPairBiasSlidingWindow(
                c_s=dim, c_z=dim_pairwise, num_heads=heads, window_queries=window_queries, window_keys=window_keys,
                initial_norm=False, zero_init_output=zero_init_output)
        else:
            self.pair_bias_attn = AttentionPairBias(
                c_s=dim, c_z=dim_pairwise, num_heads=heads, initial_norm=False, zero_init_output=zero_init_output,
                tile_size=512 if attn_pair_bias_tile_size is None else attn_pair_bias_tile_size)

    def forward(self, tokens: Tensor, pairs: Tensor, mask: Tensor | None = None, multiplicity: int = 1) -> Tensor:
        return self.pair_bias_attn(tokens, pairs, mask, multiplicity)


class SlidingWindowAttentionLayer(nn.Module):
    """Folds atoms into query windows around a windowed ``AttentionLayer`` (transformer.py:147-229):
    ``tokens[B*M, N, dim]``, ``pairs[B, NW, W, H, dim_pairwise]`` (or flat ``[B, N, H, dim_pairwise]``), ``mask[B, N]``."""

    def __init__(self, attn_window_queries: int, attn_window_keys: int, **atom_attention_kwargs) -> None:
        super().__init__()
        assert attn_window_queries > 1 and attn_window_keys > 1
        self.attn_window_queries, self.attn_window_keys = attn_window_queries, attn_window_keys
        self.attention_layer = AttentionLayer(**atom_attention_kwargs, is_sliding_window=True,
                                              window_queries=attn_window_queries, window_keys=attn_window_keys)

    def forward(self, tokens: Tensor, pairs: Tensor, mask: Tensor | None = None, multiplicity: int = 1) -> Tensor:
        W, H = self.attn_window_queries, self.attn_window_keys
        BM, N, D = tokens.shape
        if N % W:
            raise ValueError(f"the atom count {N} is not a multiple of the query window {W}")
        NW = N // W
        B = pairs.shape[0]
        if mask is None:
            mask = torch.ones(B, N, dtype=torch.bool, device=tokens.device)
        out = self.attention_layer(tokens.reshape(BM * NW, W, D), pairs.reshape(B, NW, W, H, -1), mask.reshape(B * NW, W),
                                   multiplicity)
        return out.view(BM, N, D)


class ConditionedTransformerLayer(PackedWeightsMixin, nn.Module):
    def __init__(self, dim: int, dim_pairwise: int, dim_cond: int, heads: int, transition_hidden: int,
                 is_sliding_window: bool = False, window_queries: int | None = None, window_keys: int | None = None,
                 attn_pair_bias_tile_size: int | None = None, lns_scale: float = 1.0) -> None:
        super().__init__()
        self.lns_scale = lns_scale
        self.dim = dim
        self.cond = nn.Sequential(nn.LayerNorm(dim_cond), nn.SiLU(), nn.Linear(dim_cond, 6 * dim))
        if is_sliding_window:
            assert window_queries is not None and window_keys is not None, (
                "sliding-window ConditionedTransformerLayer requires window_queries / window_keys.")
            self.attention: nn.Module = SlidingWindowAttentionLayer(
                attn_window_queries=window_queries, attn_window_keys=window_keys, heads=heads, dim=dim,
                dim_pairwise=dim_pairwise, attn_pair_bias_tile_size=attn_pair_bias_tile_size)
        else:
            self.attention = AttentionLayer(heads=heads, dim=dim, dim_pairwise=dim_pairwise,
                                            attn_pair_bias_tile_size=attn_pair_bias_tile_size)
        self.transition = Transition(dim=dim, hidden=transition_hidden, use_norm=False)

    def _pack_key(self):
        return tuple((p.data_ptr(), p._version, str(p.device)) for p in self.cond.parameters())

    def _build_packed(self):
        return (self.cond[2].weight.detach().to(torch.bfloat16).contiguous(),
                self.cond[2].bias.detach().float().contiguous())

    def forward(self, x: Tensor, pairs: Tensor, c: Tensor, mask: Tensor | None = None, multiplicity: int = 1) -> Tensor:
        if mask is None:  # full attention: pairs [B, T, T, .]; windowed: x [B*M, atoms, .]
            n = x.shape[1] if pairs.ndim == 5 else pairs.shape[1]
            mask = torch.ones(pairs.shape[0], n, dtype=torch.bool, device=x.device)
        return self._forward(x, pairs, c, mask, multiplicity, self.attention)

    def _forward(self, x: Tensor, pairs: Tensor, c: Tensor, mask: Tensor, multiplicity: int, attention) -> Tensor:
        """The block with the attention supplied by the caller (``attention(tokens, pairs, mask, multiplicity)``): the
        serial layer passes its own, the context-parallel wrapper the sharded one; everything else is per token."""
        w_cond, b_cond = self.packed()
        D = self.dim
        cn = F.rows_to_bf16(c, self.cond[0].weight, self.cond[0].bias, normalize=True, silu=True)
        cond = F.linear_bf16(cn, w_cond, b_cond, out_dtype=torch.float32)  # [rows, 6*dim] fp32
        x = x.contiguous().clone()
        h = attention(F.adaln(x, cond, 0, D, self.lns_scale), pairs, mask, multiplicity)
        F.gated_residual_(x, h, cond, 2 * D)
        h = self.transition(F.adaln(x, cond, 3 * D, 4 * D, self.lns_scale))
        F.gated_residual_(x, h, cond, 5 * D)
        return x
