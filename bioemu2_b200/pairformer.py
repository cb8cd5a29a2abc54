"""The composite Pairformer block the benchmark configurations describe, and its stack.

Pair track: triangle multiplication outgoing / incoming, triangle attention starting / ending node, pair
transition; single track: attention with pair bias (bias projected from z) and a transition; every
sub-block is residual.  The reference's own trunk block (``PairMixerLayer``, ``bioemu2_b200.pairmixer``) is
the first two and the fifth of these (src/bioemu2/biomoa/modules/pairmixer.py:430-456); the attention
sub-blocks are ``AttentionPairBias`` (src/bioemu2/biomoa/ops/attention_pair_bias.py:42) and the triangle
attention of ``bioemu2_b200.triangle_attention``, which the reference lacks.

Sub-module names: ``tri_mul_out``, ``tri_mul_in``, ``tri_att_start``, ``tri_att_end``, ``transition_z``,
``attention``, ``transition_s``.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from . import _lib
from .attention_pair_bias import AttentionPairBias
from .transition import Transition
from .triangle_attention import TriangleAttention
from .triangle_multiplication import TriangleMultiplication


class PairformerBlock(nn.Module):
    def __init__(self, token_s: int = 384, token_z: int = 128, tri_heads: int = 4, tri_head_dim: int = 32,
                 apb_heads: int = 16) -> None:
        super().__init__()
        self.tri_mul_out = TriangleMultiplication(token_z, "outgoing")
        self.tri_mul_in = TriangleMultiplication(token_z, "incoming")
        self.tri_att_start = TriangleAttention(token_z, tri_heads, tri_head_dim, ending=False)
        self.tri_att_end = TriangleAttention(token_z, tri_heads, tri_head_dim, ending=True)
        self.transition_z = Transition(token_z, 4 * token_z)
        self.attention = AttentionPairBias(token_s, token_z, apb_heads)
        self.transition_s = Transition(token_s, 4 * token_s)

    def forward_(self, s: Tensor, z: Tensor, token_mask: Tensor, pair_mask_u8: Tensor) -> tuple[Tensor, Tensor]:
        """In-place form: updates ``s`` and ``z`` (contiguous, fp32 or bf16) and returns them."""
        self.tri_mul_out.forward_residual_(z, pair_mask_u8)
        self.tri_mul_in.forward_residual_(z, pair_mask_u8)
        self.tri_att_start.forward_residual_(z, pair_mask_u8)
        self.tri_att_end.forward_residual_(z, pair_mask_u8)
        self.transition_z.forward_residual_(z)
        s += self.attention(s, z, token_mask)
        self.transition_s.forward_residual_(s)
        return s, z

    def forward(self, s: Tensor, z: Tensor, token_mask: Tensor) -> tuple[Tensor, Tensor]:
        if self.training:
            raise RuntimeError("bioemu2_b200 modules are inference-only: call .eval()")
        pm = (token_mask[:, :, None] & token_mask[:, None, :]).to(torch.uint8)
        return self.forward_(s.clone(), z.clone(), token_mask, pm)


class PairformerModule(nn.Module):
    def __init__(self, token_s: int = 384, token_z: int = 128, num_blocks: int = 48, **block_kwargs) -> None:
        super().__init__()
        self.num_blocks = num_blocks
        self.layers = nn.ModuleList([PairformerBlock(token_s, token_z, **block_kwargs) for _ in range(num_blocks)])

    def forward(self, s: Tensor, z: Tensor, token_mask: Tensor) -> tuple[Tensor, Tensor]:
        if self.training:
            raise RuntimeError("bioemu2_b200 modules are inference-only: call .eval()")
        s, z = s.clone(), z.clone()
        pm = (token_mask[:, :, None] & token_mask[:, None, :]).to(torch.uint8)
        self.forward_(s, z, token_mask, pm)
        _lib.raise_if_device_wait()  # a kernel whose bounded wait ran out earlier in the stack invalidates the result
        return s, z

    def forward_(self, s: Tensor, z: Tensor, token_mask: Tensor, pair_mask_u8: Tensor, overlap: bool = True):
        """The block loop in place on contiguous ``s`` and ``z``.

        The pair track never reads the single track, and the single track needs from the pair track only the 16-head
        attention bias of the block's final ``z``.  With ``overlap`` that bias is projected on the current stream
        right after the block's pair transition, and the rest of the block's single track - a handful of small,
        launch-bound kernels - runs on a side stream underneath the pair track of the NEXT block; the streams join at
        the end of the stack.  Two bias buffers alternate so that a block never overwrites a bias still being read.
        Both forms launch the same kernels on the same data and give identical results.
        """
        from . import functional as F
        from . import precision

        if (not overlap or len(self.layers) == 0 or precision.use_ieee(None, s, z)
                or any(layer.attention._bias_cache is not None for layer in self.layers)):
            for layer in self.layers:
                layer.forward_(s, z, token_mask, pair_mask_u8)
            return s, z
        dev = z.device
        main = torch.cuda.current_stream(dev)
        if self._side is None or self._side.device != dev:
            self._side = torch.cuda.Stream(device=dev)
        side = self._side
        B, N = z.shape[0], z.shape[1]
        heads = self.layers[0].attention.num_heads
        key = (B, N, heads, str(dev))
        if self._bias_key != key:
            self._bias = [torch.zeros(B, heads, N, F.pad8(N), dtype=torch.bfloat16, device=dev) for _ in range(2)]
            self._bias_key = key
        s_done = [None, None]
        side.wait_stream(main)  # s, and everything queued before this call, is ready for the side stream
        for i, layer in enumerate(self.layers):
            layer.tri_mul_out.forward_residual_(z, pair_mask_u8)
            layer.tri_mul_in.forward_residual_(z, pair_mask_u8)
            layer.tri_att_start.forward_residual_(z, pair_mask_u8)
            layer.tri_att_end.forward_residual_(z, pair_mask_u8)
            layer.transition_z.forward_residual_(z)
            k = i & 1
            if s_done[k] is not None:
                main.wait_event(s_done[k])  # the attention of block i - 2 has read this bias buffer
            w = layer.attention.packed()
            for b in range(B):
                F.pair_bias_slab(z[b], w.ln_z_w, w.ln_z_b, w.w_z, w.H, out=self._bias[k][b])
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(side):
                side.wait_event(ready)
                s += F.attention_pair_bias_with_bias(s, self._bias[k], token_mask, w)
                layer.transition_s.forward_residual_(s)
                s_done[k] = torch.cuda.Event()
                s_done[k].record(side)
        main.wait_stream(side)
        return s, z

    _side = None
    _bias = None
    _bias_key = None

    def graphed(self, s: Tensor, z: Tensor, token_mask: Tensor):
        """The block loop captured in a CUDA graph for inputs of these shapes: ``g = trunk.graphed(s, z, mask)`` once,
        then ``s_out, z_out = g(s, z[, mask])`` per forward (see ``bioemu2_b200.graph``)."""
        from .graph import GraphedTrunk

        return GraphedTrunk(self, s, z, token_mask)
