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
from . import ieee, precision
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

    _bias_cache = None   # (PairBiasCache, index of this module in it) once a cache has adopted the module

    def _build_split(self):
        wz = torch.zeros(16, self.c_z, dtype=torch.float32, device=self.proj_z.weight.device)
        wz[:self.num_heads] = self.proj_z.weight.detach().float()
        return ieee.SplitWeights(w_qkv=self.proj_qkv.weight, w_g=self.proj_g.weight, w_z=wz, w_o=self.proj_o.weight)

    def forward(self, s: Tensor, z: Tensor, mask: Tensor, multiplicity: int = 1) -> Tensor:
        """``s[B*M,N,c_s]``, ``z[B,N,N,c_z]``, ``mask[B,N]`` bool -> ``[B*M,N,c_s]``."""
        assert s.ndim == 3 and z.ndim == 4 and mask.ndim == 2, f"{s.shape}, {z.shape}, {mask.shape}"
        assert s.shape[0] == z.shape[0] * multiplicity, f"{s.shape}, {z.shape}, multiplicity={multiplicity}"
        if precision.use_ieee(None, s, z):
            return ieee.attention_pair_bias(s, z, mask, self, self.split_weights(), multiplicity)
        if self._bias_cache is not None:
            cache, index = self._bias_cache
            bias = cache.lookup(index, z)
            if bias is not None:
                return F.attention_pair_bias_with_bias(s, bias, mask, self.packed(), multiplicity)
        return F.attention_pair_bias(s, z, mask, self.packed(), multiplicity)


class AttentionPairBiasSlidingWindow(AttentionPairBias):
    """Sliding-window attention with pair bias of the atom transformer, reference contract of
    ``AttentionPairBiasSlidingWindow`` (src/bioemu2/biomoa/ops/attention_pair_bias.py:228-340): every window of
    ``window_queries`` atoms attends to the ``window_keys`` atoms centred on it, the pair bias is
    ``[B, heads, NW, W, H_keys]`` and shared by the ``multiplicity`` samples of a batch item.

    ``forward(s[B*M*NW, W, c_s], z[B, NW, W, H_keys, c_z], mask[B*NW, W], multiplicity)``.  The projections run on the
    tensor cores in bf16; scores, softmax and the weighted sum are fp32.
    """

    def __init__(self, c_s: int, c_z: int, num_heads: int, window_queries: int = 32, window_keys: int = 128,
                 inf: float = 1e6, initial_norm: bool = True, tile_size: int | None = 512,
                 zero_init_output: bool = False, use_bias_in_layer_norm: bool = False) -> None:
        super().__init__(c_s, c_z, num_heads, inf=inf, initial_norm=initial_norm, tile_size=tile_size,
                         zero_init_output=zero_init_output, use_bias_in_layer_norm=use_bias_in_layer_norm)
        if (window_keys - window_queries) % 2 or window_keys % 8 or window_keys < window_queries:
            raise ValueError("window_keys must be a multiple of 8, at least window_queries, with an even difference")
        self.window_queries, self.window_keys = window_queries, window_keys

    def _build_packed(self):
        return F.WindowApbPacked(
            self.c_s, self.c_z, self.num_heads, self.proj_qkv.weight, self.proj_q_bias, self.proj_g.weight,
            self.norm_z.weight, self.norm_z.bias, self.proj_z.weight, self.proj_o.weight,
            self.norm_s.weight if self.initial_norm else None, self.norm_s.bias if self.initial_norm else None)

    def forward(self, s: Tensor, z: Tensor, mask: Tensor, multiplicity: int = 1) -> Tensor:
        assert s.ndim == 3 and z.ndim == 5 and mask.ndim == 2, f"{s.shape}, {z.shape}, {mask.shape}"
        if s.shape[1] != self.window_queries or z.shape[3] != self.window_keys:
            raise ValueError(f"expected windows of {self.window_queries} queries and {self.window_keys} keys, got "
                             f"s {tuple(s.shape)}, z {tuple(z.shape)}")
        return F.window_attention_pair_bias(s, z, mask, self.packed(), multiplicity)


class PairBiasCache:
    """The pair biases ``proj_z(norm_z(z))`` of a stack of ``AttentionPairBias`` modules, computed in ONE pass over a
    pair tensor that stays the same for many calls.

    The diffusion module runs its token blocks once per denoising step on a pair tensor that is part of the static
    context (``compute_static_context``, src/bioemu2/biomoa/modules/diffusion.py:197-208; the layer loop :307-320), yet
    the reference projects the bias again in every layer of every step (src/bioemu2/biomoa/ops/attention_pair_bias.py:163),
    which re-reads all of ``z`` each time.  ``prepare(z)`` normalises ``z`` once (LayerNorm without its affine part,
    bf16) and multiplies it by all layers' projection weights at once -- the LayerNorm weights are folded into the
    projection rows -- giving ``[L, B, H, N, N]`` in bf16, already in the base-2 units the attention kernel works in.
    Afterwards a forward call of an adopted module that is handed the SAME tensor object (same storage, same version
    counter, same shape) skips its own projection and reads its slice; any other ``z`` takes the normal path.

        cache = PairBiasCache([layer.token_block.attention.pair_bias_attn for layer in diffusion.layers])
        cache.prepare(context.z)          # once per static context
        ...                               # the model's forward calls are unchanged

    Modules whose ``norm_z`` carries a bias, or a token count that is not a multiple of 8, fall back to one projection
    pass per layer inside ``prepare`` (still once per static context instead of once per step).
    """

    def __init__(self, attentions) -> None:
        self.attentions = list(attentions)
        if not self.attentions:
            raise ValueError("PairBiasCache needs at least one AttentionPairBias module")
        for i, a in enumerate(self.attentions):
            if not isinstance(a, AttentionPairBias):
                raise TypeError(f"module {i} is a {type(a).__name__}, not a bioemu2_b200 AttentionPairBias")
            a._bias_cache = (self, i)
        self._key = None
        self._bias = None
        self._weights = None
        self._weights_key = None

    def release(self) -> None:
        self._key, self._bias = None, None

    @staticmethod
    def _z_key(z: Tensor):
        return (z.data_ptr(), z._version, tuple(z.shape), z.dtype, str(z.device))

    def _fused_weights(self, device):
        key = tuple((a.proj_z.weight.data_ptr(), a.proj_z.weight._version, a.norm_z.weight.data_ptr(),
                     a.norm_z.weight._version) for a in self.attentions) + (str(device),)
        if self._weights is None or key != self._weights_key:
            with torch.no_grad():
                rows = [a.proj_z.weight.detach().float() * a.norm_z.weight.detach().float()[None, :] * F.LOG2E
                        for a in self.attentions]
                self._weights = torch.cat(rows, dim=0).to(device=device, dtype=torch.bfloat16).contiguous()
            self._weights_key = key
        return self._weights

    def prepare(self, z: Tensor) -> Tensor:
        """Compute and keep the biases of every adopted module for ``z[B, N, N, 128]``; returns ``[L, B, H, N, pitch]``."""
        if z.ndim != 4 or z.shape[1] != z.shape[2] or z.shape[3] != 128:
            raise ValueError(f"expected z[B,N,N,128], got {tuple(z.shape)}")
        B, N = z.shape[0], z.shape[1]
        heads = {a.num_heads for a in self.attentions}
        one_pass = (len(heads) == 1 and N % 8 == 0 and all(a.norm_z.bias is None for a in self.attentions))
        with torch.no_grad():
            if one_pass:
                H, L = heads.pop(), len(self.attentions)
                w_all = self._fused_weights(z.device)                               # [L*H, 128]
                bias = torch.empty(L, B, H, N, N, dtype=torch.bfloat16, device=z.device)
                zc = z.contiguous()
                for b in range(B):
                    zhat = F.rows_to_bf16(zc[b].view(N * N, 128), None, None, normalize=True)   # [N*N, 128]
                    out = bias[:, b].view(1, L * H, N * N) if B == 1 else torch.empty(1, L * H, N * N, dtype=torch.bfloat16,
                                                                                     device=z.device)
                    F.bmm_nt_into(w_all.view(1, L * H, 128), zhat.view(1, N * N, 128), out)
                    if B != 1:
                        bias[:, b] = out.view(L, H, N, N)
            else:
                per_layer = []
                for a in self.attentions:
                    pk = a.packed()
                    per_layer.append(torch.stack([F.pair_bias_slab(z[b], pk.ln_z_w, pk.ln_z_b, pk.w_z, pk.H) for b in range(B)]))
                bias = per_layer  # a list: head counts or pitches may differ between layers
        self._bias = bias
        self._key = self._z_key(z)
        return bias

    def lookup(self, index: int, z: Tensor):
        """The bias of module ``index`` if ``z`` is the tensor ``prepare`` saw, else ``None``."""
        if self._bias is None or self._key != self._z_key(z):
            return None
        return self._bias[index]
