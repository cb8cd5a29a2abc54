"""fp32-accurate ("ieee") forms of the pinned pair ops, still on the bf16 tensor cores.

The reference keeps several products in fp32 whatever the autocast state (attention core,
src/bioemu2/biomoa/ops/attention_pair_bias.py:165-167; outer-product contraction, outer_product_mean.py:66-74; the whole
denoiser, biomoa/models/score_model.py:355) and offers ``matmul_precision="ieee"`` on its kernel variants
(triangle_multiplication.py:119-136).  Here an fp32 value travels as ``hi = bf16(x)``, ``lo = bf16(x - hi)``; one operand
is laid out along K as ``(hi | hi | lo)``, the other as ``(hi | lo | hi)``, and the ordinary tcgen05 GEMM of width 3K
accumulates ``hi.hi + hi.lo + lo.hi`` in fp32 (relative error of a product ~2^-16).  LayerNorm, gates, SwiGLU and the
softmax run in fp32 with exact exponentials.  The compositions below are un-fused -- every intermediate goes through
HBM and the layout changes between pair-major and channel-major tensors are plain tensor permutes -- because this mode
exists for the 1e-4 accuracy contract, not for speed; the bf16 path is the fast one.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor

from . import _lib
from . import functional as F
from ._lib import lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def split(x: Tensor, order: int, ln_w: Tensor | None = None, ln_b: Tensor | None = None, normalize: bool = False,
          eps: float = 1e-5) -> Tensor:
    """``x[..., C]`` fp32 -> bf16 ``[..., 3C]``: (hi | hi | lo) for ``order`` 0, (hi | lo | hi) for 1, after an optional
    fp32 LayerNorm over the last axis."""
    if x.dtype != torch.float32:
        x = x.float()
    x = x.contiguous()
    cols = x.shape[-1]
    y = torch.empty(x.shape[:-1] + (3 * cols,), dtype=torch.bfloat16, device=x.device)
    w = ln_w.detach().float().contiguous() if ln_w is not None else None
    b = ln_b.detach().float().contiguous() if ln_b is not None else None
    _lib.check(lib.b200_split_rows(x.data_ptr(), y.data_ptr(), w.data_ptr() if w is not None else None,
                                   b.data_ptr() if b is not None else None, x.numel() // cols, cols, eps,
                                   1 if normalize else 0, order, _stream()))
    return y


def pad_last(x: Tensor, multiple: int = 8) -> Tensor:
    n = x.shape[-1]
    if n % multiple == 0:
        return x.contiguous()
    out = x.new_zeros(x.shape[:-1] + ((n + multiple - 1) // multiple * multiple,))
    out[..., :n] = x
    return out


def linear32(xs: Tensor, ws: Tensor, bias: Tensor | None = None, residual: Tensor | None = None) -> Tensor:
    """fp32 ``x @ w.T [+ bias] [+ residual]`` from split operands ``xs[..., 3K]`` (order 0) and ``ws[out, 3K]`` (order 1)."""
    return F.linear_bf16(xs, ws, bias, residual, out_dtype=torch.float32)


def gate(a: Tensor, b: Tensor, mode: int, rowmask: Tensor | None = None) -> Tensor:
    """fp32 rows: ``a * sigmoid(b)`` (mode 0), ``silu(a) * b`` (mode 1), ``a`` (mode 2); ``a``/``b`` may be column blocks
    of a wider tensor (unit stride in the last axis); ``rowmask`` (one byte per row) zeroes masked rows."""
    cols = a.shape[-1]
    rows = a.numel() // cols
    a2, b2 = a.reshape(rows, cols) if a.is_contiguous() else a, b.reshape(rows, cols) if b.is_contiguous() else b
    if a2.ndim != 2 or b2.ndim != 2 or a2.stride(1) != 1 or b2.stride(1) != 1:
        raise ValueError("gate needs 2-D operands with unit stride in the last axis")
    out = torch.empty(rows, cols, dtype=torch.float32, device=a.device)
    m = F.mask_u8(rowmask).reshape(-1) if rowmask is not None else None
    _lib.check(lib.b200_gate_rows_f32(a2.data_ptr(), a2.stride(0), b2.data_ptr(), b2.stride(0),
                                      m.data_ptr() if m is not None else None, out.data_ptr(), rows, cols, mode, _stream()))
    return out


class SplitWeights:
    """Order-1 split copies of a module's projection weights, built once per parameter version."""

    def __init__(self, **weights: Tensor) -> None:
        for k, v in weights.items():
            setattr(self, k, split(v.detach(), 1))


# ------------------------------------------------------------------------------------------------------ the ops
def transition(x: Tensor, norm, fc1, fc2, fc3, ws: SplitWeights, add_residual: bool = False) -> Tensor:
    shape = x.shape
    x2 = x.float().contiguous().view(-1, shape[-1])
    xs = split(x2, 0, norm.weight if norm is not None else None, norm.bias if norm is not None else None,
               normalize=norm is not None)
    h12 = linear32(xs, ws.w12)
    hidden = h12.shape[-1] // 2
    h = gate(h12[:, :hidden], h12[:, hidden:], 1)
    out = linear32(split(h, 0), ws.w3, residual=x2 if add_residual else None)
    return out.view(shape[:-1] + (out.shape[-1],))


def triangle_multiplication(x: Tensor, mask: Tensor, mod, ws: SplitWeights) -> Tensor:
    B, N, _, D = x.shape
    outs = []
    Nk = (N + 7) // 8 * 8
    for b in range(B):
        xb = x[b].float().contiguous().view(N * N, D)
        hs = split(xb, 0, mod.norm_in.weight, mod.norm_in.bias, normalize=True)
        pg = linear32(hs, ws.w_in)                                     # [P, 4D]: p_in | g_in
        ab = gate(pg[:, :2 * D], pg[:, 2 * D:], 0, rowmask=mask[b]).view(N, N, 2 * D)
        perm = (2, 1, 0) if mod.mode == "incoming" else (2, 0, 1)       # -> [d][i or j][k]
        a_t = torch.zeros(D, Nk, Nk, dtype=torch.float32, device=x.device)
        b_t = torch.zeros(D, Nk, Nk, dtype=torch.float32, device=x.device)
        a_t[:, :N, :N] = ab[:, :, :D].permute(*perm)
        b_t[:, :N, :N] = ab[:, :, D:].permute(*perm)
        t = torch.empty(D, Nk, Nk, dtype=torch.float32, device=x.device)
        F.bmm_nt_into(split(a_t, 0), split(b_t, 1), t)                 # t[d][i][j] = sum_k a.b, fp32
        tp = t[:, :N, :N].permute(1, 2, 0).contiguous().view(N * N, D)
        ts = split(tp, 0, mod.norm_out.weight, mod.norm_out.bias, normalize=True)
        outs.append(gate(linear32(ts, ws.w_p_out), linear32(hs, ws.w_g_out), 0).view(N, N, D))
    return torch.stack(outs)


def outer_product_mean(m: Tensor, mask: Tensor, mod, ws: SplitWeights) -> Tensor:
    B, S, N, C = m.shape
    ch = mod.c_hidden
    outs = []
    for b in range(B):
        ms = split(m[b].float().contiguous().view(S * N, C), 0, mod.norm.weight, mod.norm.bias, normalize=True)
        ab = linear32(ms, ws.w_ab)                                      # [S*N, 2*ch]
        if mask.ndim == 3:
            rowmask = mask[b]
            n_valid = float(mask[b].any(dim=-1).sum().clamp(min=1))
        else:
            rowmask = mask[b][None, :].expand(S, N)
            n_valid = 1.0
        ab = gate(ab, ab, 2, rowmask=rowmask.contiguous()).view(S, N, 2 * ch)
        a_t = pad_last(ab[:, :, :ch].permute(1, 2, 0).reshape(N * ch, S))   # [(i, c)][s]
        b_t = pad_last(ab[:, :, ch:].permute(1, 2, 0).reshape(N * ch, S))
        outer = torch.empty(1, N * ch, N * ch, dtype=torch.float32, device=m.device)
        F.bmm_nt_into(split(a_t, 0).unsqueeze(0), split(b_t, 1).unsqueeze(0), outer, scale=1.0 / n_valid)
        zz = outer.view(N, ch, N, ch).permute(0, 2, 1, 3).contiguous().view(N * N, ch * ch)
        outs.append(linear32(split(zz, 0), ws.w_o, bias=mod.proj_o.bias.detach().float().contiguous()).view(N, N, -1))
    return torch.stack(outs)


def attention_pair_bias(s: Tensor, z: Tensor, mask: Tensor, mod, ws: SplitWeights, multiplicity: int = 1) -> Tensor:
    BM, N, c = s.shape
    B, H = z.shape[0], mod.num_heads
    dh = c // H
    if N % 8:
        raise ValueError("the fp32-accurate attention needs a token count that is a multiple of 8 (pad and mask)")
    norm_s = mod.norm_s if mod.initial_norm else None
    ss = split(s.float().contiguous().view(BM * N, c), 0, norm_s.weight if norm_s is not None else None,
               norm_s.bias if norm_s is not None else None, normalize=norm_s is not None)
    qb = torch.zeros(3 * c, dtype=torch.float32, device=s.device)
    qb[:c] = mod.proj_q_bias.detach().float()
    qkv = linear32(ss, ws.w_qkv, bias=qb).view(BM, N, 3, H, dh)
    g = linear32(ss, ws.w_g)                                            # raw gate logits [BM*N, c]
    # pair bias, head-major: [H_pad][B*N*N] = W_z . LN_z(z)^T
    zs = split(z.float().contiguous().view(B * N * N, z.shape[-1]), 0, mod.norm_z.weight, mod.norm_z.bias, normalize=True)
    bias = torch.empty(1, ws.w_z.shape[0], B * N * N, dtype=torch.float32, device=s.device)
    # the activation (hi | hi | lo) sits on the B side here, the weight (hi | lo | hi) on the A side: the same three products
    F.bmm_nt_into(ws.w_z.unsqueeze(0), zs.unsqueeze(0), bias)
    bias = bias[0, :H].view(H, B, N, N).permute(1, 0, 2, 3).contiguous()              # [B, H, N, N]
    q = qkv[:, :, 0].permute(0, 2, 1, 3).contiguous().view(BM * H, N, dh)
    k = qkv[:, :, 1].permute(0, 2, 1, 3).contiguous().view(BM * H, N, dh)
    vT = qkv[:, :, 2].permute(0, 2, 3, 1).contiguous().view(BM * H, dh, N)
    logits = torch.empty(BM * H, N, N, dtype=torch.float32, device=s.device)
    F.bmm_nt_into(split(q, 0), split(k, 1), logits, scale=1.0 / math.sqrt(dh))
    m8 = F.mask_u8(mask)
    _lib.check(lib.b200_softmax_bias_f32(logits.data_ptr(), bias.data_ptr(), m8.data_ptr(), BM * H, N, H, multiplicity,
                                         _stream()))
    dhp = (dh + 7) // 8 * 8
    vT_p = vT if dhp == dh else torch.cat([vT, vT.new_zeros(BM * H, dhp - dh, N)], dim=1)
    o = torch.empty(BM * H, N, dhp, dtype=torch.float32, device=s.device)
    F.bmm_nt_into(split(logits, 0), split(vT_p, 1), o)
    o = o[:, :, :dh].reshape(BM, H, N, dh).permute(0, 2, 1, 3).contiguous().view(BM * N, c)
    og = gate(o, g, 0)
    return linear32(split(og, 0), ws.w_o).view(BM, N, c)
