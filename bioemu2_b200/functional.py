"""Tensor-level entry points: torch tensors in, the C ABI underneath.

Every function runs on the current CUDA stream, allocates only through torch's caching allocator
(outputs and the shared scratch buffer) and raises ``ValueError`` for bad shapes, as the reference's
modules do, before anything is launched.
"""
from __future__ import annotations

import ctypes

import torch
from torch import Tensor

from . import _lib
from ._lib import lib

_WORKSPACES: dict[tuple[int, int], Tensor] = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def workspace(nbytes: int, device: torch.device) -> Tensor:
    """Scratch buffer shared by all ops on (device, stream); grown on demand, 1024-byte aligned."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes + 1024:
        buf = torch.empty(nbytes + 1024, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buf
    off = (-buf.data_ptr()) % 1024
    return buf[off:off + nbytes]


def release_workspaces() -> None:
    _WORKSPACES.clear()


def _zdtype(t: Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.DTYPE_F32
    if t.dtype == torch.bfloat16:
        return _lib.DTYPE_BF16
    raise ValueError(f"pair tensor must be float32 or bfloat16, got {t.dtype}")


def mask_u8(mask: Tensor) -> Tensor:
    """Masks travel as one byte per entry, non-zero = valid (bool tensors are reinterpreted, not copied)."""
    if mask.dtype == torch.uint8:
        return mask.contiguous()
    if mask.dtype == torch.bool:
        return mask.contiguous().view(torch.uint8)
    return (mask != 0).to(torch.uint8).contiguous()


def _require_cuda(*tensors: Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("bioemu2_b200 runs on CUDA tensors only (there is no CPU path)")


def layernorm(x: Tensor, weight: Tensor | None, bias: Tensor | None, eps: float = 1e-5) -> Tensor:
    _require_cuda(x)
    if x.dtype != torch.bfloat16:
        raise ValueError("layernorm expects bfloat16 rows")
    x = x.contiguous()
    cols = x.shape[-1]
    y = torch.empty_like(x)
    w = weight.float().contiguous() if weight is not None else None
    b = bias.float().contiguous() if bias is not None else None
    _lib.check(lib.b200_layernorm_fwd(x.data_ptr(), y.data_ptr(), w.data_ptr() if w is not None else None,
                                      b.data_ptr() if b is not None else None, x.numel() // cols, cols, eps,
                                      _stream()))
    return y


def bmm_nt(a: Tensor, b: Tensor, scale: float = 1.0) -> Tensor:
    """c[n] = scale * a[n] @ b[n].T for bf16 a[batch, M, K], b[batch, N, K]."""
    _require_cuda(a, b)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise ValueError("bmm_nt expects bfloat16 operands")
    if a.ndim != 3 or b.ndim != 3 or a.shape[0] != b.shape[0] or a.shape[2] != b.shape[2]:
        raise ValueError(f"bmm_nt shapes {tuple(a.shape)} x {tuple(b.shape)}")
    a, b = a.contiguous(), b.contiguous()
    batch, M, K = a.shape
    N = b.shape[1]
    c = torch.empty(batch, M, N, dtype=torch.bfloat16, device=a.device)
    _lib.check(lib.b200_bmm_nt_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), batch, M, N, K, K, K, N, M * K, N * K,
                                    M * N, scale, _stream()))
    return c


class TriMulPacked:
    """Device copies of the triangle-multiplication weights in the layouts ``b200_trimul_fwd`` expects."""

    def __init__(self, norm_in_w, norm_in_b, p_in, g_in, norm_out_w, norm_out_b, p_out, g_out):
        D = p_out.shape[0]
        if D != 128 or tuple(p_in.shape) != (256, 128):
            raise ValueError("the triangle-multiplication kernels are built for dim=128")
        bf = torch.bfloat16
        self.w_in = torch.cat([p_in[:D], g_in[:D], p_in[D:], g_in[D:]], dim=0).to(bf).contiguous()
        self.w_out = torch.cat([p_out, g_out], dim=0).to(bf).contiguous()
        self.ln = [t.detach().float().contiguous() for t in (norm_in_w, norm_in_b, norm_out_w, norm_out_b)]
        self.struct = _lib.TriMulWeights(self.w_in.data_ptr(), self.w_out.data_ptr(), *[t.data_ptr() for t in self.ln])


def trimul(x: Tensor, mask: Tensor, w: TriMulPacked, incoming: bool, add_residual: bool = False,
           out: Tensor | None = None) -> Tensor:
    """Triangle multiplication of ``x[B,N,N,128]`` (fp32 or bf16); ``out`` may be ``x`` itself."""
    _require_cuda(x, mask)
    if x.ndim != 4 or x.shape[1] != x.shape[2] or x.shape[3] != 128:
        raise ValueError(f"expected x[B,N,N,128], got {tuple(x.shape)}")
    if tuple(mask.shape) != tuple(x.shape[:3]):
        raise ValueError(f"mask shape {tuple(mask.shape)} does not match x {tuple(x.shape)}")
    zd = _zdtype(x)
    if not x.is_contiguous():
        if out is x:
            raise ValueError("in-place update needs a contiguous pair tensor")
        x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    elif out.dtype != x.dtype or out.shape != x.shape or not out.is_contiguous():
        raise ValueError("out must match x in shape and dtype and be contiguous")
    if x.numel() == 0:  # empty batch or no tokens: nothing to launch (with a residual, out = x = empty)
        return out
    m8 = mask_u8(mask)
    B, N = x.shape[0], x.shape[1]
    nbytes = lib.b200_trimul_workspace_bytes(N)
    ws = workspace(nbytes, x.device)
    _lib.check(lib.b200_trimul_fwd(x.data_ptr(), m8.data_ptr(), out.data_ptr(), ctypes.byref(w.struct), B, N,
                                   1 if incoming else 0, 1 if add_residual else 0, zd, ws.data_ptr(), nbytes,
                                   _stream()))
    return out


class TransitionPacked:
    """Weights of a 128 -> 512 -> 128 SwiGLU transition in the layout ``b200_transition_fwd`` expects.  A narrower
    hidden layer (the 128 -> 256 -> 128 transitions of the pairwise conditioning) is zero-padded to 512: the padded
    units contribute ``silu(0) * 0 = 0`` exactly, and one fused pass still beats four un-fused ones."""

    def __init__(self, norm_w, norm_b, fc1, fc2, fc3):
        hidden = fc1.shape[0]
        if fc1.shape[1] != 128 or tuple(fc2.shape) != tuple(fc1.shape) or tuple(fc3.shape) != (128, hidden) or hidden > 512:
            raise ValueError("the fused pair-transition kernel is built for dim=128, hidden<=512")
        if hidden < 512:
            pad = torch.zeros(512 - hidden, 128, dtype=fc1.dtype, device=fc1.device)
            fc1, fc2 = torch.cat([fc1.detach(), pad]), torch.cat([fc2.detach(), pad])
            fc3 = torch.cat([fc3.detach(), pad.t()], dim=1)
        bf = torch.bfloat16
        w13 = torch.cat([fc1.reshape(8, 64, 128), fc2.reshape(8, 64, 128)], dim=1)  # [8][128][128]
        self.w13 = w13.reshape(1024, 128).to(bf).contiguous()
        self.w3 = fc3.to(bf).contiguous()
        self.norm_w = norm_w.detach().float().contiguous() if norm_w is not None else None
        self.norm_b = norm_b.detach().float().contiguous() if norm_b is not None else None


def transition(x: Tensor, w: TransitionPacked, add_residual: bool = False, out: Tensor | None = None) -> Tensor:
    _require_cuda(x)
    if x.shape[-1] != 128:
        raise ValueError(f"expected x[..., 128], got {tuple(x.shape)}")
    zd = _zdtype(x)
    if not x.is_contiguous():
        if out is x:
            raise ValueError("in-place update needs a contiguous tensor")
        x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    elif out.dtype != x.dtype or out.shape != x.shape or not out.is_contiguous():
        raise ValueError("out must match x in shape and dtype and be contiguous")
    rows = x.numel() // 128
    if rows == 0:
        return out
    use_norm = w.norm_w is not None
    _lib.check(lib.b200_transition_fwd(x.data_ptr(), out.data_ptr(), w.w13.data_ptr(), w.w3.data_ptr(),
                                       w.norm_w.data_ptr() if use_norm else None,
                                       w.norm_b.data_ptr() if use_norm else None, rows, 1 if use_norm else 0,
                                       1 if add_residual else 0, zd, _stream()))
    return out


class OpmPacked:
    """Weights of the outer product mean (c_in 64, c_hidden 32, c_out 128) for ``b200_opm_fwd``."""

    def __init__(self, norm_w, norm_b, proj_ab, proj_o_w, proj_o_b):
        if tuple(proj_ab.shape) != (64, 64) or tuple(proj_o_w.shape) != (128, 1024):
            raise ValueError("the outer-product-mean kernels are built for c_in=64, c_hidden=32, c_out=128")
        bf = torch.bfloat16
        self.w_ab = proj_ab.to(bf).contiguous()
        self.w_o = proj_o_w.to(bf).contiguous()
        self.f32 = [t.detach().float().contiguous() for t in (norm_w, norm_b, proj_o_b)]
        self.struct = _lib.OpmWeights(self.w_ab.data_ptr(), self.w_o.data_ptr(), self.f32[0].data_ptr(),
                                      self.f32[1].data_ptr(), self.f32[2].data_ptr())


def outer_product_mean(m: Tensor, mask: Tensor, w: OpmPacked) -> Tensor:
    """``m[B,S,N,64]`` (fp32 or bf16), ``mask[B,S,N]`` or ``[B,N]`` -> ``[B,N,N,128]`` in ``m.dtype``."""
    _require_cuda(m, mask)
    if m.ndim != 4 or m.shape[-1] != 64:
        raise ValueError(f"expected m[B,S,N,64], got {tuple(m.shape)}")
    B, S, N, _ = m.shape
    if mask.ndim == 3:
        if tuple(mask.shape) != (B, S, N):
            raise ValueError(f"mask shape {tuple(mask.shape)} does not match m {tuple(m.shape)}")
    elif mask.ndim == 2:
        if tuple(mask.shape) != (B, N) or B != 1:
            raise ValueError("a [B,N] mask needs B == 1 (the only shape that broadcasts in the reference)")
    else:
        raise ValueError("mask must be [B,S,N] or [B,N]")
    zd = _zdtype(m)
    m = m.contiguous()
    out = torch.empty(B, N, N, 128, dtype=m.dtype, device=m.device)
    if out.numel() == 0:
        return out
    if S == 0:  # no MSA rows: the mean of nothing is zero, so every pair gets proj_o's bias
        return out.copy_(w.f32[2].to(out.dtype).expand_as(out))
    m8 = mask_u8(mask)
    nbytes = lib.b200_opm_workspace_bytes(S, N)
    ws = workspace(nbytes, m.device)
    _lib.check(lib.b200_opm_fwd(m.data_ptr(), m8.data_ptr(), mask.ndim, out.data_ptr(), ctypes.byref(w.struct), B, S, N,
                                zd, zd, ws.data_ptr(), nbytes, _stream()))
    return out


LOG2E = 1.4426950408889634


def _pad_heads(wt: Tensor, H: int, dh: int, DH: int) -> Tensor:
    """[H*dh, ...] -> [H*DH, ...] with zero rows appended to every head."""
    rest = wt.shape[1:]
    out = wt.new_zeros((H, DH) + tuple(rest))
    out[:, :dh] = wt.reshape((H, dh) + tuple(rest))
    return out.reshape((H * DH,) + tuple(rest))


class ApbPacked:
    """Weights of single-track pair-bias attention in the layouts ``b200_apb_fwd`` expects."""

    def __init__(self, c_s, c_z, H, proj_qkv, proj_q_bias, proj_g, norm_z_w, norm_z_b, proj_z, proj_o,
                 norm_s_w=None, norm_s_b=None):
        if c_z != 128:
            raise ValueError("pair-bias attention is built for c_z=128")
        dh = c_s // H
        if c_s % H or dh % 8 or dh > 64 or H > 16:
            raise ValueError("pair-bias attention needs H <= 16 and a head dim that is a multiple of 8 and <= 64")
        DH = 32 if dh <= 32 else 64
        self.c_s, self.H = c_s, H
        bf = torch.bfloat16
        wq, wk, wv = proj_qkv.detach().float().chunk(3, dim=0)
        qscale = LOG2E / (dh ** 0.5)
        self.w_qkg = torch.cat([_pad_heads(wq * qscale, H, dh, DH), _pad_heads(wk, H, dh, DH),
                                proj_g.detach().float()], dim=0).to(bf).contiguous()
        b = torch.zeros(2 * H * DH + c_s, dtype=torch.float32, device=proj_qkv.device)
        b[: H * DH] = _pad_heads(proj_q_bias.detach().float() * qscale, H, dh, DH)
        self.b_qkg = b
        self.w_v = _pad_heads(wv, H, dh, DH).to(bf).contiguous()
        wz = torch.zeros(16, 128, dtype=torch.float32, device=proj_z.device)
        wz[:H] = proj_z.detach().float()
        self.w_z = wz.to(bf).contiguous()
        self.ln_z_w = norm_z_w.detach().float().contiguous()
        self.ln_z_b = norm_z_b.detach().float().contiguous() if norm_z_b is not None else None
        self.ln_s_w = norm_s_w.detach().float().contiguous() if norm_s_w is not None else None
        self.ln_s_b = norm_s_b.detach().float().contiguous() if norm_s_b is not None else None
        self.w_o = proj_o.detach().to(bf).contiguous()
        ptr = lambda t: t.data_ptr() if t is not None else None  # noqa: E731
        self.struct = _lib.ApbWeights(ptr(self.w_qkg), ptr(self.b_qkg), ptr(self.w_v), ptr(self.w_z), ptr(self.ln_z_w),
                                      ptr(self.ln_z_b), ptr(self.ln_s_w), ptr(self.ln_s_b), ptr(self.w_o))


def attention_pair_bias(s: Tensor, z: Tensor, mask: Tensor, w: ApbPacked, multiplicity: int = 1) -> Tensor:
    """``s[B*M,N,c_s]``, ``z[B,N,N,128]``, ``mask[B,N]`` -> ``[B*M,N,c_s]`` in ``s.dtype``."""
    _require_cuda(s, z, mask)
    if s.ndim != 3 or z.ndim != 4 or mask.ndim != 2:
        raise ValueError(f"{tuple(s.shape)}, {tuple(z.shape)}, {tuple(mask.shape)}")
    B, N = z.shape[0], z.shape[1]
    if s.shape[0] != B * multiplicity or s.shape[1] != N or s.shape[2] != w.c_s:
        raise ValueError(f"{tuple(s.shape)}, {tuple(z.shape)}, multiplicity={multiplicity}")
    if tuple(z.shape) != (B, N, N, 128) or tuple(mask.shape) != (B, N):
        raise ValueError(f"z {tuple(z.shape)} / mask {tuple(mask.shape)} do not match s {tuple(s.shape)}")
    sd, zd = _zdtype(s), _zdtype(z)
    s, z = s.contiguous(), z.contiguous()
    out = torch.empty_like(s)
    if out.numel() == 0:
        return out
    m8 = mask_u8(mask)
    nbytes = lib.b200_apb_workspace_bytes(B, multiplicity, N, w.c_s, w.H)
    ws = workspace(nbytes, s.device)
    _lib.check(lib.b200_apb_fwd(s.data_ptr(), z.data_ptr(), m8.data_ptr(), out.data_ptr(), ctypes.byref(w.struct), B,
                                multiplicity, N, w.c_s, w.H, sd, zd, ws.data_ptr(), nbytes, _stream()))
    return out


class TriAttPacked:
    """Weights of triangle attention (dim 128, 4 heads x 32) in the layouts ``b200_triatt_fwd`` expects."""

    def __init__(self, ln_w, ln_b, wq, wk, wv, wb, wg, bg, wo):
        if tuple(wq.shape) != (128, 128) or tuple(wb.shape) != (4, 128) or tuple(wo.shape) != (128, 128):
            raise ValueError("triangle attention is built for dim=128, 4 heads of 32")
        bf = torch.bfloat16
        qscale = LOG2E / (32 ** 0.5)
        self.w_qkgv = torch.cat([wq.detach().float() * qscale, wk.detach().float(), wg.detach().float(),
                                 wv.detach().float()], dim=0).to(bf).contiguous()
        wb16 = torch.zeros(16, 128, dtype=torch.float32, device=wb.device)
        wb16[:4] = wb.detach().float()
        self.w_b = wb16.to(bf).contiguous()
        self.w_o = wo.detach().to(bf).contiguous()
        self.f32 = [t.detach().float().contiguous() for t in (bg, ln_w, ln_b)]
        self.struct = _lib.TriAttWeights(self.w_qkgv.data_ptr(), self.f32[0].data_ptr(), self.w_b.data_ptr(),
                                         self.w_o.data_ptr(), self.f32[1].data_ptr(), self.f32[2].data_ptr())


def triangle_attention(x: Tensor, mask: Tensor, w: TriAttPacked, ending: bool, add_residual: bool = False,
                       out: Tensor | None = None) -> Tensor:
    """Triangle attention of ``x[B,N,N,128]`` (fp32 or bf16) with ``mask[B,N,N]``; ``out`` may be ``x``."""
    _require_cuda(x, mask)
    if x.ndim != 4 or x.shape[1] != x.shape[2] or x.shape[3] != 128:
        raise ValueError(f"expected x[B,N,N,128], got {tuple(x.shape)}")
    if tuple(mask.shape) != tuple(x.shape[:3]):
        raise ValueError(f"mask shape {tuple(mask.shape)} does not match x {tuple(x.shape)}")
    zd = _zdtype(x)
    if not x.is_contiguous():
        if out is x:
            raise ValueError("in-place update needs a contiguous pair tensor")
        x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    elif out.dtype != x.dtype or out.shape != x.shape or not out.is_contiguous():
        raise ValueError("out must match x in shape and dtype and be contiguous")
    if x.numel() == 0:
        return out
    m8 = mask_u8(mask)
    B, N = x.shape[0], x.shape[1]
    nbytes = lib.b200_triatt_workspace_bytes(N)
    ws = workspace(nbytes, x.device)
    _lib.check(lib.b200_triatt_fwd(x.data_ptr(), m8.data_ptr(), out.data_ptr(), ctypes.byref(w.struct), B, N,
                                   1 if ending else 0, 1 if add_residual else 0, zd, ws.data_ptr(), nbytes, _stream()))
    return out


# ----------------------------------------------------------------------------------- single-track building blocks
def _ptr(t: Tensor | None):
    return t.data_ptr() if t is not None else None


def rows_to_bf16(x: Tensor, weight: Tensor | None = None, bias: Tensor | None = None, normalize: bool = True,
                 silu: bool = False) -> Tensor:
    """``[silu]([LayerNorm](x) * weight + bias)`` over the last axis as bf16 (x fp32 or bf16)."""
    _require_cuda(x)
    xd = _zdtype(x)
    x = x.contiguous()
    cols = x.shape[-1]
    y = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    if y.numel() == 0:
        return y
    w = weight.detach().float().contiguous() if weight is not None else None
    b = bias.detach().float().contiguous() if bias is not None else None
    _lib.check(lib.b200_rows_to_bf16(x.data_ptr(), y.data_ptr(), _ptr(w), _ptr(b), x.numel() // cols, cols, xd,
                                     1 if normalize else 0, 1 if silu else 0, _stream()))
    return y


def linear_bf16(x: Tensor, w_bf16: Tensor, bias_f32: Tensor | None = None, residual: Tensor | None = None,
                out_dtype: torch.dtype = torch.bfloat16, out: Tensor | None = None) -> Tensor:
    """``x @ w.T [+ bias] [+ residual]`` with bf16 ``x[..., in]`` and ``w[out, in]``; ``out`` may be ``residual``."""
    _require_cuda(x, w_bf16)
    if x.dtype != torch.bfloat16 or w_bf16.dtype != torch.bfloat16:
        raise ValueError("linear_bf16 expects bfloat16 x and w")
    x = x.contiguous()
    fin, fout = x.shape[-1], w_bf16.shape[0]
    if w_bf16.shape[1] != fin:
        raise ValueError(f"weight {tuple(w_bf16.shape)} does not match input width {fin}")
    rows = x.numel() // fin
    if out is None:
        out = torch.empty(x.shape[:-1] + (fout,), dtype=out_dtype, device=x.device)
    od = _zdtype(out)
    if rows == 0:
        return out
    if residual is not None and (residual.dtype != out.dtype or residual.shape != out.shape or not residual.is_contiguous()):
        raise ValueError("residual must match the output in shape and dtype and be contiguous")
    _lib.check(lib.b200_linear_bf16(x.data_ptr(), w_bf16.data_ptr(), _ptr(bias_f32), _ptr(residual), out.data_ptr(),
                                    rows, fin, fout, od, _stream()))
    return out


def rows2_to_bf16(x1: Tensor, x2: Tensor, weight: Tensor | None = None, bias: Tensor | None = None,
                  normalize: bool = True) -> Tensor:
    """``LayerNorm(cat(x1, x2, -1)) * weight + bias`` as bf16 without materialising the concatenation."""
    _require_cuda(x1, x2)
    if x1.shape[:-1] != x2.shape[:-1] or x1.dtype != x2.dtype:
        raise ValueError("x1 and x2 must agree in dtype and in every axis but the last")
    x1, x2 = x1.contiguous(), x2.contiguous()
    c1, c2 = x1.shape[-1], x2.shape[-1]
    y = torch.empty(x1.shape[:-1] + (c1 + c2,), dtype=torch.bfloat16, device=x1.device)
    if y.numel() == 0:
        return y
    w = weight.detach().float().contiguous() if weight is not None else None
    b = bias.detach().float().contiguous() if bias is not None else None
    _lib.check(lib.b200_rows2_to_bf16(x1.data_ptr(), c1, x2.data_ptr(), c2, y.data_ptr(), _ptr(w), _ptr(b),
                                      x1.numel() // c1, _zdtype(x1), 1 if normalize else 0, _stream()))
    return y


def pair_outer_sum(a: Tensor, c: Tensor, extra: Tensor | None = None) -> Tensor:
    """``a[:, :, None, :] + c[:, None, :, :] (+ extra)`` in fp32: ``a[B, Ni, D]``, ``c[B, Nj, D]``, ``extra[B, Ni, Nj, D]``."""
    _require_cuda(a, c)
    if a.dtype != torch.float32 or c.dtype != torch.float32 or (extra is not None and extra.dtype != torch.float32):
        raise ValueError("pair_outer_sum expects float32 tensors")
    B, ni, D = a.shape
    nj = c.shape[1]
    if c.shape != (B, nj, D) or (extra is not None and extra.shape != (B, ni, nj, D)):
        raise ValueError("shape mismatch between a, c and extra")
    a, c = a.contiguous(), c.contiguous()
    extra = extra.contiguous() if extra is not None else None
    z = torch.empty(B, ni, nj, D, dtype=torch.float32, device=a.device)
    if z.numel() == 0:
        return z
    for b in range(B):
        _lib.check(lib.b200_pair_outer_sum(a[b].data_ptr(), c[b].data_ptr(), extra[b].data_ptr() if extra is not None else None,
                                           z[b].data_ptr(), ni, nj, D, _stream()))
    return z


def add_rows(x: Tensor, y: Tensor, out: Tensor | None = None) -> Tensor:
    """``x + y`` for fp32 ``x[..., cols]`` where ``y`` (fp32 or bf16) has x's shape or only its trailing axes (it is
    then broadcast over the leading ones); ``out`` may be ``x``."""
    _require_cuda(x, y)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise ValueError("add_rows expects a contiguous float32 x")
    if tuple(x.shape[x.dim() - y.dim():]) != tuple(y.shape):
        raise ValueError(f"y {tuple(y.shape)} does not match the trailing axes of x {tuple(x.shape)}")
    y = y.contiguous()
    cols = x.shape[-1]
    if out is None:
        out = torch.empty_like(x)
    if x.numel() == 0:
        return out
    _lib.check(lib.b200_add_rows(x.data_ptr(), y.data_ptr(), out.data_ptr(), x.numel() // cols, y.numel() // cols, cols,
                                 _zdtype(y), _stream()))
    return out


class WindowApbPacked:
    """Weights of the sliding-window attention: ``proj_qkv`` with ``proj_q_bias`` folded into a GEMM bias on the q
    columns, gate and output projections in bf16, the tiny pair-bias projection in fp32."""

    def __init__(self, c_s, c_z, heads, proj_qkv, proj_q_bias, proj_g, norm_z_w, norm_z_b, proj_z, proj_o, norm_s_w, norm_s_b):
        bf = torch.bfloat16
        dh = c_s // heads
        if dh not in (16, 32, 64) or heads > 16:
            raise ValueError(f"the sliding-window kernel serves head dims 16, 32, 64 and up to 16 heads, got {dh} x {heads}")
        self.c_s, self.c_z, self.H, self.dh = c_s, c_z, heads, dh
        self.w_qkv = proj_qkv.detach().to(bf).contiguous()
        b = torch.zeros(3 * c_s, dtype=torch.float32, device=proj_qkv.device)
        b[:c_s] = proj_q_bias.detach().float()
        self.b_qkv = b
        self.w_g = proj_g.detach().to(bf).contiguous()
        self.w_o = proj_o.detach().to(bf).contiguous()
        self.w_z = proj_z.detach().float().contiguous()
        self.ln_z_w = norm_z_w.detach().float().contiguous()
        self.ln_z_b = norm_z_b.detach().float().contiguous() if norm_z_b is not None else None
        self.ln_s_w = norm_s_w.detach().float().contiguous() if norm_s_w is not None else None
        self.ln_s_b = norm_s_b.detach().float().contiguous() if norm_s_b is not None else None


def window_attention_pair_bias(s: Tensor, z: Tensor, mask: Tensor, w: WindowApbPacked, multiplicity: int = 1) -> Tensor:
    """Sliding-window attention with pair bias: ``s[B*M*NW, W, c_s]``, ``z[B, NW, W, Hk, c_z]``, ``mask[B*NW, W]``."""
    _require_cuda(s, z, mask)
    folded, W, c_s = s.shape
    B, NW, Wz, Hk, c_z = z.shape
    M = multiplicity
    if Wz != W or folded != B * M * NW or tuple(mask.shape) != (B * NW, W) or c_s != w.c_s or c_z != w.c_z:
        raise ValueError(f"inconsistent shapes: s {tuple(s.shape)}, z {tuple(z.shape)}, mask {tuple(mask.shape)}, "
                         f"multiplicity {M}")
    if s.numel() == 0:
        return torch.empty_like(s)
    sn = rows_to_bf16(s, w.ln_s_w, w.ln_s_b, normalize=w.ln_s_w is not None)
    qkv = linear_bf16(sn, w.w_qkv, bias_f32=w.b_qkv)
    gate = linear_bf16(sn, w.w_g)
    z = z.contiguous()
    bias = torch.empty(B, NW, w.H, W, Hk, dtype=torch.float32, device=s.device)
    _lib.check(lib.b200_window_bias_fwd(z.data_ptr(), w.ln_z_w.data_ptr(), _ptr(w.ln_z_b), w.w_z.data_ptr(), bias.data_ptr(),
                                        B * NW, W, Hk, c_z, w.H, _zdtype(z), _stream()))
    og = torch.empty(folded, W, c_s, dtype=torch.bfloat16, device=s.device)
    m8 = mask_u8(mask).contiguous()
    _lib.check(lib.b200_window_attention_fwd(qkv.data_ptr(), gate.data_ptr(), bias.data_ptr(), m8.data_ptr(), og.data_ptr(),
                                             B, M, NW, W, Hk, w.H, w.dh, _stream()))
    return linear_bf16(og, w.w_o, out_dtype=s.dtype)


def swiglu(h12: Tensor) -> Tensor:
    """``silu(h12[..., :H]) * h12[..., H:]`` for bf16 ``h12[..., 2H]``."""
    H = h12.shape[-1] // 2
    h12 = h12.contiguous()
    out = torch.empty(h12.shape[:-1] + (H,), dtype=torch.bfloat16, device=h12.device)
    if out.numel() == 0:
        return out
    _lib.check(lib.b200_swiglu_fwd(h12.data_ptr(), out.data_ptr(), h12.numel() // (2 * H), H, _stream()))
    return out


def adaln(x: Tensor, cond: Tensor, alpha_col: int, beta_col: int, lns: float) -> Tensor:
    """``lns * (LN(x) * (1 + alpha) + beta)`` as bf16; alpha/beta are column blocks of fp32 ``cond[rows, cw]``."""
    xd = _zdtype(x)
    x = x.contiguous()
    cols = x.shape[-1]
    y = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    if y.numel() == 0:
        return y
    _lib.check(lib.b200_adaln_fwd(x.data_ptr(), cond.data_ptr(), cond.shape[-1], alpha_col, beta_col, float(lns),
                                  y.data_ptr(), x.numel() // cols, cols, xd, _stream()))
    return y


def gated_residual_(x: Tensor, h: Tensor, cond: Tensor, gamma_col: int) -> Tensor:
    """``x += gamma * h`` in place (gamma a column block of fp32 ``cond``); returns ``x``."""
    if not x.is_contiguous() or not h.is_contiguous():
        raise ValueError("gated_residual_ needs contiguous tensors")
    cols = x.shape[-1]
    if x.numel() == 0:
        return x
    _lib.check(lib.b200_gated_residual_fwd(x.data_ptr(), h.data_ptr(), cond.data_ptr(), cond.shape[-1], gamma_col,
                                           x.numel() // cols, cols, _zdtype(x), _zdtype(h), _stream()))
    return x


class TransitionGenericPacked:
    """Weights of a SwiGLU transition of any width (multiples of 8): ``w12 = [fc1; fc2]``, ``w3``."""

    def __init__(self, norm_w, norm_b, fc1, fc2, fc3):
        bf = torch.bfloat16
        self.w12 = torch.cat([fc1.detach(), fc2.detach()], dim=0).to(bf).contiguous()
        self.w3 = fc3.detach().to(bf).contiguous()
        self.norm_w, self.norm_b = norm_w, norm_b
        if fc1.shape[0] % 8 or fc1.shape[1] % 8 or fc3.shape[0] % 8 or fc1.shape[1] > 1024:
            raise ValueError("transition widths must be multiples of 8 and the input width at most 1024")


def transition_generic(x: Tensor, w: TransitionGenericPacked, add_residual: bool = False,
                       out: Tensor | None = None) -> Tensor:
    """Un-fused transition for the single track: LayerNorm/convert, fc1|fc2 GEMM, SwiGLU, fc3 GEMM (+ residual)."""
    _require_cuda(x)
    x = x.contiguous()
    xb = x if (x.dtype == torch.bfloat16 and w.norm_w is None) else rows_to_bf16(
        x, w.norm_w, w.norm_b, normalize=w.norm_w is not None)
    h = swiglu(linear_bf16(xb, w.w12))
    same_width = w.w3.shape[0] == x.shape[-1]
    if add_residual and not same_width:
        raise ValueError("the residual needs out_dim == dim")
    return linear_bf16(h, w.w3, residual=x if add_residual else None, out_dtype=x.dtype, out=out)


def attention_core(q: Tensor, k: Tensor, v: Tensor, bias: Tensor, key_mask: Tensor, gate: Tensor | None = None,
                   bias_div: int = 1, mask_div: int = 1) -> Tensor:
    """softmax(q.k/sqrt(dh) + bias, masked keys -> -1e6) v [* sigmoid(gate)] on the tcgen05 flash kernel.

    ``q, k, v, gate``: ``[batch, N, H, dh]`` (dh a multiple of 8, <= 64); ``bias``: ``[groups, H, N, N]`` (natural-log
    units); ``key_mask``: ``[batch // mask_div, N]``.  Returns bf16 ``[batch, N, H, dh]``.  The operand re-layout
    (head padding, scaling, V transposition) done here with torch ops is what the fused projection kernels of
    ``attention_pair_bias`` / ``triangle_attention`` produce directly; this entry serves tests and benchmarks.
    """
    _require_cuda(q, k, v, bias, key_mask)
    Bt, N, H, dh = q.shape
    DH = 32 if dh <= 32 else 64
    bf = torch.bfloat16
    qk = torch.zeros(Bt, N, 2 * H * DH, dtype=bf, device=q.device)
    qk.view(Bt, N, 2, H, DH)[:, :, 0, :, :dh] = (q.float() * (LOG2E / dh ** 0.5)).to(bf)
    qk.view(Bt, N, 2, H, DH)[:, :, 1, :, :dh] = k.to(bf)
    Nk = (N + 7) // 8 * 8
    vT = torch.zeros(Bt, H * DH, Nk, dtype=bf, device=q.device)
    vT.view(Bt, H, DH, Nk)[:, :, :dh, :N] = v.to(bf).permute(0, 2, 3, 1)
    groups = bias.shape[0]
    b2 = torch.zeros(groups * H, N, Nk, dtype=bf, device=q.device)
    b2[:, :, :N] = (bias.float() * LOG2E).to(bf).reshape(groups * H, N, N)
    out = torch.empty(Bt, N, H * dh, dtype=bf, device=q.device)
    g = gate.to(bf).reshape(Bt, N, H * dh).contiguous() if gate is not None else None
    m8 = mask_u8(key_mask)
    a = _lib.AttentionCoreArgs(
        qk.data_ptr(), 2 * H * DH, N * 2 * H * DH, 0, H * DH, vT.data_ptr(), Nk, b2.data_ptr(), Nk, groups, bias_div,
        m8.data_ptr(), mask_div, N, 1, _ptr(g), N * H * dh, H * dh, 0, out.data_ptr(), N * H * dh, H * dh, 0, DH, dh,
        N, H, Bt)
    _lib.check(lib.b200_attention_core_fwd(ctypes.byref(a), _stream()))
    return out.view(Bt, N, H, dh)


# ----------------------------------------------------------------------------------- staged triangle multiplication
def pad128(n: int) -> int:
    return (n + 127) // 128 * 128


def trimul_project(z_slab: Tensor, mask_slab: Tensor, w: TriMulPacked, incoming: bool) -> tuple[Tensor, Tensor]:
    """Projection stage on a slab ``z[n_rows, n_cols, 128]``: returns ``a, b`` as bf16 ``[128, lines, pos_pitch]``
    with (line, pos) = (row, col) for outgoing and (col, row) for incoming, zero-padded in ``pos``."""
    _require_cuda(z_slab, mask_slab)
    zd = _zdtype(z_slab)
    z_slab = z_slab.contiguous()
    n_rows, n_cols = z_slab.shape[0], z_slab.shape[1]
    lines, pos = (n_cols, n_rows) if incoming else (n_rows, n_cols)
    pitch = pad128(pos)
    a = torch.empty(128, lines, pitch, dtype=torch.bfloat16, device=z_slab.device)
    b = torch.empty_like(a)
    m8 = mask_u8(mask_slab)
    _lib.check(lib.b200_trimul_project(z_slab.data_ptr(), m8.data_ptr(), a.data_ptr(), b.data_ptr(), ctypes.byref(w.struct),
                                       n_rows, n_cols, n_cols * 128, n_cols, 1 if incoming else 0, pitch, zd, _stream()))
    return a, b


def trimul_output_(z_slab: Tensor, t: Tensor, w: TriMulPacked, transposed_t: bool, add_residual: bool = True) -> Tensor:
    """Output stage on the slab, in place: ``z (+)= p_out(LN(t)) * sigmoid(g_out(LN(z)))`` with ``t`` bf16
    ``[128, lines, pos_pitch]``."""
    zd = _zdtype(z_slab)
    if not z_slab.is_contiguous() or t.dtype != torch.bfloat16 or not t.is_contiguous():
        raise ValueError("trimul_output_ needs a contiguous slab and a contiguous bf16 t")
    n_rows, n_cols = z_slab.shape[0], z_slab.shape[1]
    _lib.check(lib.b200_trimul_output(t.data_ptr(), z_slab.data_ptr(), z_slab.data_ptr(), ctypes.byref(w.struct), n_rows,
                                      n_cols, n_cols * 128, 1 if transposed_t else 0, t.shape[2], 1 if add_residual else 0,
                                      zd, _stream()))
    return z_slab


def bmm_nt_into(a: Tensor, b: Tensor, out: Tensor, scale: float = 1.0) -> Tensor:
    """``out[n] = scale * a[n] @ b[n].T`` for bf16 ``a[batch, M, K]``, ``b[batch, N, K]`` given as (possibly strided in
    batch and row) views with unit stride in K; ``out[batch, M, N]`` bf16 or fp32, unit stride in N."""
    if a.stride(2) != 1 or b.stride(2) != 1 or out.stride(2) != 1:
        raise ValueError("bmm_nt_into needs unit stride along the last axis")
    batch, M, K = a.shape
    N = b.shape[1]
    _lib.check(lib.b200_bmm_nt(a.data_ptr(), b.data_ptr(), out.data_ptr(), batch, M, N, K, a.stride(1), b.stride(1),
                               out.stride(1), a.stride(0), b.stride(0), out.stride(0), scale, _zdtype(out), _stream()))
    return out


# ----------------------------------------------------------------------------------- pieces for sharded attention
def pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def pair_bias_slab(z_slab: Tensor, ln_w: Tensor, ln_b: Tensor | None, w_z_bf16: Tensor, H: int,
                   transposed: bool = False, out: Tensor | None = None) -> Tensor:
    """``log2(e) * proj(LN(z))`` on a slab ``z[n_rows, n_cols, 128]`` -> bf16 ``[H, lines, pad8(pos)]`` with
    (line, pos) = (row, col), or (col, row) when ``transposed``.  ``out``: a buffer of that shape to write into (its
    padding columns must already be zero)."""
    _require_cuda(z_slab)
    zd = _zdtype(z_slab)
    z_slab = z_slab.contiguous()
    n_rows, n_cols = z_slab.shape[0], z_slab.shape[1]
    lines, pos = (n_cols, n_rows) if transposed else (n_rows, n_cols)
    if out is None:
        out = torch.zeros(H, lines, pad8(pos), dtype=torch.bfloat16, device=z_slab.device)
    elif tuple(out.shape) != (H, lines, pad8(pos)) or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("out must be a contiguous bf16 [H, lines, pad8(pos)] buffer")
    _lib.check(lib.b200_pair_bias_fwd(z_slab.data_ptr(), ln_w.data_ptr(), _ptr(ln_b), w_z_bf16.data_ptr(), out.data_ptr(),
                                      n_rows, n_cols, n_cols * 128, lines * pad8(pos), pad8(pos), H,
                                      1 if transposed else 0, zd, _stream()))
    return out


def attention_pair_bias_with_bias(s: Tensor, bias: Tensor, mask: Tensor, w: ApbPacked, multiplicity: int = 1) -> Tensor:
    """Pair-bias attention with a precomputed bias ``[B, H, N, pitch]`` (bf16, log2(e)-scaled, see ``pair_bias_slab``)."""
    _require_cuda(s, bias, mask)
    B, N = mask.shape
    if s.shape[0] != B * multiplicity or s.shape[1] != N or s.shape[2] != w.c_s:
        raise ValueError(f"{tuple(s.shape)}, mask {tuple(mask.shape)}, multiplicity={multiplicity}")
    if bias.dtype != torch.bfloat16 or tuple(bias.shape[:3]) != (B, w.H, N) or not bias.is_contiguous():
        raise ValueError(f"bias must be contiguous bf16 [B, H, N, pitch], got {tuple(bias.shape)}")
    sd = _zdtype(s)
    s = s.contiguous()
    out = torch.empty_like(s)
    m8 = mask_u8(mask)
    nbytes = lib.b200_apb_workspace_bytes(B, multiplicity, N, w.c_s, w.H)
    ws = workspace(nbytes, s.device)
    _lib.check(lib.b200_apb_fwd_bias(s.data_ptr(), bias.data_ptr(), bias.shape[3], m8.data_ptr(), out.data_ptr(),
                                     ctypes.byref(w.struct), B, multiplicity, N, w.c_s, w.H, sd, ws.data_ptr(), nbytes,
                                     _stream()))
    return out


def triangle_attention_slab(z_slab: Tensor, mask_slab: Tensor, bias: Tensor, w: TriAttPacked, ending: bool,
                            add_residual: bool = False) -> Tensor:
    """Triangle attention for the complete attention rows held in ``z_slab[n_rows, n_cols, 128]`` (all columns for the
    starting node, all rows for the ending node), with the whole tensor's triangle bias ``[4, tokens, pitch]``."""
    _require_cuda(z_slab, mask_slab, bias)
    zd = _zdtype(z_slab)
    z_slab = z_slab.contiguous()
    n_rows, n_cols = z_slab.shape[0], z_slab.shape[1]
    out = torch.empty_like(z_slab)
    m8 = mask_u8(mask_slab)
    nbytes = lib.b200_triatt_slab_workspace_bytes(n_rows, n_cols, 1 if ending else 0)
    ws = workspace(nbytes, z_slab.device)
    _lib.check(lib.b200_triatt_slab_fwd(z_slab.data_ptr(), m8.data_ptr(), bias.data_ptr(), bias.shape[2], out.data_ptr(),
                                        ctypes.byref(w.struct), n_rows, n_cols, 1 if ending else 0,
                                        1 if add_residual else 0, zd, ws.data_ptr(), nbytes, _stream()))
    return out


def outer_product_mean_cols(m: Tensor, mask: Tensor, w: OpmPacked, j0: int, nj: int, inv_count: Tensor,
                            add_bias: bool) -> Tensor:
    """Partial outer product mean over the MSA rows in ``m[S, N, 64]`` for output columns ``j0 .. j0+nj``: fp32
    ``[N, nj, 128]`` scaled by the device scalar ``inv_count`` (fp32, 1 element)."""
    _require_cuda(m, mask, inv_count)
    S, N, _ = m.shape
    zd = _zdtype(m)
    m = m.contiguous()
    out = torch.empty(N, nj, 128, dtype=torch.float32, device=m.device)
    m8 = mask_u8(mask)
    nbytes = lib.b200_opm_workspace_bytes(S, N)
    ws = workspace(nbytes, m.device)
    _lib.check(lib.b200_opm_cols_fwd(m.data_ptr(), m8.data_ptr(), out.data_ptr(), ctypes.byref(w.struct), S, N, j0, nj,
                                     inv_count.data_ptr(), 1 if add_bias else 0, zd, _lib.DTYPE_F32, ws.data_ptr(), nbytes,
                                     _stream()))
    return out


# ----------------------------------------------------------------------------------- pair-weighted averaging
class PwaPacked:
    """Weights of pair-weighted averaging (heads of 32 channels, c_z = 128) in kernel layouts."""

    def __init__(self, norm_m_w, norm_m_b, norm_z_w, norm_z_b, proj_m, proj_g, proj_z, proj_o, num_heads: int):
        H = num_heads
        if proj_m.shape[0] != 32 * H or proj_z.shape[1] != 128 or H > 16 or proj_m.shape[1] % 8:
            raise ValueError("pair-weighted averaging is built for heads of 32 channels, at most 16 heads, c_z = 128")
        bf = torch.bfloat16
        self.H, self.c_m = H, proj_m.shape[1]
        self.w_m = proj_m.detach().to(bf).contiguous()          # [H*32, c_m]: rows h*32 .. h*32+31 are head h
        self.w_g = proj_g.detach().to(bf).contiguous()
        self.w_o = proj_o.detach().to(bf).contiguous()          # [c_m, H*32]
        wz = torch.zeros(16, 128, dtype=torch.float32, device=proj_z.device)
        wz[:H] = proj_z.detach().float()
        self.w_z = wz.to(bf).contiguous()
        self.ln_m = (norm_m_w.detach().float().contiguous(), norm_m_b.detach().float().contiguous())
        self.ln_z_w = norm_z_w.detach().float().contiguous()
        self.ln_z_b = norm_z_b.detach().float().contiguous() if norm_z_b is not None else None


def pair_weighted_averaging(m: Tensor, z: Tensor, mask: Tensor, w: PwaPacked, add_residual: bool = False) -> Tensor:
    """``m[B,S,N,c_m]``, ``z[B,N,N,128]``, ``mask[B,N,N]`` -> update ``[B,S,N,c_m]`` (plus ``m`` when ``add_residual``).

    Per batch item: ``norm_m`` and the gate / value projections of the MSA rows, the per-head weights
    ``softmax_j(proj_z(norm_z(z))[i,j,h])`` with masked pairs at -1e6, the per-head product ``w_h . v_h^T`` on the tensor
    cores (``v_h^T`` is written transposed by its projection GEMM, so both operands are K-major), gating, ``proj_o``.
    """
    _require_cuda(m, z, mask)
    if m.ndim != 4 or z.ndim != 4 or tuple(z.shape[1:]) != (m.shape[2], m.shape[2], 128) or z.shape[0] != m.shape[0]:
        raise ValueError(f"expected m[B,S,N,c_m] and z[B,N,N,128], got {tuple(m.shape)}, {tuple(z.shape)}")
    if tuple(mask.shape) != tuple(z.shape[:3]):
        raise ValueError(f"mask shape {tuple(mask.shape)} does not match z {tuple(z.shape)}")
    B, S, N, c_m = m.shape
    if c_m != w.c_m:
        raise ValueError(f"m has {c_m} channels, the module was built for {w.c_m}")
    m = m.contiguous()
    m8 = mask_u8(mask)
    out = torch.empty_like(m)
    if out.numel() == 0:
        return out
    for b in range(B):
        mn = pwa_norm(m[b], w)
        logits = pair_bias_slab(z[b], w.ln_z_w, w.ln_z_b, w.w_z, w.H)                               # [H, N, Nk], base 2
        pwa_apply(mn, mn, logits, m8[b], w, m[b] if add_residual else None, out[b])
    return out


def pwa_norm(m: Tensor, w: PwaPacked) -> Tensor:
    """``norm_m`` of MSA rows ``m[S, n, c_m]`` as bf16."""
    return rows_to_bf16(m.contiguous(), w.ln_m[0], w.ln_m[1], normalize=True)


def pwa_apply(mn_all: Tensor, mn_own: Tensor, logits: Tensor, mask8: Tensor, w: PwaPacked, residual: Tensor | None,
              out: Tensor) -> Tensor:
    """The averaging itself for the token rows ``i`` a caller owns: ``mn_all[S, N, c_m]`` (normalised MSA, every token:
    the values), ``mn_own[S, n_i, c_m]`` (the same for the owned tokens: the gate), ``logits[H, n_i, pad8(N)]`` (base-2
    pair-bias logits of the owned rows), ``mask8[n_i, N]`` -> ``out[S, n_i, c_m]`` (plus ``residual``).  Single GPU:
    ``n_i = N`` and the two MSA tensors are the same object; a rank of a context-parallel grid owns a block of tokens."""
    S, N, c_m = mn_all.shape
    n_i = mn_own.shape[1]
    H, Nk = w.H, pad8(N)
    bf = torch.bfloat16
    if tuple(logits.shape) != (H, n_i, Nk) or tuple(mask8.shape) != (n_i, N) or tuple(out.shape) != (S, n_i, c_m):
        raise ValueError(f"inconsistent shapes: logits {tuple(logits.shape)}, mask {tuple(mask8.shape)}, out {tuple(out.shape)}")
    mn_p = mn_all
    if N != Nk:   # the token axis is the GEMM's column count, which the kernel wants in multiples of 8
        mn_p = torch.zeros(S, Nk, c_m, dtype=bf, device=mn_all.device)
        mn_p[:, :N] = mn_all
    vT = torch.empty(H, S * 32, Nk, dtype=bf, device=mn_all.device)                                # [h][(s, d)][j]
    for h in range(H):   # v_h^T[s] = W_m[h] . mn[s]^T : one A for all S batch items
        bmm_nt_into(w.w_m[h * 32:(h + 1) * 32].unsqueeze(0).expand(S, 32, c_m), mn_p, vT[h].view(S, 32, Nk))
    wts = torch.empty_like(logits)
    _lib.check(lib.b200_masked_softmax_rows(logits.data_ptr(), mask8.contiguous().data_ptr(), wts.data_ptr(), H, n_i, N, Nk,
                                            _stream()))
    o = torch.empty(H, n_i, S * 32, dtype=bf, device=mn_all.device)
    bmm_nt_into(wts, vT, o)                                                                        # o[h][i][(s, d)]
    g = linear_bf16(mn_own.contiguous().view(S * n_i, c_m), w.w_g)                                 # [S*n_i, H*32]
    og = torch.empty(S * n_i, H * 32, dtype=bf, device=mn_all.device)
    _lib.check(lib.b200_pwa_gate(o.data_ptr(), g.data_ptr(), og.data_ptr(), S, n_i, H, _stream()))
    linear_bf16(og, w.w_o, residual=residual.view(S * n_i, c_m) if residual is not None else None, out_dtype=out.dtype,
                out=out.view(S * n_i, c_m))
    return out
