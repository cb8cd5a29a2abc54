"""A CPU stand-in for the four local steps of context-parallel triangle multiplication, built from the oracle's
primitives.  TEST INFRASTRUCTURE: it lets the exchange pattern and the index arithmetic of
``bioemu2_b200.context_parallel`` run as gloo ranks on a machine without a GPU."""
from __future__ import annotations

import torch

from oracle import pair_ops as O


class OracleWeights:
    """Plays the role of the packed-weights object: just the state dict."""

    def __init__(self, w: dict, mode: str):
        self.w = w
        self.mode = mode


class CpuTriMulBackend:
    def project(self, z_slab, mask_slab, packed, incoming):
        w = packed.w
        h = O.layer_norm(z_slab, w["norm_in.weight"], w["norm_in.bias"])
        proj = O.linear(h, w["p_in.weight"]) * torch.sigmoid(O.linear(h, w["g_in.weight"]))
        proj = torch.where(mask_slab.bool().unsqueeze(-1), proj, torch.zeros_like(proj))
        a, b = proj.chunk(2, dim=-1)  # [n_r, n_c, D]
        perm = (2, 1, 0) if incoming else (2, 0, 1)  # -> [D, lines, pos]
        out = []
        for t in (a, b):
            t = t.permute(*perm)
            pitch = (t.shape[2] + 127) // 128 * 128
            buf = torch.zeros(t.shape[0], t.shape[1], pitch, dtype=t.dtype)
            buf[:, :, :t.shape[2]] = t
            out.append(buf)
        return out[0], out[1]

    def contract_into(self, lhs, rhs_rows, out):
        out.copy_(torch.einsum("dik,djk->dij", lhs, rhs_rows))

    def empty_partial(self, shape, device):
        return torch.full(shape, float("nan"), dtype=torch.float64)  # NaN: nothing may depend on unwritten padding

    def to_operand(self, t):
        return t

    def output_(self, z_slab, t, packed, transposed):
        w = packed.w
        n_r, n_c = z_slab.shape[0], z_slab.shape[1]
        tt = t[:, :n_c, :n_r].permute(2, 1, 0) if transposed else t[:, :n_r, :n_c].permute(1, 2, 0)
        h = O.layer_norm(z_slab, w["norm_in.weight"], w["norm_in.bias"])
        upd = O.linear(O.layer_norm(tt, w["norm_out.weight"], w["norm_out.bias"]), w["p_out.weight"])
        z_slab += upd * torch.sigmoid(O.linear(h, w["g_out.weight"]))

    def check_block(self, n_rows, n_cols):
        pass


class Packed:
    """Stand-in for a packed-weights object on CPU: the state dict and the head count."""

    def __init__(self, w: dict, H: int = 0):
        self.w = w
        self.H = H


def _pad_last(t: torch.Tensor) -> torch.Tensor:
    pitch = (t.shape[-1] + 7) // 8 * 8
    out = t.new_zeros(t.shape[:-1] + (pitch,))
    out[..., :t.shape[-1]] = t
    return out


class CpuAttentionLocal:
    """Oracle-backed local steps of the context-parallel attention ops (biases in natural-log units)."""

    def pair_bias(self, z_slab, packed):
        w = packed.w
        zb = O.linear(O.layer_norm(z_slab, w["norm_z.weight"], w.get("norm_z.bias")), w["proj_z.weight"])
        return _pad_last(zb.permute(2, 0, 1))

    def attention(self, s_full, bias_full, mask_full, packed, multiplicity):
        n = s_full.shape[1]
        return O.attention_pair_bias(s_full, None, mask_full, packed.w, packed.H, multiplicity, bias=bias_full[..., :n])

    def tri_bias(self, z_slab, packed, ending):
        w = packed.w
        tb = O.linear(O.layer_norm(z_slab, w["layer_norm.weight"], w["layer_norm.bias"]), w["linear_b.weight"])
        return _pad_last(tb.permute(2, 1, 0) if ending else tb.permute(2, 0, 1))

    def tri_slab(self, slab, mask_slab, bias_full, packed, ending):
        import math

        w = packed.w
        x, m = (slab.transpose(0, 1), mask_slab.transpose(0, 1)) if ending else (slab, mask_slab)  # [lines, N, D]
        L, N, _ = x.shape
        H, dh = 4, w["linear_q.weight"].shape[0] // 4
        h = O.layer_norm(x, w["layer_norm.weight"], w["layer_norm.bias"])
        q = O.linear(h, w["linear_q.weight"]).view(L, N, H, dh)
        k = O.linear(h, w["linear_k.weight"]).view(L, N, H, dh)
        v = O.linear(h, w["linear_v.weight"]).view(L, N, H, dh)
        g = torch.sigmoid(O.linear(h, w["linear_g.weight"], w["linear_g.bias"]))
        logits = torch.einsum("ijhd,ikhd->ihjk", q, k) / math.sqrt(dh) + bias_full[None, :, :, :N]
        logits = torch.where(m.bool().view(L, 1, 1, N), logits, torch.full_like(logits, -1e6))
        o = torch.einsum("ihjk,ikhd->ijhd", logits.softmax(-1), v).reshape(L, N, H * dh)
        out = O.linear(g * o, w["linear_o.weight"])
        return out.transpose(0, 1) if ending else out

    def opm_partial(self, m_rows, mask_rows, packed, j0, nj, inv_count, add_bias):
        w = packed.w
        mp = O.linear(O.layer_norm(m_rows, w["norm.weight"], w["norm.bias"]), w["proj_ab.weight"])
        mp = torch.where(mask_rows.bool().unsqueeze(-1), mp, torch.zeros_like(mp))
        a, b = mp.chunk(2, dim=-1)
        z = torch.einsum("sic,sjd->ijcd", a, b[:, j0:j0 + nj]).reshape(a.shape[1], nj, -1) * inv_count.to(m_rows.dtype)
        return O.linear(z, w["proj_o.weight"], w["proj_o.bias"] if add_bias else None)

    # ---- pair-weighted averaging (logits in natural-log units here; the GPU path carries them in base-2 units)
    def pwa_logits(self, z_slab, packed):
        w = packed.w
        zb = O.linear(O.layer_norm(z_slab, w["norm_z.weight"], w.get("norm_z.bias")), w["proj_z.weight"])
        return _pad_last(zb.permute(2, 0, 1))

    def pwa_norm(self, m_loc, packed):
        return O.layer_norm(m_loc, packed.w["norm_m.weight"], packed.w["norm_m.bias"])

    def pwa_apply(self, mn_all, mn_own, logits, mask_rows, packed, residual):
        w, H = packed.w, packed.H
        S, n, _ = mn_all.shape
        n_i = mn_own.shape[1]
        v = O.linear(mn_all, w["proj_m.weight"]).view(S, n, H, -1)
        b = torch.where(mask_rows.bool()[None], logits[:, :, :n], torch.full_like(logits[:, :, :n], -1e6))
        o = torch.einsum("hij,sjhd->sihd", b.softmax(dim=-1), v).reshape(S, n_i, -1)
        out = O.linear(torch.sigmoid(O.linear(mn_own, w["proj_g.weight"])) * o, w["proj_o.weight"])
        return out + residual if residual is not None else out

