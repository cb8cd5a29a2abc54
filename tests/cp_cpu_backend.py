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
