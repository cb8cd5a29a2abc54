"""Definitions of the golden cases: how inputs and weights are drawn from a seed.

Shared by ``make_golden.py`` (which runs the reference's own modules on them)
and by the tests (which re-draw the same tensors and compare against the
stored outputs).  A checksum of every drawn tensor is stored beside the output
so that a change in the RNG stream is reported instead of silently comparing
against the wrong inputs.
"""
from __future__ import annotations

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import helpers as H  # noqa: E402

GOLDEN_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_fp32.pt")


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def checksum(tensors) -> float:
    tot = 0.0
    for t in tensors:
        t = t.double().flatten()
        idx = torch.arange(1, t.numel() + 1, dtype=torch.float64)
        tot += float((t * torch.cos(idx)).sum())
    return tot


def trimul_case(mode: str, seed: int = 11, B: int = 2, N: int = 24, D: int = 128):
    g = _gen(seed)
    w = H.trimul_weights(g, D)
    x = torch.randn(B, N, N, D, generator=g)
    mask = torch.rand(B, N, N, generator=g) > 0.25
    return dict(kind="trimul", mode=mode, w=w, x=x, mask=mask)


def transition_case(seed: int = 12, shape=(2, 24, 24, 128), hidden: int = 512, use_norm: bool = True):
    g = _gen(seed)
    w = H.transition_weights(g, shape[-1], hidden, use_norm)
    x = torch.randn(*shape, generator=g)
    return dict(kind="transition", w=w, x=x, hidden=hidden, use_norm=use_norm)


def apb_case(seed: int = 13, B: int = 2, M: int = 1, N: int = 24, c_s: int = 384, c_z: int = 128,
             heads: int = 16, initial_norm: bool = True):
    g = _gen(seed)
    w = H.apb_weights(g, c_s, c_z, heads, initial_norm)
    s = torch.randn(B * M, N, c_s, generator=g)
    z = torch.randn(B, N, N, c_z, generator=g)
    mask = torch.ones(B, N, dtype=torch.bool)
    mask[0, N - 5:] = False
    mask[B - 1, 3] = False
    return dict(kind="apb", w=w, s=s, z=z, mask=mask, heads=heads, M=M, initial_norm=initial_norm)


def opm_case(seed: int = 14, B: int = 2, S: int = 40, N: int = 24, c_in: int = 64, c_hidden: int = 32,
             c_out: int = 128, mask_2d: bool = False):
    g = _gen(seed)
    w = H.opm_weights(g, c_in, c_hidden, c_out)
    m = torch.randn(B, S, N, c_in, generator=g)
    if mask_2d:
        # A [B, N] mask only broadcasts against m[B, S, N, C] when B == 1
        # (src/bioemu2/biomoa/ops/outer_product_mean.py:62); the divisor is then 1.
        assert B == 1
        mask = torch.rand(B, N, generator=g) > 0.2
    else:
        rows = torch.rand(B, S, generator=g) > 0.1
        mask = rows[:, :, None].expand(B, S, N).clone()
        mask[:, 1, -3:] = False  # a partially padded row, as the reference's tests use
        mask[0, :, -2:] = False  # padded tokens
    return dict(kind="opm", w=w, m=m, mask=mask, c_hidden=c_hidden, c_out=c_out)


def pairmixer_case(seed: int = 15, N: int = 24, D: int = 128):
    g = _gen(seed)
    w = H.pairmixer_layer_weights(g, D)
    z = torch.randn(1, N, N, D, generator=g)
    tok = torch.ones(1, N, dtype=torch.bool)
    tok[0, N - 3:] = False
    pair_mask = tok[:, :, None] & tok[:, None, :]
    return dict(kind="pairmixer", w=w, z=z, pair_mask=pair_mask)


def cond_layer_case(seed: int = 16, B: int = 1, M: int = 2, N: int = 24, dim: int = 384, dim_pair: int = 128,
                    dim_cond: int = 384, heads: int = 16, hidden: int = 768):
    g = _gen(seed)
    w = {}
    w["cond.0.weight"], w["cond.0.bias"] = H.ln_params(g, dim_cond)
    w["cond.2.weight"] = H.kaiming_linear(g, 6 * dim, dim_cond)
    w["cond.2.bias"] = 0.05 * torch.randn(6 * dim, generator=g)
    w.update(H.prefixed("attention.pair_bias_attn", H.apb_weights(g, dim, dim_pair, heads, initial_norm=False)))
    w.update(H.prefixed("transition", H.transition_weights(g, dim, hidden, use_norm=False)))
    x = torch.randn(B * M, N, dim, generator=g)
    c = torch.randn(B * M, N, dim_cond, generator=g)
    z = torch.randn(B, N, N, dim_pair, generator=g)
    mask = torch.ones(B, N, dtype=torch.bool)
    mask[0, N - 4:] = False
    return dict(kind="cond_layer", w=w, x=x, c=c, z=z, mask=mask, heads=heads, M=M, hidden=hidden,
                lns_scale=0.5)


def cond_layer_window_case(seed: int = 30, B: int = 1, M: int = 2, NW: int = 3, W: int = 32, Hk: int = 128,
                           dim: int = 128, dim_pair: int = 16, dim_cond: int = 128, heads: int = 4, hidden: int = 256):
    """The atom transformer's block: ``ConditionedTransformerLayer(is_sliding_window=True)``."""
    g = _gen(seed)
    N = NW * W
    w = {}
    w["cond.0.weight"], w["cond.0.bias"] = H.ln_params(g, dim_cond)
    w["cond.2.weight"] = H.kaiming_linear(g, 6 * dim, dim_cond)
    w["cond.2.bias"] = 0.05 * torch.randn(6 * dim, generator=g)
    w.update(H.prefixed("attention.attention_layer.pair_bias_attn", H.apb_weights(g, dim, dim_pair, heads, initial_norm=False)))
    w.update(H.prefixed("transition", H.transition_weights(g, dim, hidden, use_norm=False)))
    x = torch.randn(B * M, N, dim, generator=g)
    c = torch.randn(B * M, N, dim_cond, generator=g)
    z = torch.randn(B, NW, W, Hk, dim_pair, generator=g)
    mask = torch.ones(B, N, dtype=torch.bool)
    mask[0, N - 13:] = False
    return dict(kind="cond_layer", w=w, x=x, c=c, z=z, mask=mask, heads=heads, M=M, hidden=hidden, lns_scale=0.5,
                window=(W, Hk))


def pwa_case(seed: int = 17, B: int = 2, S: int = 10, N: int = 24, c_m: int = 64, c_z: int = 128):
    g = _gen(seed)
    w = H.pwa_weights(g, c_m, c_z, 32, 8)
    m = torch.randn(B, S, N, c_m, generator=g)
    z = torch.randn(B, N, N, c_z, generator=g)
    tok = torch.ones(B, N, dtype=torch.bool)
    tok[0, N - 4:] = False
    mask = tok[:, :, None] & tok[:, None, :]
    return dict(kind="pwa", w=w, m=m, z=z, mask=mask)


def msa_layer_case(seed: int = 18, S: int = 12, N: int = 24):
    g = _gen(seed)
    w = H.msa_layer_weights(g)
    m = torch.randn(1, S, N, 64, generator=g)
    z = torch.randn(1, N, N, 128, generator=g)
    tok = torch.ones(1, N, dtype=torch.bool)
    tok[0, N - 3:] = False
    pair_mask = tok[:, :, None] & tok[:, None, :]
    msa_mask = tok[:, None, :].expand(1, S, N).clone()
    msa_mask[0, 2] = False
    return dict(kind="msa_layer", w=w, m=m, z=z, pair_mask=pair_mask, msa_mask=msa_mask)


def pairwise_conditioning_case(seed: int = 19, N: int = 24):
    g = _gen(seed)
    w = H.pairwise_conditioning_weights(g)
    z = torch.randn(1, N, N, 128, generator=g)
    rel = torch.randn(1, N, N, 128, generator=g)
    return dict(kind="pairwise_conditioning", w=w, z=z, rel=rel)


def msa_feats(g: torch.Generator, S: int, N: int, n_pad: int) -> dict:
    """Seeded stand-ins for the MSA features of the reference's feature dict (one-hot rows, 0/1 flags, a real value)."""
    tok = torch.ones(1, N, dtype=torch.bool)
    tok[0, N - n_pad:] = False
    msa = torch.nn.functional.one_hot(torch.randint(0, 33, (1, S, N), generator=g), 33).float()
    msa_mask = tok[:, None, :].expand(1, S, N).clone()
    msa_mask[0, S - 1, : N // 2] = False
    return dict(msa=msa, msa_mask=msa_mask,
                has_deletion=(torch.rand(1, S, N, generator=g) < 0.2).float(),
                deletion_value=torch.rand(1, S, N, generator=g),
                msa_paired=(torch.rand(1, S, N, generator=g) < 0.5).float(),
                token_pad_mask=tok)


def msa_module_case(seed: int = 20, S: int = 10, N: int = 24, s_input_dim: int = 100, blocks: int = 2):
    g = _gen(seed)
    w = H.msa_module_weights(g, s_input_dim, blocks)
    z = torch.randn(1, N, N, 128, generator=g)
    emb = torch.randn(1, N, s_input_dim, generator=g)
    return dict(kind="msa_module", w=w, z=z, emb=emb, feats=msa_feats(g, S, N, 3), blocks=blocks)


def sequence_trunk_case(seed: int = 26, S: int = 8, N: int = 24, s_input_dim: int = 100, unconditional: bool = False):
    g = _gen(seed)
    w = H.sequence_trunk_weights(g, s_input_dim, msa_blocks=1, num_blocks=1)
    s_inputs = torch.randn(1, N, s_input_dim, generator=g)
    pair_terms = torch.randn(1, N, N, 128, generator=g)
    return dict(kind="sequence_trunk", w=w, s_inputs=s_inputs, pair_terms=pair_terms, feats=msa_feats(g, S, N, 2),
                recycles=1, msa_blocks=1, num_blocks=1, unconditional=unconditional)


def window_apb_case(seed: int = 28, B: int = 1, M: int = 2, NW: int = 3, W: int = 32, Hk: int = 128, c_s: int = 128,
                    c_z: int = 16, heads: int = 4, n_pad: int = 9):
    g = _gen(seed)
    w = H.apb_weights(g, c_s, c_z, heads, True)
    s = torch.randn(B * M * NW, W, c_s, generator=g)
    z = torch.randn(B, NW, W, Hk, c_z, generator=g)
    mask = torch.ones(B, NW * W, dtype=torch.bool)
    mask[:, NW * W - n_pad:] = False
    mask[0, 40] = False
    return dict(kind="window_apb", w=w, s=s, z=z, mask=mask.reshape(B * NW, W), heads=heads, M=M, W=W, Hk=Hk)


CASES = {
    "trimul_outgoing": lambda: trimul_case("outgoing"),
    "trimul_incoming": lambda: trimul_case("incoming", seed=21),
    "transition_pair": lambda: transition_case(),
    "transition_single_nonorm": lambda: transition_case(seed=22, shape=(2, 24, 384), hidden=1536, use_norm=False),
    "apb": lambda: apb_case(),
    "apb_multiplicity": lambda: apb_case(seed=23, B=2, M=3),
    "apb_nonorm_dh48": lambda: apb_case(seed=24, B=1, M=2, c_s=768, heads=16, initial_norm=False),
    "opm": lambda: opm_case(),
    "opm_mask2d": lambda: opm_case(seed=25, B=1, S=3, mask_2d=True),
    "pairmixer_layer": lambda: pairmixer_case(),
    "cond_layer": lambda: cond_layer_case(),
    "pwa": lambda: pwa_case(),
    "msa_layer": lambda: msa_layer_case(),
    "pairwise_conditioning": lambda: pairwise_conditioning_case(),
    "msa_module": lambda: msa_module_case(),
    "sequence_trunk": lambda: sequence_trunk_case(),
    "sequence_trunk_unconditional": lambda: sequence_trunk_case(seed=27, unconditional=True),
    "cond_layer_window": lambda: cond_layer_window_case(),
    "window_apb": lambda: window_apb_case(),
    "window_apb_batch2": lambda: window_apb_case(seed=29, B=2, M=1, NW=2, n_pad=40),
}


def case_tensors(case: dict):
    out = [v for _, v in sorted(case["w"].items())]
    for k in ("x", "s", "z", "m", "c", "mask", "pair_mask", "msa_mask", "rel", "emb", "s_inputs", "pair_terms"):
        if k in case:
            out.append(case[k].float())
    for _, v in sorted(case.get("feats", {}).items()):
        out.append(v.float())
    return out
