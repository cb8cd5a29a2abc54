"""Shared builders for seeded weights and inputs used by the parity tests."""
from __future__ import annotations

import math

import torch


def kaiming_linear(gen: torch.Generator, out_f: int, in_f: int) -> torch.Tensor:
    """torch.nn.Linear's default init (Kaiming-uniform, a=sqrt(5)) -> U(-1/sqrt(in), 1/sqrt(in))."""
    bound = 1.0 / math.sqrt(in_f)
    return (torch.rand(out_f, in_f, generator=gen) * 2 - 1) * bound


def ln_params(gen: torch.Generator, dim: int, perturbed: bool = True):
    if perturbed:
        return 1.0 + 0.1 * torch.randn(dim, generator=gen), 0.1 * torch.randn(dim, generator=gen)
    return torch.ones(dim), torch.zeros(dim)


def trimul_weights(gen, dim=128, perturbed=True) -> dict:
    w = {}
    w["norm_in.weight"], w["norm_in.bias"] = ln_params(gen, dim, perturbed)
    w["p_in.weight"] = kaiming_linear(gen, 2 * dim, dim)
    w["g_in.weight"] = kaiming_linear(gen, 2 * dim, dim)
    w["norm_out.weight"], w["norm_out.bias"] = ln_params(gen, dim, perturbed)
    w["p_out.weight"] = kaiming_linear(gen, dim, dim)
    w["g_out.weight"] = kaiming_linear(gen, dim, dim)
    return w


def transition_weights(gen, dim=128, hidden=512, use_norm=True, perturbed=True) -> dict:
    w = {}
    if use_norm:
        w["norm.weight"], w["norm.bias"] = ln_params(gen, dim, perturbed)
    w["fc1.weight"] = kaiming_linear(gen, hidden, dim)
    w["fc2.weight"] = kaiming_linear(gen, hidden, dim)
    w["fc3.weight"] = kaiming_linear(gen, dim, hidden)
    return w


def apb_weights(gen, c_s=384, c_z=128, heads=16, initial_norm=True, perturbed=True) -> dict:
    w = {}
    if initial_norm:
        w["norm_s.weight"], w["norm_s.bias"] = ln_params(gen, c_s, perturbed)
    w["proj_qkv.weight"] = kaiming_linear(gen, 3 * c_s, c_s)
    w["proj_q_bias"] = 0.02 * torch.randn(c_s, generator=gen)
    w["proj_g.weight"] = kaiming_linear(gen, c_s, c_s)
    w["norm_z.weight"] = ln_params(gen, c_z, perturbed)[0]
    w["proj_z.weight"] = kaiming_linear(gen, heads, c_z)
    w["proj_o.weight"] = kaiming_linear(gen, c_s, c_s)
    return w


def opm_weights(gen, c_in=64, c_hidden=32, c_out=128, perturbed=True) -> dict:
    w = {}
    w["norm.weight"], w["norm.bias"] = ln_params(gen, c_in, perturbed)
    w["proj_ab.weight"] = kaiming_linear(gen, 2 * c_hidden, c_in)
    w["proj_o.weight"] = kaiming_linear(gen, c_out, c_hidden * c_hidden)
    w["proj_o.bias"] = (torch.rand(c_out, generator=gen) * 2 - 1) / math.sqrt(c_hidden * c_hidden)
    return w


def triatt_weights(gen, dim=128, heads=4, head_dim=32, perturbed=True) -> dict:
    w = {}
    w["layer_norm.weight"], w["layer_norm.bias"] = ln_params(gen, dim, perturbed)
    for n in ("q", "k", "v"):
        w[f"linear_{n}.weight"] = kaiming_linear(gen, heads * head_dim, dim)
    w["linear_b.weight"] = kaiming_linear(gen, heads, dim)
    w["linear_g.weight"] = kaiming_linear(gen, heads * head_dim, dim)
    w["linear_g.bias"] = torch.ones(heads * head_dim)
    w["linear_o.weight"] = kaiming_linear(gen, dim, heads * head_dim)
    return w


def pwa_weights(gen, c_m=64, c_z=128, c_h=32, heads=8, perturbed=True) -> dict:
    w = {}
    w["norm_m.weight"], w["norm_m.bias"] = ln_params(gen, c_m, perturbed)
    w["norm_z.weight"], w["norm_z.bias"] = ln_params(gen, c_z, perturbed)
    w["proj_m.weight"] = kaiming_linear(gen, c_h * heads, c_m)
    w["proj_g.weight"] = kaiming_linear(gen, c_h * heads, c_m)
    w["proj_z.weight"] = kaiming_linear(gen, heads, c_z)
    w["proj_o.weight"] = kaiming_linear(gen, c_m, c_h * heads)
    return w


def msa_layer_weights(gen, msa_s=64, token_z=128, perturbed=True) -> dict:
    """State dict of the reference's ``PairMixerMSALayer`` in module-construction order."""
    w = {}
    w.update(prefixed("msa_transition", transition_weights(gen, msa_s, 4 * msa_s, True, perturbed)))
    w.update(prefixed("pair_weighted_averaging", pwa_weights(gen, msa_s, token_z, 32, 8, perturbed)))
    w.update(prefixed("tri_mul_out", trimul_weights(gen, token_z, perturbed)))
    w.update(prefixed("tri_mul_in", trimul_weights(gen, token_z, perturbed)))
    w.update(prefixed("z_transition", transition_weights(gen, token_z, 4 * token_z, True, perturbed)))
    w.update(prefixed("outer_product_mean", opm_weights(gen, msa_s, 32, token_z, perturbed)))
    return w


def pairwise_conditioning_weights(gen, token_z=128, rel=128, a_z=128, num_transitions=2, factor=2, perturbed=True) -> dict:
    """State dict of the reference's ``PairwiseConditioning``."""
    w = {}
    w["dim_pairwise_init_proj.0.weight"], w["dim_pairwise_init_proj.0.bias"] = ln_params(gen, token_z + rel, perturbed)
    w["dim_pairwise_init_proj.1.weight"] = kaiming_linear(gen, a_z, token_z + rel)
    for i in range(num_transitions):
        w.update(prefixed(f"transitions.{i}", transition_weights(gen, a_z, factor * a_z, True, perturbed)))
    return w


def msa_module_weights(gen, s_input_dim, blocks, msa_s=64, token_z=128, msa_feat=36, perturbed=True) -> dict:
    """State dict of the reference's ``PairMixerMSAModule`` (``msa_feat`` = num_tokens + 2 + paired flag)."""
    w = {"s_proj.weight": kaiming_linear(gen, msa_s, s_input_dim), "msa_proj.weight": kaiming_linear(gen, msa_s, msa_feat)}
    for i in range(blocks):
        w.update(prefixed(f"layers.{i}", msa_layer_weights(gen, msa_s, token_z, perturbed)))
    return w


def sequence_trunk_weights(gen, s_input_dim, msa_blocks, num_blocks, token_s=384, token_z=128, perturbed=True) -> dict:
    """The reference ``PairMixerSequenceEmbedder``'s state dict without its feature encoders (rel_pos, token_bonds)."""
    w = {"s_init.weight": kaiming_linear(gen, token_s, s_input_dim),
         "z_init_1.weight": kaiming_linear(gen, token_z, s_input_dim),
         "z_init_2.weight": kaiming_linear(gen, token_z, s_input_dim)}
    w.update(prefixed("msa_module", msa_module_weights(gen, s_input_dim, msa_blocks, 64, token_z, 36, perturbed)))
    for i in range(num_blocks):
        w.update(prefixed(f"pairmixer_module.layers.{i}", pairmixer_layer_weights(gen, token_z, perturbed)))
    w["s_recycle.weight"] = kaiming_linear(gen, token_s, token_s)
    w["z_recycle.weight"] = kaiming_linear(gen, token_z, token_z)
    w["s_norm.weight"], w["s_norm.bias"] = ln_params(gen, token_s, perturbed)
    w["z_norm.weight"], w["z_norm.bias"] = ln_params(gen, token_z, perturbed)
    w.update(prefixed("uncond_transition", transition_weights(gen, token_z, 4 * token_z, True, perturbed)))
    return w


def prefixed(prefix: str, w: dict) -> dict:
    return {f"{prefix}.{k}": v for k, v in w.items()}


def pairmixer_layer_weights(gen, dim=128, perturbed=True) -> dict:
    w = {}
    w.update(prefixed("tri_mul_out", trimul_weights(gen, dim, perturbed)))
    w.update(prefixed("tri_mul_in", trimul_weights(gen, dim, perturbed)))
    w.update(prefixed("transition_z", transition_weights(gen, dim, 4 * dim, True, perturbed)))
    return w


def rel_err(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """max|a-e| / max|e| : the relative error the parity bars are stated in."""
    a, e = actual.double(), expected.double()
    return float((a - e).abs().max() / e.abs().max().clamp_min(1e-30))
