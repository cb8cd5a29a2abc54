"""Triangle attention has no counterpart in the reference, so its oracle cannot be pinned on reference outputs.
These CPU tests pin it the other way round: against a second, independently written formulation (one call of
``torch.nn.functional.scaled_dot_product_attention`` per attention line, fp64, additive mask), and through the
masking / padding invariances the reference tests for its own pair ops."""
import math

import pytest
import torch
import torch.nn.functional as F

import helpers as H
from oracle import pair_ops as O


def _sdpa_formulation(x, mask, w, heads, ending):
    """Per attention line: q, k, v of that line, the shared bias plus -inf on masked keys as an additive mask."""
    if ending:
        x, mask = x.transpose(1, 2), mask.transpose(1, 2)
    B, N, _, D = x.shape
    mu = x.mean(-1, keepdim=True)
    h = (x - mu) * torch.rsqrt(x.var(-1, unbiased=False, keepdim=True) + 1e-5)
    h = h * w["layer_norm.weight"] + w["layer_norm.bias"]
    dh = w["linear_q.weight"].shape[0] // heads
    bias = F.linear(h, w["linear_b.weight"]).permute(0, 3, 1, 2)            # [B, H, j, k]
    out = torch.empty(B, N, N, D, dtype=x.dtype)
    for b in range(B):
        for i in range(N):
            line = h[b, i]                                                   # [N, D]
            q = F.linear(line, w["linear_q.weight"]).view(N, heads, dh).transpose(0, 1)
            k = F.linear(line, w["linear_k.weight"]).view(N, heads, dh).transpose(0, 1)
            v = F.linear(line, w["linear_v.weight"]).view(N, heads, dh).transpose(0, 1)
            add = bias[b] + torch.where(mask[b, i], 0.0, -math.inf).to(x.dtype)[None, None, :]
            o = F.scaled_dot_product_attention(q[None], k[None], v[None], attn_mask=add[None])[0]   # [H, N, dh]
            gate = torch.sigmoid(F.linear(line, w["linear_g.weight"], w["linear_g.bias"]))
            out[b, i] = F.linear(gate * o.transpose(0, 1).reshape(N, heads * dh), w["linear_o.weight"])
    return out.transpose(1, 2) if ending else out


@pytest.mark.parametrize("ending", [False, True])
def test_oracle_agrees_with_per_line_sdpa(ending):
    g = torch.Generator().manual_seed(21)
    N = 23
    w = {k: v.double() for k, v in H.triatt_weights(g).items()}
    x = torch.randn(2, N, N, 128, generator=g).double()
    mask = torch.rand(2, N, N, generator=g) > 0.3
    mask[:, :, 0] = True        # every line keeps at least one key: -inf (additive) and -1e6 (replacing) then agree
    mask[:, 0, :] = True
    got = O.triangle_attention(x, mask, w, 4, ending)
    want = _sdpa_formulation(x, mask, w, 4, ending)
    assert float((got - want).abs().max()) < 1e-10


def test_fully_masked_line_averages_all_keys():
    """The reference's convention for attention (masked logits are REPLACED by a finite -1e6,
    src/bioemu2/biomoa/ops/attention_pair_bias.py:183-190): a line without any valid key weighs all keys equally."""
    g = torch.Generator().manual_seed(22)
    N = 9
    w = {k: v.double() for k, v in H.triatt_weights(g).items()}
    x = torch.randn(1, N, N, 128, generator=g).double()
    mask = torch.ones(1, N, N, dtype=torch.bool)
    mask[0, 3, :] = False
    got = O.triangle_attention(x, mask, w, 4, ending=False)[0, 3]
    h = O.layer_norm(x[0, 3], w["layer_norm.weight"], w["layer_norm.bias"])
    v_mean = O.linear(h, w["linear_v.weight"]).mean(0, keepdim=True).expand(N, -1)
    want = O.linear(torch.sigmoid(O.linear(h, w["linear_g.weight"], w["linear_g.bias"])) * v_mean, w["linear_o.weight"])
    assert float((got - want).abs().max()) < 1e-10
    assert torch.isfinite(got).all()


@pytest.mark.parametrize("ending", [False, True])
def test_masked_inputs_do_not_leak_and_padding_is_invisible(ending):
    """Modelled on tests/biomoa/ops/test_triangle_multiplication.py:303-388 in the reference: poisoning the masked
    tokens, or appending masked tokens filled with 1000.0, leaves the valid region of the update unchanged."""
    g = torch.Generator().manual_seed(23)
    N, P = 14, 3
    w = {k: v.double() for k, v in H.triatt_weights(g).items()}
    x = torch.randn(1, N, N, 128, generator=g).double()
    tok = torch.ones(1, N, dtype=torch.bool)
    tok[0, N - 4:] = False
    mask = tok[:, :, None] & tok[:, None, :]
    base = O.triangle_attention(x, mask, w, 4, ending)
    poisoned = x.clone()
    poisoned[~mask] = 1000.0
    got = O.triangle_attention(poisoned, mask, w, 4, ending)
    assert float((got - base)[mask].abs().max()) < 1e-9
    xp = torch.full((1, N + P, N + P, 128), 1000.0, dtype=torch.float64)
    xp[:, :N, :N] = x
    mp = torch.zeros(1, N + P, N + P, dtype=torch.bool)
    mp[:, :N, :N] = mask
    got = O.triangle_attention(xp, mp, w, 4, ending)[:, :N, :N]
    assert float((got - base)[mask].abs().max()) < 1e-9


def test_ending_node_is_the_starting_node_of_the_transpose():
    g = torch.Generator().manual_seed(24)
    N = 11
    w = {k: v.double() for k, v in H.triatt_weights(g).items()}
    x = torch.randn(1, N, N, 128, generator=g).double()
    mask = torch.rand(1, N, N, generator=g) > 0.2
    a = O.triangle_attention(x, mask, w, 4, ending=True)
    b = O.triangle_attention(x.transpose(1, 2), mask.transpose(1, 2), w, 4, ending=False).transpose(1, 2)
    assert torch.equal(a, b)


def test_line_slab_equals_the_full_result():
    g = torch.Generator().manual_seed(25)
    N = 13
    w = {k: v.double() for k, v in H.triatt_weights(g).items()}
    x = torch.randn(1, N, N, 128, generator=g).double()
    mask = torch.rand(1, N, N, generator=g) > 0.2
    for ending in (False, True):
        full = O.triangle_attention(x, mask, w, 4, ending)
        part = O.triangle_attention(x, mask, w, 4, ending, row_chunk=2, lines=slice(4, 9))
        want = full[:, :, 4:9] if ending else full[:, 4:9]
        assert float((part - want).abs().max()) < 1e-12
