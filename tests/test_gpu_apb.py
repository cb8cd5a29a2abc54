"""Single-track pair-bias attention on the GPU against the golden vectors and the CPU oracle."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import cases as C  # noqa: E402
import helpers as H  # noqa: E402
from gpu_util import assert_close  # noqa: E402
from oracle import pair_ops as O  # noqa: E402

pytestmark = pytest.mark.gpu


def _module(w: dict, c_s=384, heads=16, initial_norm=True):
    import bioemu2_b200 as b

    m = b.AttentionPairBias(c_s, 128, heads, initial_norm=initial_norm).eval()
    m.load_state_dict(w, strict=True)
    return m.cuda()


@pytest.mark.parametrize("name", ["apb", "apb_multiplicity", "apb_nonorm_dh48"])
def test_apb_golden(name):
    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES[name]()
    mod = _module(case["w"], case["s"].shape[-1], case["heads"], case["initial_norm"])
    with torch.no_grad():
        out = mod(case["s"].cuda(), case["z"].cuda(), case["mask"].cuda(), multiplicity=case["M"])
    assert_close(f"apb_golden_{name}", out, golden[name]["output"])


@pytest.mark.parametrize("N,c_s,heads,M,dtype", [
    (64, 384, 16, 1, torch.float32),     # the reference's own test shape (C_S=384, C_Z=128, H=16, N=64)
    (64, 384, 8, 3, torch.float32),      # H=8 -> head dim 48 (padded to 64), multiplicity 3
    (200, 384, 16, 2, torch.bfloat16),   # two key tiles, ragged last tile
    (300, 768, 16, 1, torch.float32),    # diffusion-module shape (c_token 768, dh 48), three key tiles
])
def test_apb_vs_oracle(N, c_s, heads, M, dtype):
    B = 2
    g = torch.Generator().manual_seed(400 + N + heads)
    w = H.apb_weights(g, c_s, 128, heads)
    s = torch.randn(B * M, N, c_s, generator=g).to(dtype)
    z = torch.randn(B, N, N, 128, generator=g).to(dtype)
    mask = torch.ones(B, N, dtype=torch.bool)
    mask[0, N - 9:] = False
    mask[1, 3] = False
    ref = O.attention_pair_bias(s.double(), z.double(), mask, {k: v.double() for k, v in w.items()}, heads, M)
    mod = _module(w, c_s, heads)
    with torch.no_grad():
        out = mod(s.cuda(), z.cuda(), mask.cuda(), multiplicity=M)
    assert out.dtype == dtype
    assert_close(f"apb_N{N}_c{c_s}_H{heads}_M{M}_{dtype}", out, ref)


def test_apb_fully_masked_and_padding():
    """A fully masked batch element stays finite (uniform average, attention_pair_bias.py:183-190 in the
    reference) and appended masked tokens filled with 1000.0 leave valid outputs unchanged
    (tests/biomoa/ops/test_attention_pair_bias.py:805-951)."""
    N, P, c_s, heads = 48, 5, 384, 16
    g = torch.Generator().manual_seed(55)
    w = H.apb_weights(g, c_s, 128, heads)
    s = torch.randn(2, N, c_s, generator=g)
    z = torch.randn(2, N, N, 128, generator=g)
    mask = torch.ones(2, N, dtype=torch.bool)
    mask[1] = False
    mod = _module(w, c_s, heads)
    ref = O.attention_pair_bias(s.double(), z.double(), mask, {k: v.double() for k, v in w.items()}, heads, 1)
    with torch.no_grad():
        out = mod(s.cuda(), z.cuda(), mask.cuda())
    assert torch.isfinite(out).all()
    assert_close("apb_fully_masked", out, ref)
    sp = torch.full((2, N + P, c_s), 1000.0)
    sp[:, :N] = s
    zp = torch.full((2, N + P, N + P, 128), 1000.0)
    zp[:, :N, :N] = z
    mp = torch.zeros(2, N + P, dtype=torch.bool)
    mp[0, :N] = True
    with torch.no_grad():
        out_p = mod(sp.cuda(), zp.cuda(), mp.cuda())
    torch.testing.assert_close(out_p[0, :N], out[0], atol=2e-3, rtol=0)


@pytest.mark.parametrize("Bt,N,H,dh", [(3, 200, 4, 32), (2, 130, 2, 48), (1, 512, 4, 32)])
def test_attention_core_entry_point(Bt, N, H, dh):
    """The exported flash core against a plain fp64 softmax on the same (bf16-rounded) operands."""
    import math

    from bioemu2_b200 import functional as F

    g = torch.Generator(device="cuda").manual_seed(Bt * 100 + N)
    q = torch.randn(Bt, N, H, dh, device="cuda", generator=g).bfloat16()
    k = torch.randn(Bt, N, H, dh, device="cuda", generator=g).bfloat16()
    v = torch.randn(Bt, N, H, dh, device="cuda", generator=g).bfloat16()
    gate = torch.randn(Bt, N, H, dh, device="cuda", generator=g).bfloat16()
    bias = torch.randn(1, H, N, N, device="cuda", generator=g).bfloat16()
    mask = torch.rand(Bt, N, device="cuda", generator=g) > 0.2
    out = F.attention_core(q, k, v, bias, mask, gate, bias_div=Bt)
    logits = torch.einsum("bihd,bjhd->bhij", q.double(), k.double()) / math.sqrt(dh) + bias.double()
    logits = torch.where(mask[:, None, None, :], logits, torch.full_like(logits, -1e6))
    ref = torch.einsum("bhij,bjhd->bihd", logits.softmax(-1), v.double()) * torch.sigmoid(gate.double())
    assert_close(f"attention_core_B{Bt}_N{N}_H{H}_dh{dh}", out, ref)


@pytest.mark.parametrize("B,N", [(1, 136), (2, 72), (1, 77)])
def test_pair_bias_cache_one_pass_matches_per_layer_projection(B, N):
    """Three token-block attentions (c_token 768, 16 heads) sharing one static pair tensor: the biases computed in one
    pass over z give the same attention output as every layer projecting its own, and both match the oracle.  N = 77
    is not a multiple of 8 and takes the per-layer fallback inside ``prepare``."""
    import bioemu2_b200 as b

    g = torch.Generator().manual_seed(700 + N)
    L, c_s, heads, M = 3, 768, 16, 2
    ws = [H.apb_weights(g, c_s, 128, heads, initial_norm=False) for _ in range(L)]
    mods = [_module(w, c_s, heads, initial_norm=False) for w in ws]
    s = torch.randn(B * M, N, c_s, generator=g)
    z = torch.randn(B, N, N, 128, generator=g)
    mask = torch.ones(B, N, dtype=torch.bool)
    mask[0, N - 5:] = False
    sd, zd, md = s.cuda(), z.cuda(), mask.cuda()
    with torch.no_grad():
        plain = [m(sd, zd, md, multiplicity=M) for m in mods]
        cache = b.PairBiasCache(mods)
        bias = cache.prepare(zd)
        assert all(cache.lookup(i, zd) is not None for i in range(L))
        assert cache.lookup(0, zd.clone()) is None, "another tensor object must not hit the cache"
        cached = [m(sd, zd, md, multiplicity=M) for m in mods]
        zd.add_(1.0)  # an in-place change bumps the version counter: the cache no longer applies
        assert cache.lookup(0, zd) is None
    if N % 8 == 0:
        assert tuple(bias.shape) == (L, B, heads, N, N)
    for i in range(L):
        ref = O.attention_pair_bias(s.double(), z.double(), mask, {k: v.double() for k, v in ws[i].items()}, heads, M)
        assert_close(f"apb_cached_bias_layer{i}_B{B}_N{N}", cached[i], ref)
        assert_close(f"apb_plain_bias_layer{i}_B{B}_N{N}", plain[i], ref)
