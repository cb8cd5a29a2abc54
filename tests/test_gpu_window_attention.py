"""Sliding-window attention with pair bias (the atom transformer's attention) on the GPU against the golden vectors of
the reference's ``AttentionPairBiasSlidingWindow`` and against the CPU oracle."""
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


def _module(w, c_s, c_z, heads, W, Hk):
    import bioemu2_b200 as b

    m = b.AttentionPairBiasSlidingWindow(c_s, c_z, heads, window_queries=W, window_keys=Hk).eval()
    m.load_state_dict(w, strict=True)
    return m.cuda()


@pytest.mark.parametrize("name", ["window_apb", "window_apb_batch2"])
def test_window_attention_golden(name):
    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES[name]()
    mod = _module(case["w"], case["s"].shape[-1], case["z"].shape[-1], case["heads"], case["W"], case["Hk"])
    with torch.no_grad():
        out = mod(case["s"].cuda(), case["z"].cuda(), case["mask"].cuda(), multiplicity=case["M"])
    assert out.dtype == torch.float32 and out.shape == case["s"].shape
    assert_close(name, out, golden[name]["output"])


@pytest.mark.parametrize("B,M,NW,W,Hk,c_s,c_z,heads,dtype", [
    (2, 3, 7, 32, 128, 128, 16, 4, torch.float32),     # the atom transformer's shape
    (1, 1, 5, 32, 128, 64, 16, 4, torch.float32),      # head dim 16
    (1, 2, 4, 32, 128, 128, 24, 2, torch.bfloat16),    # head dim 64, bf16 streams
    (1, 2, 9, 16, 48, 128, 16, 4, torch.float32),      # other window sizes
])
def test_window_attention_vs_oracle(B, M, NW, W, Hk, c_s, c_z, heads, dtype):
    g = torch.Generator().manual_seed(1000 + NW * W + c_s)
    w = H.apb_weights(g, c_s, c_z, heads, True)
    s = torch.randn(B * M * NW, W, c_s, generator=g).to(dtype)
    z = torch.randn(B, NW, W, Hk, c_z, generator=g).to(dtype)
    mask = torch.rand(B, NW * W, generator=g) > 0.15
    mask[:, NW * W - 11:] = False                       # ragged end
    if NW > 4:
        mask[0, : 3 * W] = False                        # windows whose keys are nearly all masked
    mask = mask.reshape(B * NW, W)
    ref = O.attention_pair_bias_sliding_window(s.double(), z.double(), mask, {k: v.double() for k, v in w.items()}, heads, M)
    with torch.no_grad():
        out = _module(w, c_s, c_z, heads, W, Hk)(s.cuda(), z.cuda(), mask.cuda(), multiplicity=M)
    assert out.dtype == dtype
    assert_close(f"window_apb_B{B}_M{M}_NW{NW}_W{W}_H{Hk}_c{c_s}_{dtype}", out, ref)


def test_window_attention_all_keys_masked_gives_the_mean_of_the_window():
    """With every key masked all logits equal -1e6: uniform weights over the H keys, zero rows included."""
    g = torch.Generator().manual_seed(1100)
    w = H.apb_weights(g, 128, 16, 4, True)
    s = torch.randn(3, 32, 128, generator=g)
    z = torch.randn(1, 3, 32, 128, 16, generator=g)
    mask = torch.zeros(3, 32, dtype=torch.bool)
    ref = O.attention_pair_bias_sliding_window(s.double(), z.double(), mask, {k: v.double() for k, v in w.items()}, 4, 1)
    with torch.no_grad():
        out = _module(w, 128, 16, 4, 32, 128)(s.cuda(), z.cuda(), mask.cuda())
    assert_close("window_apb_all_masked", out, ref)


def test_window_attention_masked_atoms_do_not_leak():
    """Pair features under masked keys and the rows of masked atoms do not reach the valid queries' outputs: a masked
    logit is replaced, not added to."""
    g = torch.Generator().manual_seed(1101)
    w = H.apb_weights(g, 128, 16, 4, True)
    NW, W, Hk = 4, 32, 128
    s = torch.randn(NW, W, 128, generator=g)
    z = torch.randn(1, NW, W, Hk, 16, generator=g)
    mask = torch.ones(1, NW * W, dtype=torch.bool)
    mask[0, 50:70] = False
    sp, zp = s.clone().reshape(NW * W, 128), z.clone()
    sp[50:70] = 100.0
    key_atom = torch.arange(NW)[:, None] * W - (Hk - W) // 2 + torch.arange(Hk)[None, :]      # [NW, Hk]
    bad = (key_atom >= 50) & (key_atom < 70)
    zp[0][bad[:, None, :].expand(NW, W, Hk)] = 1000.0
    mod = _module(w, 128, 16, 4, W, Hk)
    m2 = mask.reshape(NW, W).cuda()
    with torch.no_grad():
        a = mod(s.cuda(), z.cuda(), m2)
        b = mod(sp.reshape(NW, W, 128).cuda(), zp.cuda(), m2)
    valid = mask.reshape(NW * W).cuda()
    assert torch.equal(a.reshape(NW * W, 128)[valid], b.reshape(NW * W, 128)[valid])


def test_window_attention_shape_errors():
    g = torch.Generator().manual_seed(1102)
    mod = _module(H.apb_weights(g, 128, 16, 4, True), 128, 16, 4, 32, 128)
    s = torch.zeros(2, 32, 128).cuda()
    with pytest.raises(ValueError, match="windows of 32 queries"):
        mod(s, torch.zeros(1, 2, 32, 96, 16).cuda(), torch.ones(2, 32, dtype=torch.bool).cuda())
    with pytest.raises(ValueError, match="inconsistent shapes"):
        mod(s, torch.zeros(1, 3, 32, 128, 16).cuda(), torch.ones(3, 32, dtype=torch.bool).cuda())
