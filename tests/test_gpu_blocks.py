"""Composite blocks on the GPU: single-track transition, conditioned transformer layer (golden vectors of
the reference), and the benchmark's Pairformer block (CPU oracle)."""
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


def test_transition_single_track_golden():
    import bioemu2_b200 as b

    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES["transition_single_nonorm"]()
    m = b.Transition(384, 1536, use_norm=False).eval()
    m.load_state_dict(case["w"], strict=True)
    m.cuda()
    with torch.no_grad():
        out = m(case["x"].cuda())
        z = case["x"].cuda().clone()
        m.forward_residual_(z)
    assert_close("transition_single_golden", out, golden["transition_single_nonorm"]["output"])
    torch.testing.assert_close(z, case["x"].cuda() + out, atol=1e-5, rtol=1e-5)


def test_conditioned_transformer_layer_golden():
    import bioemu2_b200 as b

    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES["cond_layer"]()
    m = b.ConditionedTransformerLayer(dim=384, dim_pairwise=128, dim_cond=384, heads=case["heads"],
                                      transition_hidden=case["hidden"], lns_scale=case["lns_scale"]).eval()
    m.load_state_dict(case["w"], strict=True)
    m.cuda()
    x = case["x"].cuda()
    with torch.no_grad():
        out = m(x, case["z"].cuda(), case["c"].cuda(), case["mask"].cuda(), multiplicity=case["M"])
    assert out.data_ptr() != x.data_ptr()
    assert_close("cond_layer_golden", out, golden["cond_layer"]["output"])


def test_conditioned_transformer_layer_sliding_window_golden():
    """The atom transformer's block: windowed attention inside the same conditioned layer, mask given and omitted."""
    import bioemu2_b200 as b

    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES["cond_layer_window"]()
    W, Hk = case["window"]
    m = b.ConditionedTransformerLayer(dim=128, dim_pairwise=16, dim_cond=128, heads=case["heads"],
                                      transition_hidden=case["hidden"], lns_scale=case["lns_scale"],
                                      is_sliding_window=True, window_queries=W, window_keys=Hk).eval()
    m.load_state_dict(case["w"], strict=True)
    m.cuda()
    assert isinstance(m.attention, b.SlidingWindowAttentionLayer)
    x, z, c = case["x"].cuda(), case["z"].cuda(), case["c"].cuda()
    with torch.no_grad():
        out = m(x, z, c, case["mask"].cuda(), multiplicity=case["M"])
        flat = m(x, z.reshape(1, -1, Hk, 16), c, case["mask"].cuda(), multiplicity=case["M"])   # flat [B, N, H, c] pairs
        full = m(x, z, c, None, multiplicity=case["M"])
        ones = m(x, z, c, torch.ones_like(case["mask"]).cuda(), multiplicity=case["M"])
    assert_close("cond_layer_window_golden", out, golden["cond_layer_window"]["output"])
    assert torch.equal(out, flat) and torch.equal(full, ones)


def _pairformer_weights(g):
    w = {}
    w.update(H.prefixed("tri_mul_out", H.trimul_weights(g)))
    w.update(H.prefixed("tri_mul_in", H.trimul_weights(g)))
    w.update(H.prefixed("tri_att_start", H.triatt_weights(g)))
    w.update(H.prefixed("tri_att_end", H.triatt_weights(g)))
    w.update(H.prefixed("transition_z", H.transition_weights(g, 128, 512)))
    w.update(H.prefixed("attention", H.apb_weights(g, 384, 128, 16)))
    w.update(H.prefixed("transition_s", H.transition_weights(g, 384, 1536)))
    return w


@pytest.mark.parametrize("N", [40, 128])
def test_pairformer_block_vs_oracle(N):
    """Benchmark config 0's block (N=128, all-ones mask) and a ragged smaller one."""
    import bioemu2_b200 as b

    g = torch.Generator().manual_seed(0)
    w = _pairformer_weights(g)
    z = torch.randn(1, N, N, 128, generator=g)
    s = torch.randn(1, N, 384, generator=g)
    tok = torch.ones(1, N, dtype=torch.bool)
    if N != 128:
        tok[0, N - 6:] = False
    s_ref, z_ref = O.pairformer_block(s, z, tok, w)
    blk = b.PairformerBlock().eval()
    blk.load_state_dict(w, strict=True)
    blk.cuda()
    with torch.no_grad():
        s_out, z_out = blk(s.cuda(), z.cuda(), tok.cuda())
    pm = (tok[:, :, None] & tok[:, None, :])[0]
    assert_close(f"pairformer_block_z_N{N}", z_out[0][pm.cuda()], z_ref[0][pm])
    assert_close(f"pairformer_block_s_N{N}", s_out[0][tok[0].cuda()], s_ref[0][tok[0]])
