"""Pair-weighted averaging and the PairMixer MSA block on the GPU against the reference's golden vectors and the CPU
oracle (the reference's own suite for the op: tests/biomoa/ops/test_pair_weighted_averaging.py)."""
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


def _pwa(w):
    import bioemu2_b200 as b

    m = b.PairWeightedAveraging(c_m=64, c_z=128, c_h=32, num_heads=8).eval()
    m.load_state_dict(w, strict=True)
    return m.cuda()


def test_pwa_golden():
    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES["pwa"]()
    mod = _pwa(case["w"])
    with torch.no_grad():
        out = mod(case["m"].cuda(), case["z"].cuda(), case["mask"].cuda())
    assert_close("pwa_golden", out, golden["pwa"]["output"])


@pytest.mark.parametrize("B,S,N,dtype", [(2, 5, 37, torch.float32), (1, 130, 136, torch.float32), (1, 9, 200, torch.bfloat16)])
def test_pwa_vs_oracle(B, S, N, dtype):
    """Ragged token counts, a random pair mask and one token whose row of the mask is empty (uniform weights)."""
    g = torch.Generator().manual_seed(800 + N)
    w = H.pwa_weights(g)
    m = torch.randn(B, S, N, 64, generator=g).to(dtype)
    z = torch.randn(B, N, N, 128, generator=g).to(dtype)
    mask = torch.rand(B, N, N, generator=g) > 0.2
    mask[0, 3, :] = False
    ref = O.pair_weighted_averaging(m.double(), z.double(), mask, {k: v.double() for k, v in w.items()})
    mod = _pwa(w)
    with torch.no_grad():
        out = mod(m.cuda(), z.cuda(), mask.cuda())
        res = mod.forward_residual(m.cuda(), z.cuda(), mask.cuda())
    assert out.dtype == dtype and tuple(out.shape) == (B, S, N, 64)
    assert_close(f"pwa_B{B}_S{S}_N{N}_{dtype}", out, ref)
    torch.testing.assert_close(res.float(), m.cuda().float() + out.float(), atol=2e-2 if dtype == torch.bfloat16 else 1e-5,
                               rtol=1e-2 if dtype == torch.bfloat16 else 1e-5)


def test_pwa_masked_pairs_do_not_leak():
    """Values of z under the mask are irrelevant (the masked logit is replaced, not added to)."""
    g = torch.Generator().manual_seed(801)
    w = H.pwa_weights(g)
    m = torch.randn(1, 4, 48, 64, generator=g)
    z = torch.randn(1, 48, 48, 128, generator=g)
    mask = torch.rand(1, 48, 48, generator=g) > 0.3
    zp = z.clone()
    zp[~mask] = 1000.0
    mod = _pwa(w)
    with torch.no_grad():
        a = mod(m.cuda(), z.cuda(), mask.cuda())
        b = mod(m.cuda(), zp.cuda(), mask.cuda())
    assert torch.equal(a, b)


def test_msa_layer_golden():
    import bioemu2_b200 as b

    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES["msa_layer"]()
    layer = b.PairMixerMSALayer(token_s=384, msa_s=64, token_z=128).eval()
    layer.load_state_dict(case["w"], strict=True)
    layer.cuda()
    z_in, m_in = case["z"].cuda(), case["m"].cuda()
    z0, m0 = z_in.clone(), m_in.clone()
    s = torch.zeros(1, z_in.shape[1], 384, device="cuda")
    with torch.no_grad():
        s_out, z_out, m_out = layer(s, z_in, m_in, case["pair_mask"].cuda(), case["msa_mask"].cuda())
    assert s_out is s
    assert torch.equal(z_in, z0) and torch.equal(m_in, m0), "forward must not modify its inputs"
    want = golden["msa_layer"]["output"]
    nz = z_out.numel()
    # two updated tensors after six residual updates: the per-element bar with its absolute part doubled
    assert_close("msa_layer_golden_z", z_out.flatten(), want[:nz], atol=4e-2)
    assert_close("msa_layer_golden_m", m_out.flatten(), want[nz:], atol=4e-2)
