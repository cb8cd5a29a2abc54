"""Triangle attention on the GPU against the CPU oracle.  The reference has no such op, so there are no
golden vectors from it: parity is against the oracle's fp64 statement of the algorithm, plus the
masking / padding invariances the reference tests for its own pair ops."""
import pytest
import torch

import helpers as H
from gpu_util import assert_close
from oracle import pair_ops as O

pytestmark = pytest.mark.gpu


def _module(w: dict, ending: bool):
    import bioemu2_b200 as b

    m = b.TriangleAttention(ending=ending).eval()
    m.load_state_dict(w, strict=True)
    return m.cuda()


@pytest.mark.parametrize("ending", [False, True])
@pytest.mark.parametrize("N,dtype", [(24, torch.float32), (128, torch.float32), (200, torch.bfloat16), (129, torch.float32)])
def test_triatt_vs_oracle(ending, N, dtype):
    g = torch.Generator().manual_seed(500 + N)
    w = H.triatt_weights(g)
    x = torch.randn(1, N, N, 128, generator=g).to(dtype)
    mask = torch.rand(1, N, N, generator=g) > 0.2
    ref = O.triangle_attention(x.double(), mask, {k: v.double() for k, v in w.items()}, 4, ending)
    m = _module(w, ending)
    with torch.no_grad():
        out = m(x.cuda(), mask.cuda())
    assert out.dtype == dtype
    assert_close(f"triatt_{'end' if ending else 'start'}_N{N}_{dtype}", out, ref)


@pytest.mark.parametrize("ending", [False, True])
def test_triatt_residual_inplace_and_padding(ending):
    N, P = 70, 6
    g = torch.Generator().manual_seed(77)
    w = H.triatt_weights(g)
    x = torch.randn(2, N, N, 128, generator=g)
    tok = torch.ones(2, N, dtype=torch.bool)
    tok[0, N - 4:] = False
    mask = tok[:, :, None] & tok[:, None, :]
    m = _module(w, ending)
    with torch.no_grad():
        upd = m(x.cuda(), mask.cuda())
        z = x.cuda().clone()
        ret = m.forward_residual_(z, mask.cuda())
        assert ret.data_ptr() == z.data_ptr()
        torch.testing.assert_close(z, x.cuda() + upd, atol=1e-5, rtol=1e-5)
        xp = torch.full((2, N + P, N + P, 128), 1000.0)
        xp[:, :N, :N] = x
        mp = torch.zeros(2, N + P, N + P, dtype=torch.bool)
        mp[:, :N, :N] = mask
        upd_p = m(xp.cuda(), mp.cuda())[:, :N, :N]
    valid = (tok[:, :, None] & tok[:, None, :]).cuda()
    torch.testing.assert_close(upd_p[valid], upd[valid], atol=2e-3, rtol=0)
