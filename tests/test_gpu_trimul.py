"""Triangle multiplication on the GPU against the CPU oracle and the reference's golden vectors."""
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


def _module(w: dict, mode: str):
    import bioemu2_b200 as b

    m = b.TriangleMultiplication(128, mode).eval()
    m.load_state_dict(w, strict=True)
    return m.cuda()


@pytest.mark.parametrize("mode", ["outgoing", "incoming"])
def test_trimul_golden(mode):
    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES[f"trimul_{mode}"]()
    m = _module(case["w"], mode)
    with torch.no_grad():
        out = m(case["x"].cuda(), case["mask"].cuda())
    assert out.dtype == torch.float32
    assert_close(f"trimul_golden_{mode}", out, golden[f"trimul_{mode}"]["output"])


@pytest.mark.parametrize("mode", ["outgoing", "incoming"])
@pytest.mark.parametrize("N,dtype", [(128, torch.float32), (129, torch.float32), (200, torch.bfloat16), (7, torch.float32)])
def test_trimul_vs_oracle(mode, N, dtype):
    g = torch.Generator().manual_seed(100 + N)
    w = H.trimul_weights(g)
    x = torch.randn(1, N, N, 128, generator=g)
    mask = torch.rand(1, N, N, generator=g) > 0.25
    xin = x.to(dtype)
    ref = O.triangle_multiplication(xin.double(), mask, {k: v.double() for k, v in w.items()}, mode)
    m = _module(w, mode)
    with torch.no_grad():
        out = m(xin.cuda(), mask.cuda())
    assert out.dtype == dtype
    assert_close(f"trimul_{mode}_N{N}_{dtype}", out, ref)


def test_trimul_residual_inplace_and_masked_poison():
    """z += update in place equals the separate add; poisoned masked entries do not leak
    (tests/biomoa/ops/test_triangle_multiplication.py:373-388 in the reference)."""
    N = 96
    g = torch.Generator().manual_seed(7)
    w = H.trimul_weights(g)
    x = torch.randn(1, N, N, 128, generator=g)
    mask = torch.rand(1, N, N, generator=g) > 0.25
    m = _module(w, "outgoing")
    with torch.no_grad():
        upd = m(x.cuda(), mask.cuda())
        z = x.cuda().clone()
        ret = m.forward_residual_(z, mask.cuda())
        assert ret.data_ptr() == z.data_ptr()
        torch.testing.assert_close(z, x.cuda() + upd, atol=1e-5, rtol=1e-5)
        poisoned = x.clone()
        poisoned[~mask] = 1000.0
        upd_p = m(poisoned.cuda(), mask.cuda())
    mk = mask.cuda()
    assert torch.equal(upd[mk], upd_p[mk])


def test_trimul_padding_invariance():
    """Appending masked rows/columns filled with 1000.0 leaves the valid region unchanged
    (tests/biomoa/ops/test_triangle_multiplication.py:303-371 in the reference)."""
    N, P = 60, 4
    g = torch.Generator().manual_seed(8)
    w = H.trimul_weights(g)
    x = torch.randn(1, N, N, 128, generator=g)
    mask = torch.rand(1, N, N, generator=g) > 0.25
    xp = torch.full((1, N + P, N + P, 128), 1000.0)
    xp[:, :N, :N] = x
    mp = torch.zeros(1, N + P, N + P, dtype=torch.bool)
    mp[:, :N, :N] = mask
    for mode in ("outgoing", "incoming"):
        m = _module(w, mode)
        with torch.no_grad():
            a = m(x.cuda(), mask.cuda())
            b = m(xp.cuda(), mp.cuda())[:, :N, :N]
        torch.testing.assert_close(a, b, atol=1e-6, rtol=0)


def test_trimul_rejects_bad_shapes():
    import bioemu2_b200 as b

    m = b.TriangleMultiplication(128, "outgoing").eval().cuda()
    with pytest.raises(ValueError):
        m(torch.zeros(1, 8, 9, 128, device="cuda"), torch.ones(1, 8, 9, dtype=torch.bool, device="cuda"))
    with pytest.raises(ValueError):
        m(torch.zeros(1, 8, 8, 128, device="cuda"), torch.ones(1, 8, 7, dtype=torch.bool, device="cuda"))
    with pytest.raises(ValueError):
        b.TriangleMultiplication(64, "outgoing")
