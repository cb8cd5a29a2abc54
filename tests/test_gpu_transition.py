"""Fused pair transition on the GPU against the CPU oracle and the golden vectors."""
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


def _module(w: dict, use_norm=True):
    import bioemu2_b200 as b

    m = b.Transition(128, 512, use_norm=use_norm).eval()
    m.load_state_dict(w, strict=True)
    return m.cuda()


def test_transition_golden():
    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES["transition_pair"]()
    m = _module(case["w"])
    with torch.no_grad():
        out = m(case["x"].cuda())
    assert_close("transition_golden", out, golden["transition_pair"]["output"])


@pytest.mark.parametrize("rows,dtype,use_norm", [
    (128, torch.float32, True), (1000, torch.float32, True), (128 * 300 + 5, torch.bfloat16, True),
    (777, torch.float32, False), (1, torch.float32, True),
])
def test_transition_vs_oracle(rows, dtype, use_norm):
    g = torch.Generator().manual_seed(200 + rows)
    w = H.transition_weights(g, 128, 512, use_norm)
    x = (torch.randn(rows, 128, generator=g) * 2 + 0.5).to(dtype)
    ref = O.transition(x.double(), {k: v.double() for k, v in w.items()})
    m = _module(w, use_norm)
    with torch.no_grad():
        out = m(x.cuda())
    assert out.dtype == dtype
    assert_close(f"transition_rows{rows}_{dtype}_norm{use_norm}", out, ref)


def test_transition_residual_inplace():
    g = torch.Generator().manual_seed(9)
    w = H.transition_weights(g)
    x = torch.randn(3, 50, 50, 128, generator=g)
    m = _module(w)
    with torch.no_grad():
        upd = m(x.cuda())
        z = x.cuda().clone()
        ret = m.forward_residual_(z)
    assert ret.data_ptr() == z.data_ptr()
    torch.testing.assert_close(z, x.cuda() + upd, atol=1e-5, rtol=1e-5)
