"""Outer product mean on the GPU against the golden vectors and the CPU oracle."""
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


def _module(w: dict):
    import bioemu2_b200 as b

    m = b.OuterProductMean(64, 32, 128).eval()
    m.load_state_dict(w, strict=True)
    return m.cuda()


@pytest.mark.parametrize("name", ["opm", "opm_mask2d"])
def test_opm_golden(name):
    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES[name]()
    mod = _module(case["w"])
    with torch.no_grad():
        out = mod(case["m"].cuda(), case["mask"].cuda())
    assert_close(f"opm_golden_{name}", out, golden[name]["output"], rel=2.5e-2)


@pytest.mark.parametrize("B,S,N,dtype", [(2, 300, 37, torch.float32), (1, 130, 128, torch.bfloat16),
                                          (1, 64, 200, torch.float32)])
def test_opm_vs_oracle(B, S, N, dtype):
    """Shapes of the reference's own test (S=300, N=37, B=2; tests/biomoa/ops/test_outer_product_mean.py)
    plus sizes that cross tile boundaries.  Tolerance 2.5e-2 is the reference's bf16 bar for this op."""
    g = torch.Generator().manual_seed(300 + S + N)
    w = H.opm_weights(g)
    m = torch.randn(B, S, N, 64, generator=g).to(dtype)
    mask = torch.ones(B, S, N, dtype=torch.bool)
    mask[:, 1, -3:] = False
    mask[0, -10:] = False
    mask[:, :, 5] = False
    ref = O.outer_product_mean(m.double(), mask, {k: v.double() for k, v in w.items()})
    mod = _module(w)
    with torch.no_grad():
        out = mod(m.cuda(), mask.cuda())
    assert out.dtype == dtype and tuple(out.shape) == (B, N, N, 128)
    assert_close(f"opm_B{B}_S{S}_N{N}_{dtype}", out, ref, rel=2.5e-2)


def test_opm_masked_inputs_do_not_leak():
    """tests/biomoa/ops/test_outer_product_mean.py:288-299 in the reference: values under the mask are irrelevant."""
    g = torch.Generator().manual_seed(41)
    w = H.opm_weights(g)
    m = torch.randn(1, 50, 40, 64, generator=g)
    mask = torch.rand(1, 50, 40, generator=g) > 0.3
    changed = m.clone()
    changed[~mask] = 1000.0
    mod = _module(w)
    with torch.no_grad():
        a = mod(m.cuda(), mask.cuda())
        b = mod(changed.cuda(), mask.cuda())
    assert torch.equal(a, b)


def test_opm_config1_shape_runs():
    """Benchmark config 1: m[1,1024,384,64] bf16, 10 % of MSA rows masked, seed 1."""
    g = torch.Generator().manual_seed(1)
    w = H.opm_weights(g, perturbed=False)
    m = torch.randn(1, 1024, 384, 64, generator=g).bfloat16()
    rows = torch.rand(1, 1024, generator=g) > 0.1
    mask = rows[:, :, None].expand(1, 1024, 384).contiguous()
    mod = _module(w)
    with torch.no_grad():
        out = mod(m.cuda(), mask.cuda())
    # oracle on a 48x48 corner (the full fp64 oracle needs 1.2 GB and ~10 s; the corner pins the same code path)
    ref = O.outer_product_mean(m[:, :, :48].double(), mask[:, :, :48], {k: v.double() for k, v in w.items()})
    assert_close("opm_config1_corner", out[:, :48, :48], ref, rel=2.5e-2)
