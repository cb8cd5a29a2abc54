"""Pin the CPU oracle: against the golden vectors the reference's modules produced,
and -- where the reference checkout is present -- against those modules run live."""
from __future__ import annotations

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import cases as C  # noqa: E402
from oracle import pair_ops as O  # noqa: E402
from oracle import reference_shim  # noqa: E402
from helpers import rel_err  # noqa: E402

GOLDEN = torch.load(C.GOLDEN_PATH)

FP32_REL = 1e-4  # the stated fp32 bar; the oracle is far inside it (reductions reorder only)


def run_oracle(case: dict, dtype=torch.float32) -> torch.Tensor:
    w = {k: v.to(dtype) for k, v in case["w"].items()}
    f = lambda t: t.to(dtype)  # noqa: E731
    kind = case["kind"]
    if kind == "trimul":
        return O.triangle_multiplication(f(case["x"]), case["mask"], w, case["mode"])
    if kind == "transition":
        return O.transition(f(case["x"]), w)
    if kind == "apb":
        return O.attention_pair_bias(f(case["s"]), f(case["z"]), case["mask"], w, case["heads"], case["M"])
    if kind == "opm":
        return O.outer_product_mean(f(case["m"]), case["mask"], w)
    if kind == "pairmixer":
        return O.pairmixer_layer(f(case["z"]), case["pair_mask"], w)
    if kind == "cond_layer":
        return O.conditioned_transformer_layer(f(case["x"]), f(case["z"]), f(case["c"]), case["mask"], w,
                                               case["heads"], case["M"], case["lns_scale"])
    if kind == "pwa":
        return O.pair_weighted_averaging(f(case["m"]), f(case["z"]), case["mask"], w)
    if kind == "msa_layer":
        z, m = O.pairmixer_msa_layer(f(case["z"]), f(case["m"]), case["pair_mask"], case["msa_mask"], w)
        return torch.cat([z.flatten(), m.flatten()])
    if kind == "pairwise_conditioning":
        return O.pairwise_conditioning(f(case["z"]), f(case["rel"]), w)
    if kind == "msa_module":
        return O.pairmixer_msa_module(f(case["z"]), f(case["emb"]), _feats(case, dtype), w, case["blocks"])
    if kind == "sequence_trunk":
        s, z = O.sequence_trunk(f(case["s_inputs"]), f(case["pair_terms"]), _feats(case, dtype), w, recycles=case["recycles"],
                                msa_blocks=case["msa_blocks"], num_blocks=case["num_blocks"],
                                unconditional=case["unconditional"])
        return torch.cat([z.flatten(), s.flatten()])
    if kind == "window_apb":
        return O.attention_pair_bias_sliding_window(f(case["s"]), f(case["z"]), case["mask"], w, case["heads"], case["M"])
    raise KeyError(kind)


def _feats(case: dict, dtype) -> dict:
    return {k: (v if v.dtype == torch.bool else v.to(dtype)) for k, v in case["feats"].items()}


@pytest.mark.parametrize("name", sorted(C.CASES))
def test_inputs_reproducible(name):
    case = C.CASES[name]()
    assert C.checksum(C.case_tensors(case)) == pytest.approx(GOLDEN[name]["input_checksum"], rel=1e-9, abs=1e-9), (
        "seeded inputs differ from the ones the golden file was generated with")


@pytest.mark.parametrize("name", sorted(C.CASES))
def test_oracle_matches_golden(name):
    case = C.CASES[name]()
    got = run_oracle(case, torch.float64)
    assert rel_err(got, GOLDEN[name]["output"]) < 2e-6
    got32 = run_oracle(case, torch.float32)
    assert rel_err(got32, GOLDEN[name]["output"]) < FP32_REL


@pytest.mark.skipif(not reference_shim.available(), reason="reference checkout not on this machine")
@pytest.mark.parametrize("name", sorted(C.CASES))
def test_oracle_matches_live_reference(name):
    import make_golden

    case = C.CASES[name]()
    ref = make_golden.run_reference(case)
    assert rel_err(run_oracle(case, torch.float32), ref) < 1e-5


def test_trimul_masked_inputs_do_not_leak():
    """Poisoned masked inputs leave valid outputs unchanged
    (tests/biomoa/ops/test_triangle_multiplication.py:373-388 in the reference)."""
    case = C.trimul_case("outgoing")
    x = case["x"].double()
    w = {k: v.double() for k, v in case["w"].items()}
    poisoned = x.clone()
    poisoned[~case["mask"]] = 1000.0
    a = O.triangle_multiplication(x, case["mask"], w, "outgoing")
    b = O.triangle_multiplication(poisoned, case["mask"], w, "outgoing")
    # the output gate reads LN(x) of every pair, so only compare where x is untouched
    assert torch.equal(a[case["mask"]], b[case["mask"]])


def test_triangle_attention_ending_is_transposed_starting():
    import helpers as Hh

    g = torch.Generator().manual_seed(5)
    w = {k: v.double() for k, v in Hh.triatt_weights(g).items()}
    x = torch.randn(1, 12, 12, 128, generator=g).double()
    mask = torch.rand(1, 12, 12, generator=g) > 0.2
    a = O.triangle_attention(x, mask, w, 4, ending=True)
    b = O.triangle_attention(x.transpose(1, 2), mask.transpose(1, 2), w, 4, ending=False).transpose(1, 2)
    assert torch.equal(a, b)
