"""Empty inputs (no tokens, no batch items, no MSA rows, no windows): every module returns the empty result the torch
reference would, without launching a kernel."""
import pytest
import torch

pytestmark = pytest.mark.gpu

E = lambda *shape, dtype=torch.float32: torch.empty(*shape, dtype=dtype, device="cuda")  # noqa: E731


def _cases():
    import bioemu2_b200 as b

    dev = "cuda"
    tm = b.TriangleMultiplication(128, "outgoing").eval().to(dev)
    ta = b.TriangleAttentionStartingNode().eval().to(dev)
    tr, tr2 = b.Transition(128, 512).eval().to(dev), b.Transition(384, 1536).eval().to(dev)
    apb = b.AttentionPairBias(384, 128, 16).eval().to(dev)
    opm = b.OuterProductMean(64, 32, 128).eval().to(dev)
    pwa = b.PairWeightedAveraging(64, 128, 32, 8).eval().to(dev)
    win = b.AttentionPairBiasSlidingWindow(128, 16, 4).eval().to(dev)
    cond = b.PairwiseConditioning(128, 128).eval().to(dev)
    blk = b.PairformerBlock().eval().to(dev)
    tok = b.ConditionedTransformerLayer(dim=768, dim_pairwise=128, dim_cond=768, heads=16, transition_hidden=3072).eval().to(dev)
    B_ = torch.bool
    return {
        "trimul_no_tokens": (lambda: tm(E(1, 0, 0, 128), E(1, 0, 0, dtype=B_)), (1, 0, 0, 128)),
        "trimul_no_batch": (lambda: tm(E(0, 16, 16, 128), E(0, 16, 16, dtype=B_)), (0, 16, 16, 128)),
        "trimul_in_place": (lambda: tm.forward_residual_(E(1, 0, 0, 128), E(1, 0, 0, dtype=B_)), (1, 0, 0, 128)),
        "triatt_no_tokens": (lambda: ta(E(1, 0, 0, 128), E(1, 0, 0, dtype=B_)), (1, 0, 0, 128)),
        "transition_pair": (lambda: tr(E(1, 0, 0, 128)), (1, 0, 0, 128)),
        "transition_single": (lambda: tr2(E(2, 0, 384)), (2, 0, 384)),
        "apb_no_tokens": (lambda: apb(E(1, 0, 384), E(1, 0, 0, 128), E(1, 0, dtype=B_)), (1, 0, 384)),
        "opm_no_tokens": (lambda: opm(E(1, 4, 0, 64), E(1, 4, 0, dtype=B_)), (1, 0, 0, 128)),
        "pwa_no_rows": (lambda: pwa(E(1, 0, 16, 64), torch.randn(1, 16, 16, 128, device=dev),
                                    torch.ones(1, 16, 16, dtype=B_, device=dev)), (1, 0, 16, 64)),
        "pwa_no_tokens": (lambda: pwa(E(1, 3, 0, 64), E(1, 0, 0, 128), E(1, 0, 0, dtype=B_)), (1, 3, 0, 64)),
        "window_no_windows": (lambda: win(E(0, 32, 128), E(1, 0, 32, 128, 16), E(0, 32, dtype=B_)), (0, 32, 128)),
        "pairwise_conditioning": (lambda: cond(E(1, 0, 0, 128), E(1, 0, 0, 128)), (1, 0, 0, 128)),
        "pairformer_block": (lambda: blk(E(1, 0, 384), E(1, 0, 0, 128), E(1, 0, dtype=B_))[1], (1, 0, 0, 128)),
        "token_block": (lambda: tok(E(2, 0, 768), E(1, 0, 0, 128), E(2, 0, 768), E(1, 0, dtype=B_), multiplicity=2), (2, 0, 768)),
    }


def test_empty_inputs_give_empty_outputs_without_launches():
    import bioemu2_b200 as b

    with torch.no_grad():
        cases = _cases()
        torch.cuda.synchronize()
        n0 = b._lib.launch_count()
        for name, (fn, shape) in cases.items():
            out = fn()
            assert tuple(out.shape) == shape, (name, tuple(out.shape))
        torch.cuda.synchronize()
    assert b._lib.launch_count() == n0, "an empty input must not launch a kernel"
    assert b._lib.device_status() == 0


def test_outer_product_mean_without_msa_rows_is_the_output_bias():
    """The mean over no rows is zero (the reference divides by a count clamped to 1), so proj_o's bias is what is left."""
    import bioemu2_b200 as b

    opm = b.OuterProductMean(64, 32, 128).eval().cuda()
    with torch.no_grad():
        opm.proj_o.bias.normal_()
        out = opm(E(1, 0, 9, 64), E(1, 0, 9, dtype=torch.bool))
    assert tuple(out.shape) == (1, 9, 9, 128)
    assert torch.equal(out, opm.proj_o.bias.expand(1, 9, 9, 128))
