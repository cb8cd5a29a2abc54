"""``swap_into`` on the reference's own modules (imported in place where the checkout exists): every recognised op is
replaced by its twin with the same constructor attributes and an identical ``state_dict``."""
import pytest
import torch
import torch.nn as nn

from oracle import reference_shim

pytestmark = pytest.mark.skipif(not reference_shim.available(), reason="reference checkout not on this machine")


def _same_state(a: nn.Module, b_sd: dict) -> None:
    sd = a.state_dict()
    assert list(sd) == list(b_sd)
    for k in sd:
        assert sd[k].shape == b_sd[k].shape and torch.equal(sd[k], b_sd[k]), k


def test_swap_replaces_every_reference_op_and_keeps_the_weights():
    import bioemu2_b200 as b

    R = reference_shim.modules()
    torch.manual_seed(0)

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.trunk = R.PairMixerModule(token_s=384, token_z=128, num_blocks=2, trimul_variant="full")
            self.apb = R.AttentionPairBias(c_s=384, c_z=128, num_heads=16)
            self.apb_token = R.AttentionPairBias(c_s=768, c_z=128, num_heads=16, initial_norm=False)
            self.single = R.Transition(dim=384, hidden=1536)
            self.opm = R.OuterProductMeanVanilla(c_in=64, c_hidden=32, c_out=128)
            self.narrow = R.TriangleMultiplicationFull(dim=64, mode="outgoing")  # a width the kernels do not serve
            self.other = nn.Linear(8, 8)

    model = Model().eval()
    before = {k: v.clone() for k, v in model.state_dict().items()}
    report = b.swap_into(model)

    for i in range(2):
        layer = model.trunk.layers[i]
        assert isinstance(layer.tri_mul_out, b.TriangleMultiplication) and layer.tri_mul_out.mode == "outgoing"
        assert isinstance(layer.tri_mul_in, b.TriangleMultiplication) and layer.tri_mul_in.mode == "incoming"
        assert isinstance(layer.transition_z, b.Transition) and layer.transition_z.hidden == 512
    assert isinstance(model.apb, b.AttentionPairBias)
    assert (model.apb.c_s, model.apb.c_z, model.apb.num_heads, model.apb.initial_norm) == (384, 128, 16, True)
    assert isinstance(model.apb_token, b.AttentionPairBias) and not model.apb_token.initial_norm
    assert isinstance(model.single, b.Transition) and model.single.use_norm
    assert isinstance(model.opm, b.OuterProductMean) and model.opm.c_hidden == 32
    assert type(model.narrow).__module__.startswith("bioemu2.biomoa")     # left in place ...
    assert report["narrow"][1].startswith("kept:")                        # ... and reported
    assert isinstance(model.other, nn.Linear)
    assert report["trunk.layers.0.tri_mul_out"] == ("TriangleMultiplicationFull", "TriangleMultiplication")
    _same_state(model, before)
    assert all(not m.training for m in model.modules())
    # a second pass finds nothing left to do
    assert [k for k, v in b.swap_into(model).items() if not v[1].startswith("kept:")] == []


def test_strict_swap_raises_on_an_unsupported_width():
    import bioemu2_b200 as b

    R = reference_shim.modules()
    with pytest.raises(ValueError, match="dim=128"):
        b.swap_into(nn.Sequential(R.TriangleMultiplicationFull(dim=64, mode="incoming")), strict=True)


def test_context_parallel_wrappers_adopt_reference_layers():
    """The reference-style constructors accept the reference's serial layers and carry their weights over."""
    import bioemu2_b200 as b
    from bioemu2_b200.context_parallel import ops

    R = reference_shim.modules()
    torch.manual_seed(1)
    ref_tm = R.TriangleMultiplicationFull(dim=128, mode="incoming")
    own = ops.adopt_trimul(ref_tm, "incoming")
    assert isinstance(own, b.TriangleMultiplication) and own.mode == "incoming"
    _same_state(own, ref_tm.state_dict())
    ref_apb = R.AttentionPairBias(c_s=384, c_z=128, num_heads=16)
    _same_state(ops.adopt_apb(ref_apb), ref_apb.state_dict())
    ref_tr = R.Transition(dim=128, hidden=512)
    _same_state(ops.adopt_transition(ref_tr), ref_tr.state_dict())
    ref_opm = R.OuterProductMeanVanilla(c_in=64, c_hidden=32, c_out=128)
    _same_state(ops.adopt_opm(ref_opm), ref_opm.state_dict())
    with pytest.raises(ValueError, match="Invalid direction"):
        ops._mode_of("sideways")


def test_swap_takes_the_composite_modules_whole():
    """``PairwiseConditioning`` and ``PairMixerSequenceEmbedder`` (with its MSA module) are replaced glue and all; the
    embedder's feature encoders move across as the reference's own objects and the state dict is unchanged."""
    import bioemu2_b200 as b

    reference_shim.install()
    from bioemu2.biomoa.modules.diffusion import PairwiseConditioning
    from bioemu2.biomoa.modules.pairmixer import PairMixerSequenceEmbedder

    torch.manual_seed(2)

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.embedder = PairMixerSequenceEmbedder(
                token_s=384, token_z=128, s_input_dim=100, msa_s=64, msa_blocks=2, num_blocks=2, trimul_variant="full",
                opm_variant="vanilla", use_contact_conditioning=False, use_method_conditioning=False,
                use_paired_feature=True, use_unconditional_branch=True)
            self.cond = PairwiseConditioning(token_z=128, dim_token_rel_pos_feats=128)

    model = Model().eval()
    before = {k: v.clone() for k, v in model.state_dict().items()}
    rel_pos, token_bonds = model.embedder.rel_pos, model.embedder.token_bonds
    report = b.swap_into(model)
    assert report["embedder"] == ("PairMixerSequenceEmbedder", "PairMixerSequenceEmbedder")
    assert report["cond"] == ("PairwiseConditioning", "PairwiseConditioning")
    e, c = model.embedder, model.cond
    assert isinstance(e, b.PairMixerSequenceEmbedder) and isinstance(e.msa_module, b.PairMixerMSAModule)
    assert e.rel_pos is rel_pos and e.token_bonds is token_bonds
    assert (e.token_s, e.token_z, e.s_input_dim, e.use_unconditional_branch) == (384, 128, 100, True)
    assert len(e.msa_module.layers) == 2 and len(e.pairmixer_module.layers) == 2 and e.msa_module.use_paired_feature
    assert isinstance(e.msa_module.layers[0].pair_weighted_averaging, b.PairWeightedAveraging)
    assert isinstance(c, b.PairwiseConditioning) and (c.token_z, c.dim_token_rel_pos_feats, c.a_z) == (128, 128, 128)
    assert len(c.transitions) == 2 and c.transitions[0].hidden == 256
    sd = model.state_dict()
    assert sorted(sd) == sorted(before)
    for k in before:
        assert torch.equal(sd[k], before[k]), k


def test_swap_recognises_the_sliding_window_attention():
    import bioemu2_b200 as b

    reference_shim.install()
    from bioemu2.biomoa.ops.attention_pair_bias import AttentionPairBiasSlidingWindow

    torch.manual_seed(3)
    model = nn.Sequential(AttentionPairBiasSlidingWindow(128, 16, 4, window_queries=32, window_keys=128)).eval()
    before = {k: v.clone() for k, v in model.state_dict().items()}
    report = b.swap_into(model)
    twin = model[0]
    assert report["0"] == ("AttentionPairBiasSlidingWindow", "AttentionPairBiasSlidingWindow")
    assert isinstance(twin, b.AttentionPairBiasSlidingWindow)
    assert (twin.c_s, twin.c_z, twin.num_heads, twin.window_queries, twin.window_keys) == (128, 16, 4, 32, 128)
    _same_state(model, before)
