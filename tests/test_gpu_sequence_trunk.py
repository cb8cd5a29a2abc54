"""The sequence-trunk glue (pair initialisation, recycling, MSA module) and PairwiseConditioning on the GPU against the
golden vectors the reference's modules produced and against the CPU oracle."""
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


def _cuda(feats: dict) -> dict:
    return {k: v.cuda() for k, v in feats.items()}


# ------------------------------------------------------------------------------------------ kernels
def test_pair_outer_sum_is_exact():
    from bioemu2_b200 import functional as F

    g = torch.Generator().manual_seed(900)
    a, c = torch.randn(2, 37, 128, generator=g).cuda(), torch.randn(2, 53, 128, generator=g).cuda()
    extra = torch.randn(2, 37, 53, 128, generator=g).cuda()
    assert torch.equal(F.pair_outer_sum(a, c), a[:, :, None] + c[:, None])
    assert torch.equal(F.pair_outer_sum(a, c, extra), (a[:, :, None] + c[:, None]) + extra)


def test_add_rows_plain_and_broadcast():
    from bioemu2_b200 import functional as F

    g = torch.Generator().manual_seed(901)
    x = torch.randn(5, 33, 64, generator=g).cuda()
    y = torch.randn(5, 33, 64, generator=g).cuda()
    yb = torch.randn(33, 64, generator=g).cuda()
    assert torch.equal(F.add_rows(x, y), x + y)
    assert torch.equal(F.add_rows(x, yb), x + yb)
    assert torch.equal(F.add_rows(x, y.bfloat16()), x + y.bfloat16().float())
    x0 = x.clone()
    assert F.add_rows(x, yb, out=x) is x and torch.equal(x, x0 + yb)


def test_two_source_layernorm_matches_the_concatenation():
    from bioemu2_b200 import functional as F

    g = torch.Generator().manual_seed(902)
    x1, x2 = torch.randn(301, 128, generator=g) * 2 + 0.5, torch.randn(301, 136, generator=g)
    w, b = torch.randn(264, generator=g), torch.randn(264, generator=g)
    want = torch.nn.functional.layer_norm(torch.cat([x1, x2], -1).double(), (264,), w.double(), b.double())
    got = F.rows2_to_bf16(x1.cuda(), x2.cuda(), w.cuda(), b.cuda())
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == (301, 264)
    assert_close("rows2_to_bf16", got, want)
    one = F.rows_to_bf16(torch.cat([x1, x2], -1).cuda(), w.cuda(), b.cuda())
    assert torch.equal(got, one)  # same arithmetic as the one-source kernel on the materialised concatenation


# ------------------------------------------------------------------------------------------ PairwiseConditioning
def _cond(w):
    import bioemu2_b200 as b

    m = b.PairwiseConditioning(token_z=128, dim_token_rel_pos_feats=128).eval()
    m.load_state_dict(w, strict=True)
    return m.cuda()


def test_pairwise_conditioning_golden():
    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES["pairwise_conditioning"]()
    mod = _cond(case["w"])
    z, rel = case["z"].cuda(), case["rel"].cuda()
    z0 = z.clone()
    with torch.no_grad():
        out = mod(z, rel)
    assert out.dtype == torch.float32 and torch.equal(z, z0)
    assert_close("pairwise_conditioning_golden", out, golden["pairwise_conditioning"]["output"], atol=4e-2)


@pytest.mark.parametrize("N", [72, 200])
def test_pairwise_conditioning_vs_oracle(N):
    g = torch.Generator().manual_seed(910 + N)
    w = H.pairwise_conditioning_weights(g)
    z = torch.randn(1, N, N, 128, generator=g)
    rel = torch.randn(1, N, N, 128, generator=g)
    ref = O.pairwise_conditioning(z.double(), rel.double(), {k: v.double() for k, v in w.items()})
    with torch.no_grad():
        out = _cond(w)(z.cuda(), rel.cuda())
    assert_close(f"pairwise_conditioning_N{N}", out, ref, atol=4e-2)


# ------------------------------------------------------------------------------------------ MSA module, trunk
def test_msa_module_golden():
    import bioemu2_b200 as b

    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES["msa_module"]()
    mod = b.PairMixerMSAModule(token_s=384, msa_s=64, token_z=128, s_input_dim=case["emb"].shape[-1],
                               msa_blocks=case["blocks"], use_paired_feature=True).eval()
    mod.load_state_dict(case["w"], strict=True)
    mod.cuda()
    f = _cuda(case["feats"])
    with torch.no_grad():
        s, z = mod(None, case["z"].cuda(), case["emb"].cuda(), f["msa"], f["msa_mask"], f["has_deletion"],
                   f["deletion_value"], f["msa_paired"], f["token_pad_mask"])
    assert s is None
    # two MSA blocks = eight residual updates of the pair tensor
    assert_close("msa_module_golden", z, golden["msa_module"]["output"], atol=4e-2)


def _embedder(case):
    import bioemu2_b200 as b

    mod = b.PairMixerSequenceEmbedder(token_s=384, token_z=128, s_input_dim=case["s_inputs"].shape[-1], msa_s=64,
                                      msa_blocks=case["msa_blocks"], num_blocks=case["num_blocks"],
                                      use_paired_feature=True, use_unconditional_branch=True).eval()
    mod.load_state_dict(case["w"], strict=True)
    return mod.cuda()


@pytest.mark.parametrize("name", ["sequence_trunk", "sequence_trunk_unconditional"])
def test_sequence_trunk_golden(name):
    """One recycle (two passes through the MSA block and the PairMixer block) and the unconditional branch; the
    encoders' pair terms enter through ``feats["pair_init_terms"]``."""
    golden = torch.load(C.GOLDEN_PATH)
    case = C.CASES[name]()
    mod = _embedder(case)
    feats = dict(_cuda(case["feats"]), pair_init_terms=case["pair_terms"].cuda())
    with torch.no_grad():
        s, z = mod(case["s_inputs"].cuda(), feats, num_steps_recycle=case["recycles"], unconditional=case["unconditional"])
    want = golden[name]["output"]
    nz = z.numel()
    assert s.dtype == torch.float32 and z.dtype == torch.float32
    assert_close(f"{name}_z", z.flatten(), want[:nz], atol=4e-2)
    assert_close(f"{name}_s", s.flatten(), want[nz:], atol=4e-2)


def test_sequence_trunk_encoders_are_called_like_the_reference():
    """Feature encoders assigned to the module are called with the reference's keyword arguments and summed."""
    import bioemu2_b200 as b

    case = C.CASES["sequence_trunk_unconditional"]()
    mod = _embedder(case)
    seen = {}

    class RelPos(torch.nn.Module):
        def forward(self, asym_id, entity_id, residue_index, sym_id):
            seen["rel_pos"] = (asym_id, entity_id, residue_index, sym_id)
            return case["pair_terms"].cuda() * 0.25

    class Bonds(torch.nn.Module):
        def forward(self, token_bonds):
            seen["token_bonds"] = token_bonds
            return case["pair_terms"].cuda() * 0.75

    feats = dict(_cuda(case["feats"]), asym_id=1, entity_id=2, residue_index=3, sym_id=4, token_bonds=5)
    with torch.no_grad():
        want = mod(case["s_inputs"].cuda(), dict(feats, pair_init_terms=case["pair_terms"].cuda()), unconditional=True)
        mod.rel_pos, mod.token_bonds = RelPos(), Bonds()
        got = mod(case["s_inputs"].cuda(), feats, unconditional=True)
    assert seen == {"rel_pos": (1, 2, 3, 4), "token_bonds": 5}
    assert "rel_pos" in dict(mod.named_children())
    torch.testing.assert_close(got[1], want[1], atol=1e-5, rtol=1e-5)
    assert isinstance(mod, b.PairMixerSequenceEmbedder)


def test_sequence_trunk_argument_errors():
    case = C.CASES["sequence_trunk"]()
    mod = _embedder(case)
    feats = _cuda(case["feats"])
    with pytest.raises(ValueError, match="non-negative"):
        mod(case["s_inputs"].cuda(), feats, num_steps_recycle=-1)
    mod.use_unconditional_branch = False
    with pytest.raises(ValueError, match="use_unconditional_branch"):
        mod(case["s_inputs"].cuda(), feats, unconditional=True)


def test_context_parallel_wrappers_of_the_per_pair_glue():
    """The per-pair ops need no exchange: the wrappers run the serial kernels on a rank's block, so a block of the
    full result equals the result on the block."""
    import bioemu2_b200 as b
    from bioemu2_b200.context_parallel import ops

    g = torch.Generator().manual_seed(920)
    w = H.pairwise_conditioning_weights(g)
    serial = _cond(w)
    z = torch.randn(1, 96, 96, 128, generator=g).cuda()
    rel = torch.randn(1, 96, 96, 128, generator=g).cuda()
    with torch.no_grad():
        full = serial(z, rel)
        blk = ops.DistributedPairwiseConditioning(serial)(z[:, 48:, :40].contiguous(), rel[:, 48:, :40].contiguous())
        assert torch.equal(blk, full[:, 48:, :40])
        tiled = ops.LayerNormLinearParamsReplicatedTiled(serial.dim_pairwise_init_proj)
        assert sorted(tiled.state_dict()) == ["0.bias", "0.weight", "1.weight"]
        proj = tiled(z, rel)
        ln = serial.dim_pairwise_init_proj[0]
        want = torch.nn.functional.linear(
            torch.nn.functional.layer_norm(torch.cat([z, rel], -1).double(), (256,), ln.weight.double(), ln.bias.double()),
            serial.dim_pairwise_init_proj[1].weight.double())
        assert_close("ln_linear_tiled", proj, want)
    with pytest.raises(RuntimeError, match="forward-only"):
        tiled(z, rel)
    assert isinstance(serial, b.PairwiseConditioning)
