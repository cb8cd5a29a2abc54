"""``trunk.graphed(...)``: the block loop captured in a CUDA graph gives the eager forward's result, follows new inputs
and new masks, and refuses other shapes."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import helpers as H  # noqa: E402

pytestmark = pytest.mark.gpu


def test_graphed_pairformer_trunk_matches_eager():
    import bioemu2_b200 as b

    torch.manual_seed(41)
    trunk = b.PairformerModule(384, 128, 3).eval().cuda()
    g = torch.Generator().manual_seed(42)
    N = 72
    s, z = torch.randn(1, N, 384, generator=g), torch.randn(1, N, N, 128, generator=g)
    tok = torch.ones(1, N, dtype=torch.bool)
    tok[0, N - 5:] = False
    with torch.no_grad():
        s_ref, z_ref = trunk(s.cuda(), z.cuda(), tok.cuda())
        gt = trunk.graphed(s.cuda(), z.cuda(), tok.cuda())
        n0 = b._lib.launch_count()
        s_out, z_out = gt(s.pin_memory(), z.pin_memory())                       # inputs from pinned host memory
        assert b._lib.launch_count() == n0, "a replay issues no launch from the host"
        assert torch.equal(s_out, s_ref) and torch.equal(z_out, z_ref)
        # new inputs, new mask: the static buffers follow
        s2, z2 = torch.randn(1, N, 384, generator=g).cuda(), torch.randn(1, N, N, 128, generator=g).cuda()
        tok2 = torch.ones(1, N, dtype=torch.bool, device="cuda")
        tok2[0, :3] = False
        s_ref2, z_ref2 = trunk(s2, z2, tok2)
        s_out2, z_out2 = gt(s2, z2, tok2)
        assert torch.equal(s_out2, s_ref2) and torch.equal(z_out2, z_ref2)
        assert s_out2.data_ptr() == s_out.data_ptr(), "outputs live in static buffers"
        with pytest.raises(ValueError, match="captured"):
            gt(s2[:, :64], z2[:, :64, :64])


def test_graphed_pairmixer_trunk_matches_eager():
    import bioemu2_b200 as b

    g = torch.Generator().manual_seed(43)
    w = {}
    for i in range(2):
        w.update(H.prefixed(f"layers.{i}", H.pairmixer_layer_weights(g, 128)))
    trunk = b.PairMixerModule(384, 128, 2).eval()
    trunk.load_state_dict(w, strict=True)
    trunk.cuda()
    N = 40
    z = torch.randn(1, N, N, 128, generator=g).cuda()
    s = torch.zeros(1, N, 384).cuda()
    pm = (torch.rand(1, N, N, generator=g) > 0.2).cuda()
    with torch.no_grad():
        _, z_ref = trunk(s, z, pm)
        _, z_out = trunk.graphed(s, z, pm)(s, z)
    assert torch.equal(z_out, z_ref)


def test_two_stream_trunk_loop_equals_the_serial_loop():
    """``PairformerModule.forward_`` runs each block's single track on a side stream under the next block's pair
    track; the kernels and their inputs are those of the serial loop, so the results are identical."""
    import bioemu2_b200 as b

    torch.manual_seed(44)
    trunk = b.PairformerModule(384, 128, 4).eval().cuda()
    g = torch.Generator().manual_seed(45)
    N = 136
    s, z = torch.randn(2, N, 384, generator=g).cuda(), torch.randn(2, N, N, 128, generator=g).cuda()
    tok = torch.ones(2, N, dtype=torch.bool, device="cuda")
    tok[0, N - 9:] = False
    pm = (tok[:, :, None] & tok[:, None, :]).to(torch.uint8)
    with torch.no_grad():
        s1, z1 = trunk.forward_(s.clone(), z.clone(), tok, pm, overlap=True)
        s2, z2 = trunk.forward_(s.clone(), z.clone(), tok, pm, overlap=False)
        torch.cuda.synchronize()
    assert torch.equal(z1, z2) and torch.equal(s1, s2)
