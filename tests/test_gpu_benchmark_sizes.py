"""Parity at the sizes the benchmark quotes its numbers on.

The other GPU tests use small ragged shapes; these run the inputs ``bench.py`` itself builds (same seeds, same
padding) and compare with the fp32 CPU oracle, every cell, masked cells included (the reference defines the update
there too).  Where the whole oracle would take the CPU minutes (N = 1536) a slab of attention lines / output rows is
checked, which exercises the same kernels on the full-size operands.
"""
import pytest
import torch

import bench
import helpers as H
from gpu_util import assert_close
from oracle import pair_ops as O

pytestmark = pytest.mark.gpu


def test_pairformer_block_n512_last_37_tokens_padded():
    """One block of the 48-block trunk the headline number is measured on: N = 512, last 37 tokens masked, seed 2."""
    import bioemu2_b200 as b

    w, s, z, tok = bench.workload(512, 1, "pairformer", seed=2)
    assert int((~tok).sum()) == 37
    w0 = O._sub(w, "layers.0")
    with torch.no_grad():
        s_ref, z_ref = O.pairformer_block(s, z, tok, w0, row_chunk=32)
    blk = b.PairformerBlock().eval()
    blk.load_state_dict(w0, strict=True)
    blk.cuda()
    with torch.no_grad():
        s_out, z_out = blk(s.cuda(), z.cuda(), tok.cuda())
    assert_close("pairformer_block_z_N512_pad37", z_out, z_ref)
    assert_close("pairformer_block_s_N512_pad37", s_out, s_ref)


def test_trunk_48_blocks_n128_drift():
    """48 stacked blocks on the GPU (fp32 residual streams, bf16 arithmetic) against 48 fp32 oracle blocks.  The
    reference states its bf16 bar per op; for the depth of the benchmarked trunk the error accumulated over
    48 x 7 residual updates must stay under 2e-2 of the result's largest magnitude, and under 2e-2 in the rms sense.
    (The per-element form |d| <= 2e-2 + 2e-2 |ref| is logged, not asserted: an element near zero in a stream whose
    rms has grown to several units cannot meet an absolute 2e-2 after 336 bf16-rounded updates.)"""
    import bioemu2_b200 as b
    from gpu_util import errors, record

    N, blocks = 128, 48
    w, s, z, tok = bench.workload(N, blocks, "pairformer", seed=2)
    s_ref, z_ref = s, z
    with torch.no_grad():
        for i in range(blocks):
            s_ref, z_ref = O.pairformer_block(s_ref, z_ref, tok, O._sub(w, f"layers.{i}"))
    trunk = b.PairformerModule(384, 128, blocks).eval()
    trunk.load_state_dict(w, strict=True)
    trunk.cuda()
    with torch.no_grad():
        s_out, z_out = trunk(s.cuda(), z.cuda(), tok.cuda())
    assert b._lib.device_status() == 0
    for name, got, ref in (("z", z_out, z_ref), ("s", s_out, s_ref)):
        st = errors(got, ref)
        record(f"pairformer_trunk48_{name}_N128", st)
        assert not st["nan"]
        assert st["rel_max"] <= 2e-2, st
        assert st["rel_rms"] <= 2e-2, st


def test_opm_config1_full_output():
    """m[1,1024,384,64] bf16 with a random 10 % of the MSA rows masked (seed 1): the whole [384,384,128] output."""
    import bioemu2_b200 as b

    w, m, mask = bench.opm_workload()
    with torch.no_grad():
        ref = O.outer_product_mean(m.float(), mask, w, i_chunk=32)
    mod = b.OuterProductMean(64, 32, 128).eval()
    mod.load_state_dict(w, strict=True)
    mod.cuda()
    with torch.no_grad():
        out = mod(m.cuda(), mask.cuda())
    assert out.dtype == torch.bfloat16
    assert_close("opm_config1_full", out, ref, rel=2.5e-2)


@pytest.mark.parametrize("mode", ["outgoing", "incoming"])
def test_trimul_n1536_row_slab(mode):
    """Triangle multiplication at N = 1536 (seed 3, full mask): output rows 700..731 against the oracle."""
    import bioemu2_b200 as b

    N, rows = 1536, slice(700, 732)
    g = torch.Generator().manual_seed(3)
    w = H.trimul_weights(g, perturbed=False)
    z = torch.randn(1, N, N, 128, generator=g)
    mask = torch.ones(1, N, N, dtype=torch.bool)
    with torch.no_grad():
        ref = O.triangle_multiplication(z, mask, w, mode, rows=rows)
    m = b.TriangleMultiplication(128, mode).eval()
    m.load_state_dict(w, strict=True)
    m.cuda()
    with torch.no_grad():
        out = m(z.cuda(), mask.cuda())
    assert_close(f"trimul_{mode}_N1536_rows", out[:, rows], ref)


@pytest.mark.parametrize("ending", [False, True])
def test_triatt_n1536_line_slab(ending):
    """Triangle attention at N = 1536 (seed 3, full mask): 16 attention lines against the oracle."""
    import bioemu2_b200 as b

    N, lines = 1536, slice(1000, 1016)
    g = torch.Generator().manual_seed(3)
    w = H.triatt_weights(g, perturbed=False)
    z = torch.randn(1, N, N, 128, generator=g)
    mask = torch.ones(1, N, N, dtype=torch.bool)
    with torch.no_grad():
        ref = O.triangle_attention(z, mask, w, 4, ending, row_chunk=4, lines=lines)
    m = b.TriangleAttention(ending=ending).eval()
    m.load_state_dict(w, strict=True)
    m.cuda()
    with torch.no_grad():
        out = m(z.cuda(), mask.cuda())
    got = out[:, :, lines] if ending else out[:, lines]
    assert_close(f"triatt_{'end' if ending else 'start'}_N1536_lines", got, ref)
