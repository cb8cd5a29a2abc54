"""Context-parallel PairMixer blocks on GPUs against the single-GPU modules.

The 1x1 grid runs in-process on one GPU and exercises the staged kernels (rectangular projection / output
stages, fp32-output contraction); the 1x2 / 2x2 / 2x4 grids spawn one process per GPU over NCCL and are skipped
when the box has fewer GPUs.
"""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import helpers as H  # noqa: E402

pytestmark = pytest.mark.gpu


def _run_rank(rank, world, rows, cols, port, n_tokens, blocks, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import bioemu2_b200 as b
        from bioemu2_b200.context_parallel import CPGrid, CPPairMixerModule

        g = torch.Generator().manual_seed(11)
        w = {}
        for i in range(blocks):
            w.update(H.prefixed(f"layers.{i}", H.pairmixer_layer_weights(g, 128, perturbed=False)))
        z = torch.randn(1, n_tokens, n_tokens, 128, generator=g)
        tok = torch.ones(1, n_tokens, dtype=torch.bool)
        tok[0, n_tokens - 5:] = False
        pm = tok[:, :, None] & tok[:, None, :]
        serial = b.PairMixerModule(384, 128, blocks).eval()
        serial.load_state_dict(w, strict=True)
        serial.to(dev)
        with torch.no_grad():
            _, ref = serial(torch.zeros(1, n_tokens, 384, device=dev), z.to(dev), pm.to(dev))
        grid = CPGrid(rows, cols)
        cp = CPPairMixerModule(serial, grid)
        z_loc = grid.shard_pair(z).to(dev)
        m_loc = grid.shard_pair(pm).to(dev)
        ret = cp(z_loc, m_loc)
        torch.cuda.synchronize()
        assert ret.data_ptr() == z_loc.data_ptr()
        ref_loc = grid.shard_pair(ref.cpu()).to(dev)
        num = float((z_loc[0] - ref_loc[0]).abs().max())  # every cell: the update is defined at masked pairs too
        den = float(ref.abs().max())
        q.put((rank, num / den, b._lib.device_status()))
    finally:
        dist.destroy_process_group()


def _launch(rows, cols, n_tokens, blocks=2):
    world = rows * cols
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() + rows * 31 + cols * 17 + n_tokens) % 1500
    procs = [ctx.Process(target=_run_rank, args=(r, world, rows, cols, port, n_tokens, blocks, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    res = [q.get(timeout=5) for _ in range(world)]
    for rank, rel, status in res:
        assert status == 0, f"rank {rank}: device status {status:#x}"
        # sharded vs serial differ only by the bf16 rounding of t after an fp32 cross-rank sum (serial rounds the
        # full sum once as well) and by reduction order
        assert rel < 5e-3, f"rank {rank}: rel {rel}"


def test_cp_1x1_matches_serial():
    _launch(1, 1, 136)


@pytest.mark.parametrize("rows,cols,n_tokens", [(1, 2, 144), (2, 1, 144), (2, 2, 272), (2, 4, 320)])
def test_cp_grid_matches_serial(rows, cols, n_tokens):
    if torch.cuda.device_count() < rows * cols:
        pytest.skip(f"needs {rows * cols} GPUs")
    _launch(rows, cols, n_tokens)


def _run_block_rank(rank, world, rows, cols, port, n, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import bioemu2_b200 as b
        from bioemu2_b200.context_parallel import (CPConditionedTransformerLayer, CPGrid, CPOuterProductMean,
                                                   CPPairformerBlock, CPPairMixerMSALayer, shard_range)

        torch.manual_seed(21)  # same seed on every rank: replicated weights
        blk = b.PairformerBlock().eval().to(dev)
        opm = b.OuterProductMean(64, 32, 128).eval().to(dev)
        msa = b.PairMixerMSALayer(token_s=384, msa_s=64, token_z=128).eval().to(dev)
        tokblk = b.ConditionedTransformerLayer(dim=768, dim_pairwise=128, dim_cond=768, heads=16, transition_hidden=3072,
                                               lns_scale=0.5).eval().to(dev)
        with torch.no_grad():
            tokblk.attention.pair_bias_attn.proj_q_bias.normal_(0.0, 0.02)
        g = torch.Generator().manual_seed(22)
        z = torch.randn(1, n, n, 128, generator=g)
        s = torch.randn(1, n, 384, generator=g)
        tok = torch.ones(1, n, dtype=torch.bool)
        tok[0, n - 6:] = False
        S = 16 * rows
        m = torch.randn(1, S, n, 64, generator=g)
        mm = torch.ones(1, S, n, dtype=torch.bool)
        mm[0, 3] = False
        mm[0, :, n - 6:] = False
        a = torch.randn(2, n, 768, generator=g)       # token stream with multiplicity 2
        c = torch.randn(2, n, 768, generator=g)
        with torch.no_grad():
            s_ref, z_ref = blk(s.to(dev), z.to(dev), tok.to(dev))
            o_ref = opm(m.to(dev), mm.to(dev))
            a_ref = tokblk(a.to(dev), z.to(dev), c.to(dev), tok.to(dev), multiplicity=2)
        grid = CPGrid(rows, cols)
        cpb = CPPairformerBlock(blk, grid)
        z_loc, s_loc = grid.shard_pair(z).to(dev), grid.shard_single(s).to(dev)
        (r0, r1), (c0, c1) = grid.coords.my_rows(n), grid.coords.my_cols(n)
        with torch.no_grad():
            s_out, z_out = cpb(s_loc, z_loc, tok[:, r0:r1].to(dev), tok[:, c0:c1].to(dev))
            s0, s1 = shard_range(S, rows, grid.coords.r)
            o_out = CPOuterProductMean(opm, grid)(m[:, s0:s1, c0:c1].contiguous().to(dev),
                                                   mm[:, s0:s1, c0:c1].contiguous().to(dev), mm.any(-1).sum(1).to(dev))
            # the diffusion module's token block on the ORIGINAL pair block, with and without the static bias
            cpt = CPConditionedTransformerLayer(tokblk, grid)
            z_blk = grid.shard_pair(z).to(dev)
            a_loc, c_loc, t_loc = a[:, r0:r1].contiguous().to(dev), c[:, r0:r1].contiguous().to(dev), tok[:, r0:r1].to(dev)
            a_out = cpt(a_loc, z_blk, c_loc, t_loc, 2)
            cpt.attention.prepare_static(z_blk)
            a_out_static = cpt(a_loc, z_blk, c_loc, t_loc, 2)
            # the MSA block: pair-weighted averaging, MSA transition, outer product mean, triangle multiplications
            pm = tok[:, :, None] & tok[:, None, :]
            z2_ref, m2_ref = msa(None, z.to(dev), m.to(dev), pm.to(dev), mm.to(dev))[1:]
            z2_loc = grid.shard_pair(z).to(dev)
            z2_out, m2_out = CPPairMixerMSALayer(msa, grid)(
                z2_loc, m[:, s0:s1, c0:c1].contiguous().to(dev), grid.shard_pair(pm).to(dev),
                mm[:, s0:s1, c0:c1].contiguous().to(dev), mm.any(-1).sum(1).to(dev))
            assert z2_out.data_ptr() == z2_loc.data_ptr()
        torch.cuda.synchronize()
        rel = lambda x, e: float((x - e).abs().max() / e.abs().max())  # noqa: E731  (every cell, masked ones included)
        errs = {
            "z": rel(z_out[0], z_ref[0, r0:r1, c0:c1]),
            "s": rel(s_out[0], s_ref[0, r0:r1]),
            "opm": rel(o_out[0], o_ref[0, r0:r1, c0:c1]),
            "token_block": rel(a_out, a_ref[:, r0:r1]),
            "token_block_static_bias": rel(a_out_static, a_ref[:, r0:r1]),
            "msa_layer_z": rel(z2_out[0], z2_ref[0, r0:r1, c0:c1]),
            "msa_layer_m": rel(m2_out[0], m2_ref[0, s0:s1, c0:c1]),
        }
        q.put((rank, errs, b._lib.device_status()))
    finally:
        dist.destroy_process_group()


def _launch_block(rows, cols, n):
    world = rows * cols
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 30200 + (os.getpid() + rows * 31 + cols * 17 + n) % 1500
    procs = [ctx.Process(target=_run_block_rank, args=(r, world, rows, cols, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    for _ in range(world):
        rank, errs, status = q.get(timeout=5)
        assert status == 0, f"rank {rank}: device status {status:#x}"
        # sharded vs single-GPU: same kernels on differently shaped slabs; bf16 roundings fall at other places
        assert max(errs.values()) < 1e-2, (rank, errs)


def test_cp_pairformer_block_and_opm_1x1():
    _launch_block(1, 1, 136)


@pytest.mark.parametrize("rows,cols,n", [(1, 2, 144), (2, 2, 272), (2, 4, 320)])
def test_cp_pairformer_block_and_opm_grid(rows, cols, n):
    if torch.cuda.device_count() < rows * cols:
        pytest.skip(f"needs {rows * cols} GPUs")
    _launch_block(rows, cols, n)


# --------------------------------------------------------------------------------------------------------------
# The recycling trunk (pair initialisation, recycling update, MSA module, PairMixer blocks) on a grid
def _run_embedder_rank(rank, world, rows, cols, port, n, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import bioemu2_b200 as b
        from bioemu2_b200.context_parallel import CPGrid, CPPairMixerSequenceEmbedder, shard_range

        torch.manual_seed(31)  # same seed on every rank: replicated weights
        emb = b.PairMixerSequenceEmbedder(384, 128, 100, msa_s=64, msa_blocks=2, num_blocks=2).eval().to(dev)
        g = torch.Generator().manual_seed(32)
        S = 8 * rows
        s_inputs = torch.randn(1, n, 100, generator=g)
        terms = torch.randn(1, n, n, 128, generator=g)
        tok = torch.ones(1, n, dtype=torch.bool)
        tok[0, n - 7:] = False
        msa = torch.nn.functional.one_hot(torch.randint(0, 33, (1, S, n), generator=g), 33).float()
        msa_mask = tok[:, None, :].expand(1, S, n).clone()
        msa_mask[0, 2] = False
        feats = dict(msa=msa, msa_mask=msa_mask, has_deletion=(torch.rand(1, S, n, generator=g) < 0.2).float(),
                     deletion_value=torch.rand(1, S, n, generator=g), msa_paired=(torch.rand(1, S, n, generator=g) < 0.5).float(),
                     token_pad_mask=tok, pair_init_terms=terms)
        with torch.no_grad():
            s_ref, z_ref = emb(s_inputs.to(dev), {k: v.to(dev) for k, v in feats.items()}, num_steps_recycle=1)
        grid = CPGrid(rows, cols)
        (r0, r1), (c0, c1) = grid.coords.my_rows(n), grid.coords.my_cols(n)
        s0, s1 = shard_range(S, rows, grid.coords.r)
        local = {k: v[:, s0:s1, c0:c1].contiguous().to(dev) for k, v in feats.items() if k not in ("token_pad_mask", "pair_init_terms")}
        local["token_pad_mask"] = tok.to(dev)
        local["pair_init_terms"] = terms[:, r0:r1, c0:c1].contiguous().to(dev)
        with torch.no_grad():
            s_out, z_out = CPPairMixerSequenceEmbedder(emb, grid)(s_inputs.to(dev), local, num_steps_recycle=1)
        torch.cuda.synchronize()
        rel = lambda x, e: float((x - e).abs().max() / e.abs().max())  # noqa: E731
        q.put((rank, {"s": rel(s_out, s_ref), "z": rel(z_out[0], z_ref[0, r0:r1, c0:c1])}, b._lib.device_status()))
    finally:
        dist.destroy_process_group()


def _launch_embedder(rows, cols, n):
    world = rows * cols
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31900 + (os.getpid() + rows * 31 + cols * 17 + n) % 1500
    procs = [ctx.Process(target=_run_embedder_rank, args=(r, world, rows, cols, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    for _ in range(world):
        rank, errs, status = q.get(timeout=5)
        assert status == 0, f"rank {rank}: device status {status:#x}"
        assert max(errs.values()) < 1e-2, (rank, errs)


def test_cp_sequence_embedder_1x1():
    _launch_embedder(1, 1, 136)


@pytest.mark.parametrize("rows,cols,n", [(1, 2, 144), (2, 2, 272)])
def test_cp_sequence_embedder_grid(rows, cols, n):
    if torch.cuda.device_count() < rows * cols:
        pytest.skip(f"needs {rows * cols} GPUs")
    _launch_embedder(rows, cols, n)
