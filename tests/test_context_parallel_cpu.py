"""Context-parallel host logic on CPU: grid geometry against the reference's own helpers, and the
all-gather / reduce-scatter exchange of triangle multiplication as gloo ranks (world sizes 2 and 4) with the
oracle doing the local arithmetic."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import helpers as H  # noqa: E402
from oracle import pair_ops as O  # noqa: E402
from oracle import reference_shim  # noqa: E402


def test_shard_range_is_torch_chunk():
    from bioemu2_b200.context_parallel import shard_range

    for n in (1, 7, 8, 64, 100, 129):
        for parts in (1, 2, 3, 4, 8):
            chunks = torch.arange(n).chunk(parts)
            for i in range(parts):
                lo, hi = shard_range(n, parts, i)
                expect = chunks[i].tolist() if i < len(chunks) else []
                assert list(range(lo, hi)) == expect


@pytest.mark.skipif(not reference_shim.available(), reason="reference checkout not on this machine")
def test_geometry_matches_reference_helpers():
    """src/bioemu2/context_parallel/utils/mesh.py:17-55 in the reference."""
    reference_shim.install()
    from bioemu2.context_parallel.utils import mesh as ref_mesh

    from bioemu2_b200.context_parallel import pad_amount, shard_multiple, shard_range

    class FakeMesh:  # shard_multiple only asks a DeviceMesh for ndim and size(axis)
        def __init__(self, shape):
            self.shape, self.ndim = shape, len(shape)

        def size(self, i):
            return self.shape[i]

    for g in ((1, 1), (2, 2), (1, 2), (2, 4), (4, 4), (3, 2)):
        assert shard_multiple(*g) == ref_mesh.shard_multiple(FakeMesh((1,) + g))
        assert ref_mesh.pad_amount(37, shard_multiple(*g)) == pad_amount(37, shard_multiple(*g))
    for n in (7, 64, 100):
        for parts in (1, 2, 4):
            for i in range(parts):
                lo, hi = shard_range(n, parts, i)
                assert (lo, hi) == tuple(ref_mesh._shard_range(n, parts, i))


def _worker(rank, world, rows, cols, port, n_tokens, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from bioemu2_b200.context_parallel import CPGrid
        from bioemu2_b200.context_parallel.trimul import cp_triangle_multiplication_
        from cp_cpu_backend import CpuTriMulBackend, OracleWeights

        grid = CPGrid(rows, cols)
        g = torch.Generator().manual_seed(3)
        w_out = {k: v.double() for k, v in H.trimul_weights(g, 16).items()}
        w_in = {k: v.double() for k, v in H.trimul_weights(g, 16).items()}
        z = torch.randn(1, n_tokens, n_tokens, 16, generator=g).double()
        mask = torch.rand(1, n_tokens, n_tokens, generator=g) > 0.25
        ref = z + O.triangle_multiplication(z, mask, w_out, "outgoing")
        ref = ref + O.triangle_multiplication(ref, mask, w_in, "incoming")
        z_loc, m_loc = grid.shard_pair(z)[0], grid.shard_pair(mask)[0]
        be = CpuTriMulBackend()
        cp_triangle_multiplication_(z_loc, m_loc, OracleWeights(w_out, "outgoing"), grid, False, n_tokens, backend=be)
        cp_triangle_multiplication_(z_loc, m_loc, OracleWeights(w_in, "incoming"), grid, True, n_tokens, backend=be)
        err = float((z_loc - grid.shard_pair(ref)[0]).abs().max())
        q.put((rank, err))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows,cols,n_tokens", [(1, 2, 12), (2, 1, 12), (2, 2, 12), (1, 4, 8), (4, 1, 8), (2, 4, 16)])
def test_cp_trimul_matches_serial_on_gloo(rows, cols, n_tokens):
    """Outgoing then incoming triangle multiplication, sharded, against the serial oracle (reference's analogous
    test: tests/context_parallel/ops/test_trimul_serial_vs_cp.py, fp32 atol 2e-6; fp64 here)."""
    world = rows * cols
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + rows * 7 + cols * 13 + n_tokens) % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, rows, cols, port, n_tokens, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    errs = dict(q.get(timeout=5) for _ in range(world))
    assert len(errs) == world
    assert max(errs.values()) < 1e-10, errs


def _attn_worker(rank, world, rows, cols, port, n, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from bioemu2_b200.context_parallel import (CPGrid, cp_attention_pair_bias, cp_outer_product_mean,
                                                   cp_pair_weighted_averaging, cp_triangle_attention_, shard_range)
        from cp_cpu_backend import CpuAttentionLocal, Packed

        grid = CPGrid(rows, cols)
        loc = CpuAttentionLocal()
        dbl = lambda w: {k: v.double() for k, v in w.items()}  # noqa: E731
        g = torch.Generator().manual_seed(5)
        errs = {}
        # ---- single-track pair-bias attention (B=1, multiplicity 2)
        w = dbl(H.apb_weights(g, 32, 128, 4))
        s = torch.randn(2, n, 32, generator=g).double()
        z = torch.randn(1, n, n, 128, generator=g).double()
        mask = torch.ones(1, n, dtype=torch.bool)
        mask[0, n - 3:] = False
        ref = O.attention_pair_bias(s, z, mask, w, 4, 2)
        out = cp_attention_pair_bias(grid.shard_single(s), grid.shard_pair(z), grid.shard_single(mask), Packed(w, 4), grid,
                                     2, local=loc)
        errs["apb"] = float((out - grid.shard_single(ref)).abs().max())
        # ---- triangle attention, both nodes
        wt = dbl(H.triatt_weights(g))
        pm = torch.rand(1, n, n, generator=g) > 0.2
        for ending in (False, True):
            ref = z + O.triangle_attention(z, pm, wt, 4, ending)
            z_loc = grid.shard_pair(z)[0].clone()
            cp_triangle_attention_(z_loc, grid.shard_pair(pm)[0], Packed(wt), grid, ending, local=loc)
            errs[f"triatt_end{int(ending)}"] = float((z_loc - grid.shard_pair(ref)[0]).abs().max())
        # ---- outer product mean: MSA depth over grid rows, tokens over grid columns
        wo = dbl(H.opm_weights(g))
        S = 6 * rows
        m = torch.randn(1, S, n, 64, generator=g).double()
        mm = torch.ones(1, S, n, dtype=torch.bool)
        mm[0, 1] = False
        mm[0, :, n - 2:] = False
        ref = O.outer_product_mean(m, mm, wo)
        s0, s1 = shard_range(S, rows, grid.coords.r)
        c0, c1 = grid.coords.my_cols(n)
        row_count = mm.any(-1).sum(1)
        out = cp_outer_product_mean(m[0, s0:s1, c0:c1].contiguous(), mm[0, s0:s1, c0:c1].contiguous(), row_count,
                                    Packed(wo), grid, local=loc)
        errs["opm"] = float((out - grid.shard_pair(ref)[0]).abs().max())
        # ---- pair-weighted averaging: same MSA sharding, weights from the pair block, a random pair mask
        wp = dbl(H.pwa_weights(g))
        ref = m + O.pair_weighted_averaging(m, z, pm, wp)
        out = cp_pair_weighted_averaging(m[0, s0:s1, c0:c1].contiguous(), grid.shard_pair(z)[0], grid.shard_pair(pm)[0],
                                         Packed(wp, 8), grid, add_residual=True, local=loc)
        errs["pwa"] = float((out - ref[0, s0:s1, c0:c1]).abs().max())
        q.put((rank, errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows,cols,n", [(1, 2, 12), (2, 2, 12), (2, 1, 12), (2, 4, 16)])
def test_cp_attention_ops_match_serial_on_gloo(rows, cols, n):
    """Sharded pair-bias attention, triangle attention (both nodes), outer product mean and pair-weighted averaging
    against the serial oracle
    (reference's analogous tests: tests/context_parallel/ops/test_attention.py atol 5e-7, test_outer_product_mean.py)."""
    world = rows * cols
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31000 + (os.getpid() + rows * 7 + cols * 13 + n) % 2000
    procs = [ctx.Process(target=_attn_worker, args=(r, world, rows, cols, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    for _ in range(world):
        rank, errs = q.get(timeout=5)
        assert max(errs.values()) < 1e-7, (rank, errs)  # the 1/row_count scale is an fp32 scalar


# --------------------------------------------------------------------------------------------------------------
# The reference's calling convention: DTensors on a (dp, cp_axis_0, cp_axis_1) DeviceMesh, wrapper constructors
# (direction, layer, device_mesh, comm), in-place update returning the very object that was passed in.
class _OracleLayer:
    """Stands in for a loaded serial triangle multiplication on CPU: ``packed()`` hands the CPU backend its weights."""

    def __init__(self, w, mode):
        from cp_cpu_backend import OracleWeights

        self.mode = mode
        self._packed = OracleWeights(w, mode)

    def packed(self):
        return self._packed


def _dtensor_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torch.distributed.device_mesh import init_device_mesh
        from torch.distributed.tensor import DTensor, Shard, distribute_tensor

        from bioemu2_b200.context_parallel import CPGrid
        from bioemu2_b200.context_parallel.ops import TriangleMultiplicationAddRes
        from cp_cpu_backend import CpuTriMulBackend

        mesh = init_device_mesh("cpu", (1, 2, 2), mesh_dim_names=("dp", "cp_axis_0", "cp_axis_1"))
        grid = CPGrid.from_device_mesh(mesh)
        assert (grid.rows, grid.cols, grid.coords.r, grid.coords.c) == (2, 2, rank // 2, rank % 2)
        assert CPGrid.from_device_mesh(mesh) is grid  # cached: no second round of group creation
        n = 12
        g = torch.Generator().manual_seed(9)
        w = {k: v.double() for k, v in H.trimul_weights(g, 16).items()}
        z = torch.randn(1, n, n, 16, generator=g).double()
        mask = torch.rand(1, n, n, generator=g) > 0.25
        placements = (Shard(0), Shard(1), Shard(2))
        errs = {}
        for direction in ("Outgoing", "Incoming"):
            ref = z + O.triangle_multiplication(z, mask, w, direction.lower())
            zd = distribute_tensor(z.clone(), mesh, placements)
            md = distribute_tensor(mask.clone(), mesh, placements)
            op = TriangleMultiplicationAddRes(direction, _OracleLayer(w, direction.lower()), mesh, comm=None,
                                              backend=CpuTriMulBackend())
            ret = op(zd, md)
            assert ret is zd and isinstance(ret, DTensor), "the update is in place and returns the object it was given"
            errs[direction] = float((zd.full_tensor() - ref).abs().max())
        q.put((rank, errs))
    finally:
        dist.destroy_process_group()


def test_reference_style_wrapper_on_dtensors_2x2():
    """src/bioemu2/context_parallel/ops/triangle_multiplication.py:45-67 (constructor) and
    tests/context_parallel/ops/test_trimul_serial_vs_cp.py:89 (same object returned) in the reference."""
    world = 4
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 33000 + os.getpid() % 2000
    procs = [ctx.Process(target=_dtensor_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    for _ in range(world):
        rank, errs = q.get(timeout=5)
        assert max(errs.values()) < 1e-10, (rank, errs)


def _bad_shape_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from bioemu2_b200.context_parallel import CPGrid
        from bioemu2_b200.context_parallel.trimul import cp_triangle_multiplication_
        from cp_cpu_backend import CpuTriMulBackend, OracleWeights

        grid = CPGrid(1, 2)

        def no_collective(*a, **k):
            raise AssertionError("a collective was reached with inconsistent shapes")

        grid.all_gather = grid.reduce_scatter = grid.all_to_all = no_collective
        g = torch.Generator().manual_seed(3)
        w = {k: v.double() for k, v in H.trimul_weights(g, 16).items()}
        outcome = []
        for z_shape, m_shape, n_tokens in (((12, 6, 16), (12, 5), 12),     # mask does not match the block
                                           ((12, 7, 16), (12, 7), 12)):    # block is not a cell of the 1x2 grid
            try:
                cp_triangle_multiplication_(torch.zeros(z_shape, dtype=torch.float64), torch.ones(m_shape, dtype=torch.bool),
                                            OracleWeights(w, "outgoing"), grid, False, n_tokens, backend=CpuTriMulBackend())
                outcome.append("no error")
            except ValueError as exc:
                outcome.append(f"ValueError: {exc}")
        q.put((rank, outcome))
    finally:
        dist.destroy_process_group()


def test_shape_errors_are_raised_on_every_rank_before_any_collective():
    """The reference raises shape and placement violations on every rank before communicating
    (src/bioemu2/context_parallel/ops/triangular_mult_impl.py:431-522; tests/context_parallel/helpers.py:64-67)."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 35000 + os.getpid() % 2000
    procs = [ctx.Process(target=_bad_shape_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for _ in range(world):
        rank, outcome = q.get(timeout=5)
        assert len(outcome) == 2 and all(o.startswith("ValueError") for o in outcome), (rank, outcome)


def _absent_rank_worker(rank, world, port, q):
    import datetime
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    from bioemu2_b200.context_parallel import CPGrid

    grid = CPGrid(1, 2)
    t0 = time.time()
    if rank == 1:
        # this rank fails on the host before the exchange and never joins it
        q.put((rank, "raised before the collective", 0.0))
        time.sleep(8)  # stay alive past the peer's timeout, so the peer sees a missing partner, not a closed socket
        return
    try:
        grid.all_gather(torch.zeros(4), grid.row_group)
        q.put((rank, "collective returned", time.time() - t0))
    except Exception as exc:  # gloo reports the timeout as a RuntimeError / DistBackendError
        q.put((rank, f"{type(exc).__name__}", time.time() - t0))


def test_a_rank_that_never_joins_ends_the_peers_collective_with_an_error():
    """Failure made on the host: one rank raises before the exchange; the other's collective is bounded by the process
    group's timeout and surfaces as an exception instead of a hang (no GPU involved)."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 37000 + os.getpid() % 2000
    procs = [ctx.Process(target=_absent_rank_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict((r, (what, dt)) for r, what, dt in (q.get(timeout=60) for _ in range(world)))
    for p in procs:
        p.join(30)
        if p.is_alive():
            p.kill()
    assert got[1][0] == "raised before the collective"
    what, dt = got[0]
    assert what != "collective returned" and dt < 30, got
