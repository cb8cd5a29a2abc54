"""Grid geometry of the 2D context-parallel layout: which rank owns which block of the pair tensor.

Mirrors the reference's contract (src/bioemu2/context_parallel/utils/mesh.py:17-55 ``shard_multiple`` /
``_shard_range``; utils/padding.py:106-130): the pair tensor ``z[B, N, N, c]`` is split into an ``R x C`` grid,
rows over mesh axis ``cp_axis_0`` and columns over ``cp_axis_1`` with ``torch.chunk``-style ceil splits, after
the token axis has been padded to a multiple of ``lcm(R, C)``; the single representation is row-sharded and
column-replicated; parameters are replicated.  Ranks are laid out row-major: ``rank = r * C + c``.

Unlike the reference, the grid need not be square (1x2 and 2x4 are first-class here), because the exchange
pattern below is all-gather / reduce-scatter over row and column groups, not a Cannon ring.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import Tensor


def shard_multiple(rows: int, cols: int) -> int:
    """Token counts must be padded to a multiple of this (reference: lcm of the two cp axes)."""
    return math.lcm(rows, cols)


def kernel_shard_multiple(rows: int, cols: int) -> int:
    """Padding the CUDA path asks for: blocks whose sizes are multiples of 8 (128-bit stores at block offsets)."""
    return 8 * math.lcm(rows, cols)


def shard_range(n: int, parts: int, index: int) -> tuple[int, int]:
    """``torch.chunk``-style ceil split of ``range(n)`` into ``parts`` pieces: the half-open range of piece ``index``."""
    size = -(-n // parts)
    lo = min(index * size, n)
    return lo, min(lo + size, n)


def pad_amount(n: int, multiple: int) -> int:
    return (-n) % multiple


@dataclass
class GridCoords:
    rows: int
    cols: int
    r: int
    c: int

    @property
    def rank(self) -> int:
        return self.r * self.cols + self.c

    def row_ranges(self, n: int) -> list[tuple[int, int]]:
        return [shard_range(n, self.rows, i) for i in range(self.rows)]

    def col_ranges(self, n: int) -> list[tuple[int, int]]:
        return [shard_range(n, self.cols, i) for i in range(self.cols)]

    def my_rows(self, n: int) -> tuple[int, int]:
        return shard_range(n, self.rows, self.r)

    def my_cols(self, n: int) -> tuple[int, int]:
        return shard_range(n, self.cols, self.c)


class CPGrid:
    """An ``R x C`` grid over the ranks of a process group, with its row and column sub-groups.

    ``row_group``: the ranks ``(r, *)`` sharing this rank's row block; ``col_group``: the ranks ``(*, c)`` sharing its
    column block.  Every rank of ``group`` must construct the grid (sub-group creation is collective).
    """

    def __init__(self, rows: int, cols: int, group: dist.ProcessGroup | None = None) -> None:
        world = dist.get_world_size(group)
        if rows * cols != world:
            raise ValueError(f"grid {rows}x{cols} does not match world size {world}")
        self.group = group
        rank = dist.get_rank(group)
        self.coords = GridCoords(rows, cols, rank // cols, rank % cols)
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
        self.row_group = None
        self.col_group = None
        for r in range(rows):
            g = dist.new_group([ranks[r * cols + c] for c in range(cols)])
            if r == self.coords.r:
                self.row_group = g
        for c in range(cols):
            g = dist.new_group([ranks[r * cols + c] for r in range(rows)])
            if c == self.coords.c:
                self.col_group = g

    _FROM_MESH: dict = {}

    @classmethod
    def from_device_mesh(cls, device_mesh) -> "CPGrid":
        """The grid of a ``torch.distributed`` ``DeviceMesh`` laid out as the reference lays its own out:
        ``(dp, cp_axis_0, cp_axis_1)`` (src/bioemu2/context_parallel/utils/mesh.py:17-39 reads the two cp sizes from
        mesh dimensions 1 and 2).  Rows of the pair tensor go over dimension 1, columns over dimension 2; the mesh's
        own process groups along those dimensions become the column and row groups.  A 2-D mesh is taken as
        ``(cp_axis_0, cp_axis_1)``.  Collective on first use for a given mesh (the group spanning both cp axes is
        created here); the result is cached per mesh.
        """
        key = id(device_mesh)
        hit = cls._FROM_MESH.get(key)
        if hit is not None and hit[0] is device_mesh:
            return hit[1]
        if device_mesh.ndim == 3:
            d0, d1, n_dp = 1, 2, device_mesh.size(0)
        elif device_mesh.ndim == 2:
            d0, d1, n_dp = 0, 1, 1
        else:
            raise ValueError(f"expected a (dp, cp_axis_0, cp_axis_1) or (cp_axis_0, cp_axis_1) mesh, got {device_mesh.ndim} dims")
        rows, cols = device_mesh.size(d0), device_mesh.size(d1)
        layout = device_mesh.mesh.reshape(n_dp, rows, cols)
        me = dist.get_rank()
        where = (layout == me).nonzero()
        if where.shape[0] != 1:
            raise ValueError("this rank is not part of the device mesh")
        dp, r, c = (int(v) for v in where[0])
        grid = cls.__new__(cls)
        grid.coords = GridCoords(rows, cols, r, c)
        grid.row_group = device_mesh.get_group(d1)   # ranks (r, *): they differ along cp_axis_1
        grid.col_group = device_mesh.get_group(d0)   # ranks (*, c)
        grid.group = None
        for i in range(n_dp):                        # every rank creates every dp slice's group, in the same order
            members = [int(v) for v in layout[i].flatten()]
            if n_dp == 1 and members == list(range(dist.get_world_size())):
                break                                # the default group already is the cp group
            g = dist.new_group(members)
            if i == dp:
                grid.group = g
        # collectives return members in group-rank order, which torch keeps sorted by global rank: the gathers below
        # rely on that order being (r, c) row-major, c along the row group and r along the column group
        for grp, want in ((grid.group, [int(v) for v in layout[dp].flatten()]),
                          (grid.row_group, [int(v) for v in layout[dp, r]]),
                          (grid.col_group, [int(v) for v in layout[dp, :, c]])):
            have = dist.get_process_group_ranks(grp) if grp is not None else list(range(dist.get_world_size()))
            if list(have) != want:
                raise ValueError(f"device mesh layout {want} is not in increasing rank order along its cp axes ({have})")
        cls._FROM_MESH[key] = (device_mesh, grid)
        return grid

    @property
    def rows(self) -> int:
        return self.coords.rows

    @property
    def cols(self) -> int:
        return self.coords.cols

    # ------------------------------------------------------------------ collectives on whole local tensors
    @staticmethod
    def all_gather(t: Tensor, group) -> list[Tensor]:
        """Every member's tensor (all of the same shape), in group-rank order."""
        n = dist.get_world_size(group)
        if n == 1:
            return [t]
        out = torch.empty((n,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out.view(-1), t.contiguous().view(-1), group=group)
        return list(out.unbind(0))

    @staticmethod
    def reduce_scatter(chunks: Tensor, group) -> Tensor:
        """``chunks[n_members, ...]`` summed over the group; member ``i`` receives the sum of everyone's ``chunks[i]``."""
        n = dist.get_world_size(group)
        if n == 1:
            return chunks[0]
        assert chunks.shape[0] == n and chunks.is_contiguous()
        if dist.get_backend(group) == "gloo":  # gloo has no reduce-scatter: all-reduce and keep one chunk
            dist.all_reduce(chunks, group=group)
            return chunks[dist.get_rank(group)]
        out = torch.empty_like(chunks[0])
        dist.reduce_scatter_tensor(out.view(-1), chunks.view(-1), group=group)
        return out

    @staticmethod
    def all_to_all(x: Tensor, group) -> Tensor:
        """``x[g, ...]`` (contiguous, ``g`` = group size): chunk ``i`` goes to group rank ``i``; returns the chunks
        received, in group-rank order."""
        n = dist.get_world_size(group)
        if n == 1:
            return x
        assert x.shape[0] == n and x.is_contiguous()
        if dist.get_backend(group) == "gloo":  # gloo has no all-to-all: gather everything and keep what is addressed here
            me = dist.get_rank(group)
            return torch.stack([t[me] for t in CPGrid.all_gather(x, group)])
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x, group=group)
        return out

    # ------------------------------------------------------------------ host-side sharding helpers (tests, setup)
    def shard_pair(self, z: Tensor) -> Tensor:
        """This rank's block of a full pair tensor ``z[B, N, N, ...]`` (N already padded)."""
        n = z.shape[1]
        (r0, r1), (c0, c1) = self.coords.my_rows(n), self.coords.my_cols(n)
        return z[:, r0:r1, c0:c1].contiguous()

    def shard_single(self, s: Tensor) -> Tensor:
        """This rank's rows of a single representation ``s[B, N, ...]`` (replicated over the grid's columns)."""
        r0, r1 = self.coords.my_rows(s.shape[1])
        return s[:, r0:r1].contiguous()

