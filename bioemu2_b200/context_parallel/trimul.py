"""Context-parallel triangle multiplication on an ``R x C`` grid (any R, C).

Reference: ``TriangleMultiplicationAddRes`` (src/bioemu2/context_parallel/ops/triangle_multiplication.py:45-182) and
its Cannon-ring contraction ``_distributed_bmm`` (ops/triangular_mult_impl.py:113-385), which needs a square grid
of at least four ranks.  On NVSwitch every peer is one hop away, so the ring buys nothing; the exchange here is

    outgoing  out[i,j] = sum_k a[i,k] b[j,k]     rank (r,c) holds a, b on (rows I_r, cols K_c)
        1. all-gather b over the column group          -> b[all j, K_c]
        2. partial[i in I_r, all j] = a_loc . b^T      (tcgen05 GEMM per destination block, fp32)
        3. reduce-scatter over the row group           -> out[I_r, J_c], summed over every K block
    incoming  out[i,j] = sum_k a[k,i] b[k,j]     rank (r,c) holds a^T, b^T on (cols, rows I_r = k)
        the same with rows and columns exchanged; the result arrives transposed and the output kernel
        walks it that way.

Everything else (LayerNorm, projections, gates, residual) runs on the local slab with the single-GPU kernels.
The result is written into the local slab in place, as the reference op does.
"""
from __future__ import annotations

import torch
from torch import Tensor

from .mesh import CPGrid


class CudaTriMulBackend:
    """The four local steps on the GPU (C ABI: b200_trimul_project / b200_bmm_nt / b200_rows_to_bf16 / b200_trimul_output)."""

    def project(self, z_slab: Tensor, mask_slab: Tensor, packed, incoming: bool):
        from .. import functional as F

        return F.trimul_project(z_slab, mask_slab, packed, incoming)

    def contract_into(self, lhs: Tensor, rhs_rows: Tensor, out: Tensor) -> None:
        from .. import functional as F

        F.bmm_nt_into(lhs, rhs_rows, out)

    def empty_partial(self, shape, device) -> Tensor:
        return torch.empty(shape, dtype=torch.float32, device=device)

    def to_operand(self, t: Tensor) -> Tensor:
        from .. import functional as F

        return F.rows_to_bf16(t.view(-1, 128), normalize=False).view(t.shape)

    def output_(self, z_slab: Tensor, t: Tensor, packed, transposed: bool) -> None:
        from .. import functional as F

        F.trimul_output_(z_slab, t, packed, transposed, add_residual=True)

    def check_block(self, n_rows: int, n_cols: int) -> None:
        if n_rows % 8 or n_cols % 8:
            raise ValueError(
                f"the CUDA context-parallel path needs block sizes that are multiples of 8 (got {n_rows} x {n_cols}); "
                "pad the token axis to kernel_shard_multiple(R, C)")


def cp_triangle_multiplication_(z_loc: Tensor, mask_loc: Tensor, packed, grid: CPGrid, incoming: bool, n_tokens: int,
                                backend=None) -> Tensor:
    """``z_loc += TriMul(z)`` restricted to this rank's block; ``z_loc[n_r, n_c, 128]``, ``mask_loc[n_r, n_c]``.

    ``n_tokens`` is the (padded) global token count.  Collective: every rank of the grid must call it.
    """
    backend = backend or CudaTriMulBackend()
    co = grid.coords
    n_r, n_c = z_loc.shape[0], z_loc.shape[1]
    (r0, r1), (c0, c1) = co.my_rows(n_tokens), co.my_cols(n_tokens)
    if (n_r, n_c) != (r1 - r0, c1 - c0):
        raise ValueError(f"local block {n_r}x{n_c} does not match grid block {r1 - r0}x{c1 - c0} of N={n_tokens}")
    if tuple(mask_loc.shape) != (n_r, n_c):
        raise ValueError(f"mask block {tuple(mask_loc.shape)} does not match {n_r}x{n_c}")
    backend.check_block(n_r, n_c)

    a_loc, b_loc = backend.project(z_loc, mask_loc, packed, incoming)  # [128][lines][pitch], zero-padded in pos
    if not incoming:
        lhs = a_loc
        gathered = grid.all_gather(b_loc, grid.col_group)  # segment r': rows I_r' of b
        seg_parts, dest_parts = co.row_ranges(n_tokens), co.col_ranges(n_tokens)
        scatter_group = grid.row_group
    else:
        lhs = b_loc
        gathered = grid.all_gather(a_loc, grid.row_group)  # segment c': columns J_c' of a (lines of a^T)
        seg_parts, dest_parts = co.col_ranges(n_tokens), co.row_ranges(n_tokens)
        scatter_group = grid.col_group
    dest_len = {d1 - d0 for d0, d1 in dest_parts}
    if len(dest_len) != 1:
        raise ValueError("blocks must have equal sizes: pad the token axis to shard_multiple(R, C)")
    dest_pitch = (dest_len.pop() + 127) // 128 * 128
    lines = lhs.shape[1]
    partial = backend.empty_partial((len(dest_parts), lhs.shape[0], lines, dest_pitch), z_loc.device)
    for di, (d0, d1) in enumerate(dest_parts):
        for si, (s0, s1) in enumerate(seg_parts):
            lo, hi = max(d0, s0), min(d1, s1)
            if lo < hi:
                backend.contract_into(lhs, gathered[si][:, lo - s0:hi - s0, :], partial[di][:, :, lo - d0:hi - d0])
    t_loc = grid.reduce_scatter(partial, scatter_group)
    backend.output_(z_loc, backend.to_operand(t_loc), packed, incoming)
    return z_loc
