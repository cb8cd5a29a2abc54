"""Context-parallel pair-bias attention, triangle attention and outer product mean on an R x C grid.

Reference (square grids, P2P rings): ``AttentionPairBias`` wrapper src/bioemu2/context_parallel/ops/attention.py:45-105
with ``ring_attention_simple_forward`` ops/attention_impl.py:984-1183 (the projected bias travels round the ring every
step); ``DistributedOuterProductMean`` ops/outer_product_mean.py:116-262 (ring over MSA-depth shards).  The reference
has no triangle attention.

Exchange used here (all NCCL collectives over the whole grid or its row / column groups):

* pair-bias attention   every rank projects the bias of its own block of z (one pass over local z), the blocks are
                        all-gathered into the full ``[H, N, N]`` bias (bf16, small next to z), the single track is
                        all-gathered over the column group, and every rank runs the attention kernel on the full
                        (tiny) single track, keeping its own rows.  No pair-sized tensor moves.
* triangle attention    the 4-head triangle bias is assembled the same way; the pair blocks are all-gathered over the
                        row group (starting node: complete rows) or the column group (ending node: complete columns),
                        the slab kernel runs on complete attention rows and each rank keeps its own block of the
                        update.  The ranks of a group compute the same slab: this first form scales with one grid
                        axis per direction (rows for the starting node, columns for the ending node).
* pair-weighted averaging  the MSA's token axis lies along the grid's COLUMNS while the weights' row axis lies along
                        its rows, so a rank needs weight rows it does not hold.  The 8-head logits of every block (and
                        the pair mask, one byte per pair) are all-gathered over the grid - they are 1/16 of z -, each
                        rank soft-maxes the rows of ITS tokens, all-gathers the normalised MSA (bf16) over the row
                        group for the values, and averages its own (depth slice, token block) with the single-GPU
                        kernels.  Reference: a 2D ring, src/bioemu2/context_parallel/ops/pair_averaging.py:44-290.
* outer product mean    the MSA is sharded (depth over grid rows, tokens over grid columns); tokens are all-gathered
                        over the row group, every rank forms the partial result of ITS depth slice for its column
                        block with proj_o already applied (proj_o is linear, so partial sums commute with it), and a
                        reduce-scatter over the column group sums the depth slices and hands out row blocks.
"""
from __future__ import annotations

import torch
from torch import Tensor

from .mesh import CPGrid


class CudaAttentionLocal:
    """Local steps on the GPU through the C ABI."""

    def pair_bias(self, z_slab: Tensor, apb_packed) -> Tensor:
        from .. import functional as F

        return F.pair_bias_slab(z_slab, apb_packed.ln_z_w, apb_packed.ln_z_b, apb_packed.w_z, apb_packed.H)

    def attention(self, s_full, bias_full, mask_full, apb_packed, multiplicity):
        from .. import functional as F

        return F.attention_pair_bias_with_bias(s_full, bias_full, mask_full, apb_packed, multiplicity)

    def tri_bias(self, z_slab: Tensor, tri_packed, ending: bool) -> Tensor:
        from .. import functional as F

        return F.pair_bias_slab(z_slab, tri_packed.f32[1], tri_packed.f32[2], tri_packed.w_b, 4, transposed=ending)

    def tri_slab(self, slab, mask_slab, bias_full, tri_packed, ending):
        from .. import functional as F

        return F.triangle_attention_slab(slab, mask_slab, bias_full, tri_packed, ending)

    def opm_partial(self, m_rows, mask_rows, opm_packed, j0, nj, inv_count, add_bias):
        from .. import functional as F

        return F.outer_product_mean_cols(m_rows, mask_rows, opm_packed, j0, nj, inv_count, add_bias)

    def pwa_logits(self, z_slab: Tensor, pwa_packed) -> Tensor:
        from .. import functional as F

        return F.pair_bias_slab(z_slab, pwa_packed.ln_z_w, pwa_packed.ln_z_b, pwa_packed.w_z, pwa_packed.H)

    def pwa_norm(self, m_loc: Tensor, pwa_packed) -> Tensor:
        from .. import functional as F

        return F.pwa_norm(m_loc, pwa_packed)

    def pwa_apply(self, mn_all, mn_own, logits, mask_rows, pwa_packed, residual):
        from .. import functional as F

        out = torch.empty(mn_own.shape, dtype=residual.dtype if residual is not None else torch.float32, device=mn_own.device)
        return F.pwa_apply(mn_all, mn_own, logits.contiguous(), F.mask_u8(mask_rows), pwa_packed, residual, out)

    def to_exchange(self, x: Tensor) -> Tensor:
        """The pair block as it travels to the ranks that attend over its lines: bf16, half the bytes on NVLink.  The
        slab kernel normalises what it receives (LayerNorm in fp32) and rounds to bf16 for the tensor cores anyway."""
        from .. import functional as F

        if x.dtype != torch.float32:
            return x
        return F.rows_to_bf16(x.reshape(-1, x.shape[-1]), normalize=False).view(x.shape)

    bias_dtype = torch.bfloat16


def _assemble_bias(blocks: list[Tensor], grid: CPGrid, n: int, transposed: bool) -> Tensor:
    """World all-gathered per-block biases ``[..., H, lines, pitch]`` -> ``[..., H, n, pad8(n)]``."""
    co = grid.coords
    lead = blocks[0].shape[:-2]
    full = blocks[0].new_zeros(lead + (n, (n + 7) // 8 * 8))
    for rank, blk in enumerate(blocks):
        (r0, r1), (c0, c1) = co.row_ranges(n)[rank // co.cols], co.col_ranges(n)[rank % co.cols]
        if transposed:
            full[..., c0:c1, r0:r1] = blk[..., :c1 - c0, :r1 - r0]
        else:
            full[..., r0:r1, c0:c1] = blk[..., :r1 - r0, :c1 - c0]
    return full


def cp_pair_bias_full(z_loc: Tensor, apb_packed, grid: CPGrid, local=None) -> Tensor:
    """The whole ``[B, H, N, pitch]`` pair bias of one attention module, assembled from every rank's projection of its
    own block of ``z_loc[B, n_r, n_c, 128]`` (one pass over local z, one all-gather over the grid)."""
    local = local or CudaAttentionLocal()
    B, n_r = z_loc.shape[0], z_loc.shape[1]
    n = n_r * grid.rows
    zb_loc = torch.stack([local.pair_bias(z_loc[b], apb_packed) for b in range(B)])  # [B, H, n_r, pitch]
    return _assemble_bias(grid.all_gather(zb_loc, grid.group), grid, n, False)


def cp_attention_pair_bias(s_loc: Tensor, z_loc: Tensor, mask_loc: Tensor, apb_packed, grid: CPGrid,
                           multiplicity: int = 1, local=None, bias_full: Tensor | None = None) -> Tensor:
    """``s_loc[B*M, n_r, c_s]`` (rows of this rank, replicated over grid columns), ``z_loc[B, n_r, n_c, 128]``,
    ``mask_loc[B, n_r]`` -> attention update for the same rows ``[B*M, n_r, c_s]``.  ``bias_full`` (from
    ``cp_pair_bias_full``) skips the projection and its all-gather: the pair tensor of the diffusion token blocks is
    static, so a caller computes it once per context instead of once per layer and step."""
    local = local or CudaAttentionLocal()
    n = z_loc.shape[1] * grid.rows
    if bias_full is None:
        bias_full = cp_pair_bias_full(z_loc, apb_packed, grid, local)
    s_full = torch.cat(grid.all_gather(s_loc, grid.col_group), dim=1)
    mask_full = torch.cat(grid.all_gather(mask_loc, grid.col_group), dim=1)
    out_full = local.attention(s_full, bias_full, mask_full, apb_packed, multiplicity)
    r0, r1 = grid.coords.my_rows(n)
    return out_full[:, r0:r1].contiguous()


def _to_exchange(local, x: Tensor) -> Tensor:
    fn = getattr(local, "to_exchange", None)
    return fn(x) if fn is not None else x


def cp_triangle_attention_(z_loc: Tensor, mask_loc: Tensor, tri_packed, grid: CPGrid, ending: bool, local=None) -> Tensor:
    """``z_loc += TriangleAttention(z)`` restricted to this rank's block ``z_loc[n_r, n_c, 128]``; in place."""
    local = local or CudaAttentionLocal()
    n_r, n_c = z_loc.shape[0], z_loc.shape[1]
    n = n_r * grid.rows
    if n_c * grid.cols != n:
        raise ValueError("blocks must tile a square pair tensor: pad the token axis to shard_multiple(R, C)")
    tb_loc = local.tri_bias(z_loc, tri_packed, ending)
    bias_full = _assemble_bias(grid.all_gather(tb_loc, grid.group), grid, n, ending)
    # A line (a row for the starting node, a column for the ending node) needs its whole length, which is spread
    # over the row (column) group.  The group splits its lines evenly: two all-to-alls move each rank's share of
    # whole lines in and the updates back out, so the attention work per rank is 1 / (R * C) of the total.  When
    # the lines do not divide by the group size every rank of the group computes all of them (all-gather form).
    if not ending:
        g, gs = grid.row_group, grid.cols
        if gs > 1 and n_r % gs == 0:
            share = n_r // gs

            def lines_in(x):  # [n_r, n_c, ...] -> this rank's lines at full length [share, N, ...]
                got = grid.all_to_all(x.reshape(gs, share, *x.shape[1:]).contiguous(), g)   # [src c, share, n_c, ...]
                return got.transpose(0, 1).reshape(share, gs * n_c, *x.shape[2:]).contiguous()

            upd = local.tri_slab(lines_in(_to_exchange(local, z_loc)), lines_in(mask_loc), bias_full, tri_packed, False)  # [share, N, 128]
            back = grid.all_to_all(upd.reshape(share, gs, n_c, upd.shape[-1]).transpose(0, 1).contiguous(), g)
            z_loc += back.reshape(n_r, n_c, upd.shape[-1])
            return z_loc
        slab = torch.cat(grid.all_gather(_to_exchange(local, z_loc), g), dim=1)          # [n_r, N, 128]
        mslab = torch.cat(grid.all_gather(mask_loc, g), dim=1)
        upd = local.tri_slab(slab, mslab, bias_full, tri_packed, False)
        c0, c1 = grid.coords.my_cols(n)
        z_loc += upd[:, c0:c1]
    else:
        g, gs = grid.col_group, grid.rows
        if gs > 1 and n_c % gs == 0:
            share = n_c // gs

            def lines_in(x):  # [n_r, n_c, ...] -> this rank's columns at full height [N, share, ...]
                send = x.reshape(n_r, gs, share, *x.shape[2:]).transpose(0, 1).contiguous()   # [dst r, n_r, share, ...]
                return grid.all_to_all(send, g).reshape(gs * n_r, share, *x.shape[2:])

            upd = local.tri_slab(lines_in(_to_exchange(local, z_loc)), lines_in(mask_loc), bias_full, tri_packed, True)   # [N, share, 128]
            back = grid.all_to_all(upd.reshape(gs, n_r, share, upd.shape[-1]).contiguous(), g)      # [src r, n_r, share, 128]
            z_loc += back.transpose(0, 1).reshape(n_r, n_c, upd.shape[-1])
            return z_loc
        slab = torch.cat(grid.all_gather(_to_exchange(local, z_loc), g), dim=0)          # [N, n_c, 128]
        mslab = torch.cat(grid.all_gather(mask_loc, g), dim=0)
        upd = local.tri_slab(slab, mslab, bias_full, tri_packed, True)
        r0, r1 = grid.coords.my_rows(n)
        z_loc += upd[r0:r1]
    return z_loc


def _assemble_blocks(blocks: list[Tensor], grid: CPGrid, n: int) -> Tensor:
    """World all-gathered pair blocks ``[n_r, n_c]`` -> the full ``[n, n]`` tensor."""
    co = grid.coords
    full = blocks[0].new_zeros((n, n))
    for rank, blk in enumerate(blocks):
        (r0, r1), (c0, c1) = co.row_ranges(n)[rank // co.cols], co.col_ranges(n)[rank % co.cols]
        full[r0:r1, c0:c1] = blk
    return full


def cp_pair_weighted_averaging(m_loc: Tensor, z_loc: Tensor, mask_loc: Tensor, pwa_packed, grid: CPGrid,
                               add_residual: bool = False, local=None) -> Tensor:
    """``m_loc[S_r, n_c, c_m]`` (MSA depth over grid rows, tokens over grid columns), ``z_loc[n_r, n_c, 128]``,
    ``mask_loc[n_r, n_c]`` (pair mask block) -> the update of this rank's MSA block ``[S_r, n_c, c_m]`` (plus ``m_loc``
    when ``add_residual``)."""
    local = local or CudaAttentionLocal()
    n_r, n_c = z_loc.shape[0], z_loc.shape[1]
    n = n_r * grid.rows
    if n_c * grid.cols != n or m_loc.shape[1] != n_c:
        raise ValueError("blocks must tile a square pair tensor and the MSA's token block must match its columns")
    logits_full = _assemble_bias(grid.all_gather(local.pwa_logits(z_loc, pwa_packed), grid.group), grid, n, False)
    mask_full = _assemble_blocks(grid.all_gather(mask_loc.to(torch.uint8), grid.group), grid, n)
    c0, c1 = grid.coords.my_cols(n)
    mn_own = local.pwa_norm(m_loc, pwa_packed)
    mn_all = torch.cat(grid.all_gather(mn_own, grid.row_group), dim=1)           # [S_r, N, c_m]: values of every token
    return local.pwa_apply(mn_all, mn_own, logits_full[:, c0:c1], mask_full[c0:c1], pwa_packed,
                           m_loc if add_residual else None)


def cp_outer_product_mean(m_loc: Tensor, mask_loc: Tensor, row_count: Tensor, opm_packed, grid: CPGrid, local=None) -> Tensor:
    """``m_loc[S_r, n_c, 64]`` (MSA depth sharded over grid rows, tokens over grid columns), ``mask_loc[S_r, n_c]``,
    ``row_count``: global number of valid MSA rows (1-element tensor) -> pair block ``[n_r, n_c, 128]`` in fp32."""
    local = local or CudaAttentionLocal()
    n_c = m_loc.shape[1]
    n = n_c * grid.cols
    m_rows = torch.cat(grid.all_gather(m_loc, grid.row_group), dim=1)            # [S_r, N, 64]
    mask_rows = torch.cat(grid.all_gather(mask_loc, grid.row_group), dim=1)
    inv = (1.0 / row_count.to(torch.float32).clamp(min=1)).reshape(1).to(m_loc.device)
    c0, c1 = grid.coords.my_cols(n)
    partial = local.opm_partial(m_rows, mask_rows, opm_packed, c0, c1 - c0, inv, grid.coords.r == 0)  # [N, n_c, 128]
    n_r = n // grid.rows
    if n_r * grid.rows != n:
        raise ValueError("token count must be a multiple of the grid's row count")
    return grid.reduce_scatter(partial.view(grid.rows, n_r, c1 - c0, partial.shape[-1]).contiguous(), grid.col_group)
