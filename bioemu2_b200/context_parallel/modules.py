"""Context-parallel wrappers with the call pattern of the reference's distributed modules.

Reference: ``TriangleMultiplicationAddRes`` (src/bioemu2/context_parallel/ops/triangle_multiplication.py:45-182,
``forward(x, mask) -> x``, in place, returns the same object), ``DTensorAwareTransition``
(ops/transition.py:16-64, communication-free, returns the update), ``DistributedPairMixerLayer/Module``
(modules/pairmixer.py:77-115).  Each wrapper adopts an already loaded serial module, as the reference's do.

Arguments may be plain local blocks ``[B, n_r, n_c, ...]`` or ``DTensor``s with the reference's pair placements
``(Shard(0), Shard(1), Shard(2))`` over ``(dp, cp_axis_0, cp_axis_1)``; a DTensor is updated through its local shard
and handed back as the same object.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from ..attention_pair_bias import AttentionPairBias
from ..outer_product_mean import OuterProductMean
from ..transition import Transition
from ..triangle_attention import TriangleAttention
from ..triangle_multiplication import TriangleMultiplication
from .attention import (cp_attention_pair_bias, cp_outer_product_mean, cp_pair_weighted_averaging,
                        cp_triangle_attention_)
from .mesh import CPGrid
from .trimul import cp_triangle_multiplication_


def _local(x):
    return x.to_local() if hasattr(x, "to_local") else x


class CPTriangleMultiplication(nn.Module):
    """``forward(x, mask)``: ``x += TriMul(x)`` on the sharded pair tensor, in place; returns ``x`` itself."""

    def __init__(self, layer: TriangleMultiplication, grid: CPGrid, backend=None) -> None:
        super().__init__()
        self.layer = layer
        self.grid = grid
        self.backend = backend

    def forward(self, x, mask):
        xl, ml = _local(x), _local(mask)
        if xl.ndim != 4 or ml.ndim != 3 or xl.shape[:3] != ml.shape:
            raise ValueError(f"expected x[B,n_r,n_c,D] and mask[B,n_r,n_c], got {tuple(xl.shape)}, {tuple(ml.shape)}")
        if not xl.is_contiguous():
            raise ValueError("the local block must be contiguous (it is updated in place)")
        n_tokens = xl.shape[1] * self.grid.rows
        if xl.shape[2] * self.grid.cols != n_tokens:
            raise ValueError(f"block {xl.shape[1]}x{xl.shape[2]} is not one cell of a {self.grid.rows}x{self.grid.cols} "
                             "grid over a square pair tensor: pad the token axis to shard_multiple(R, C) first")
        packed = self.layer.packed()
        for b in range(xl.shape[0]):
            cp_triangle_multiplication_(xl[b], ml[b], packed, self.grid, self.layer.mode == "incoming", n_tokens,
                                        backend=self.backend)
        return x


class CPTransition(nn.Module):
    """Per-position transition on the local block: no communication (reference ops/transition.py:28-64)."""

    def __init__(self, serial: Transition, grid: CPGrid | None = None) -> None:
        super().__init__()
        self.serial = serial

    def forward(self, x):
        out = self.serial(_local(x))
        if hasattr(x, "to_local"):
            from torch.distributed.tensor import DTensor

            return DTensor.from_local(out, x.device_mesh, x.placements, run_check=False)
        return out

    def forward_residual_(self, x):
        self.serial.forward_residual_(_local(x))
        return x


def _grid(grid_or_mesh) -> CPGrid:
    """A ``CPGrid`` as given, or the one of a ``DeviceMesh`` / of an object exposing ``device_mesh_subgroups``."""
    if isinstance(grid_or_mesh, CPGrid):
        return grid_or_mesh
    return CPGrid.from_device_mesh(getattr(grid_or_mesh, "device_mesh_subgroups", grid_or_mesh))


class CPPairMixerLayer(nn.Module):
    """``z -> z`` after triangle multiplication out / in and the pair transition, all in place on the local block.
    ``grid`` may be a ``CPGrid``, a ``DeviceMesh`` or the reference's distributed manager
    (``DistributedPairMixerLayer(serial, dist_manager)``, src/bioemu2/context_parallel/modules/pairmixer.py:77-99)."""

    def __init__(self, serial, grid, backend=None) -> None:
        super().__init__()
        grid = _grid(grid)
        self.tri_mul_out = CPTriangleMultiplication(serial.tri_mul_out, grid, backend)
        self.tri_mul_in = CPTriangleMultiplication(serial.tri_mul_in, grid, backend)
        self.transition_z = CPTransition(serial.transition_z, grid)

    def forward(self, z, pair_mask):
        self.tri_mul_out(z, pair_mask)
        self.tri_mul_in(z, pair_mask)
        return self.transition_z.forward_residual_(z)


class CPPairMixerModule(nn.Module):
    """``DistributedPairMixerModule(serial, dist_manager)`` of the reference
    (src/bioemu2/context_parallel/modules/pairmixer.py:102-115); ``grid`` as for ``CPPairMixerLayer``."""

    def __init__(self, serial, grid, backend=None) -> None:
        super().__init__()
        grid = _grid(grid)
        self.layers = nn.ModuleList(CPPairMixerLayer(layer, grid, backend) for layer in serial.layers)

    def forward(self, z, pair_mask):
        with torch.no_grad():
            for layer in self.layers:
                z = layer(z, pair_mask)
        return z


class CPAttentionPairBias(nn.Module):
    """``forward(s, z, mask, multiplicity)`` on sharded inputs: ``s`` rows of this rank (replicated over grid columns),
    ``z`` this rank's pair block, ``mask`` this rank's token rows; returns the update for the same rows
    (reference wrapper: src/bioemu2/context_parallel/ops/attention.py:74-105).

    ``prepare_static(z)`` computes and keeps the assembled pair bias for a pair block that will be passed again and
    again (the diffusion module's static context): later calls with the SAME tensor object (same storage and version
    counter) skip the projection of ``z`` and the all-gather of the bias; any other ``z`` takes the normal path."""

    def __init__(self, attention: AttentionPairBias, grid: CPGrid, local=None) -> None:
        super().__init__()
        self.attention = attention
        self.grid = grid
        self.local = local
        self._static_key = None
        self._static_bias = None

    @staticmethod
    def _key(z):
        return (z.data_ptr(), z._version, tuple(z.shape), z.dtype)

    def prepare_static(self, z) -> None:
        from .attention import cp_pair_bias_full

        zl = _local(z)
        with torch.no_grad():
            self._static_bias = cp_pair_bias_full(zl, self.attention.packed(), self.grid, self.local)
        self._static_key = self._key(zl)

    def release_static(self) -> None:
        self._static_key, self._static_bias = None, None

    def forward(self, s, z, mask, multiplicity: int = 1):
        zl = _local(z)
        bias = self._static_bias if (self._static_key is not None and self._static_key == self._key(zl)) else None
        out = cp_attention_pair_bias(_local(s), zl, _local(mask), self.attention.packed(), self.grid, multiplicity,
                                     local=self.local, bias_full=bias)
        if hasattr(s, "to_local"):
            from torch.distributed.tensor import DTensor

            return DTensor.from_local(out, s.device_mesh, s.placements, run_check=False)
        return out


class CPTriangleAttention(nn.Module):
    """``forward(x, mask)``: ``x += TriangleAttention(x)`` on the sharded pair tensor, in place; returns ``x``."""

    def __init__(self, layer: TriangleAttention, grid: CPGrid, local=None) -> None:
        super().__init__()
        self.layer = layer
        self.grid = grid
        self.local = local

    def forward(self, x, mask):
        xl, ml = _local(x), _local(mask)
        packed = self.layer.packed()
        for b in range(xl.shape[0]):
            cp_triangle_attention_(xl[b], ml[b], packed, self.grid, self.layer.ending, local=self.local)
        return x


class CPOuterProductMean(nn.Module):
    """``forward(m, mask, row_count)`` with ``m[B, S_r, n_c, 64]`` sharded over (depth -> grid rows, tokens -> grid
    columns); returns this rank's pair block ``[B, n_r, n_c, 128]``
    (reference: src/bioemu2/context_parallel/ops/outer_product_mean.py:199-262)."""

    def __init__(self, serial: OuterProductMean, grid: CPGrid, local=None) -> None:
        super().__init__()
        self.serial = serial
        self.grid = grid
        self.local = local

    def forward(self, m, mask, row_count):
        ml, kl = _local(m), _local(mask)
        packed = self.serial.packed()
        outs = [cp_outer_product_mean(ml[b], kl[b], row_count[b:b + 1], packed, self.grid, local=self.local)
                for b in range(ml.shape[0])]
        out = torch.stack(outs).to(ml.dtype)
        if hasattr(m, "to_local"):  # pair placements: batch, rows and columns sharded like the input's three axes
            from torch.distributed.tensor import DTensor

            return DTensor.from_local(out, m.device_mesh, m.placements, run_check=False)
        return out


class CPPairWeightedAveraging(nn.Module):
    """``forward(m, z, mask)`` with ``m[B, S_r, n_c, c_m]`` (depth over grid rows, tokens over grid columns), the pair
    block ``z[B, n_r, n_c, 128]`` and its pair mask; returns the update of this rank's MSA block
    (reference: ``DistributedPairWeightedAveraging``, src/bioemu2/context_parallel/ops/pair_weighted_averaging.py:16-84)."""

    def __init__(self, serial, grid, local=None) -> None:
        super().__init__()
        self.serial = serial
        self.grid = _grid(grid)
        self.local = local

    def forward(self, m, z, mask, chunk_heads: bool = False, add_residual: bool = False):
        ml, zl, kl = _local(m), _local(z), _local(mask)
        packed = self.serial.packed()
        out = torch.stack([cp_pair_weighted_averaging(ml[b], zl[b], kl[b], packed, self.grid, add_residual, self.local)
                           for b in range(ml.shape[0])])
        if hasattr(m, "to_local"):
            from torch.distributed.tensor import DTensor

            return DTensor.from_local(out, m.device_mesh, m.placements, run_check=False)
        return out


class CPPairMixerMSALayer(nn.Module):
    """The MSA block on sharded tensors (reference: ``DistributedPairMixerMSALayer``,
    src/bioemu2/context_parallel/modules/pairmixer.py:118-174): ``forward(z, m, token_mask, msa_mask, msa_row_count)
    -> (z, m)``.  ``z[B, n_r, n_c, 128]`` is updated in place; ``m[B, S_r, n_c, c_m]`` has its depth over the grid's
    rows and its tokens over the grid's columns; ``token_mask`` is the pair-mask block, ``msa_mask[B, S_r, n_c]``,
    ``msa_row_count[B]`` the global number of valid MSA rows."""

    def __init__(self, serial, grid, backend=None, local=None) -> None:
        super().__init__()
        grid = _grid(grid)
        self.grid = grid
        self.msa_transition = serial.msa_transition                      # per (row, token): no communication
        self.pair_weighted_averaging = CPPairWeightedAveraging(serial.pair_weighted_averaging, grid, local)
        self.outer_product_mean = CPOuterProductMean(serial.outer_product_mean, grid, local)
        self.tri_mul_out = CPTriangleMultiplication(serial.tri_mul_out, grid, backend)
        self.tri_mul_in = CPTriangleMultiplication(serial.tri_mul_in, grid, backend)
        self.z_transition = CPTransition(serial.z_transition, grid)

    def forward(self, z, m, token_mask, msa_mask, msa_row_count):
        ml = self.pair_weighted_averaging(_local(m), z, token_mask, add_residual=True)       # a new tensor
        ml = self._msa_transition_(ml)
        zl = _local(z)
        zl += self.outer_product_mean(ml, _local(msa_mask), msa_row_count).to(zl.dtype)
        self.tri_mul_out(z, token_mask)
        self.tri_mul_in(z, token_mask)
        self.z_transition.forward_residual_(z)
        if hasattr(m, "to_local"):
            from torch.distributed.tensor import DTensor

            ml = DTensor.from_local(ml, m.device_mesh, m.placements, run_check=False)
        return z, ml

    def _msa_transition_(self, ml):
        fn = getattr(self.msa_transition, "forward_residual_", None)
        return fn(ml) if fn is not None else ml + self.msa_transition(ml)


class CPPairMixerMSAModule(nn.Module):
    """The MSA module on sharded tensors (reference: ``DistributedPairMixerMSAModule``,
    src/bioemu2/context_parallel/modules/pairmixer.py:177-263).  ``forward(z, emb, msa, msa_mask, has_deletion,
    deletion_value, msa_paired, token_pad_mask) -> z``: ``z[B, n_r, n_c, 128]`` is this rank's pair block (updated in
    place), the MSA tensors are this rank's ``[B, S_r, n_c, ...]`` block (depth over grid rows, tokens over grid
    columns), ``emb[B, T, .]`` and ``token_pad_mask[B, T]`` are replicated."""

    def __init__(self, serial, grid, backend=None, local=None) -> None:
        super().__init__()
        self.grid = _grid(grid)
        self.serial = serial
        self.layers = nn.ModuleList(CPPairMixerMSALayer(layer, self.grid, backend, local) for layer in serial.layers)

    def forward(self, z, emb, msa, msa_mask, has_deletion, deletion_value, msa_paired, token_pad_mask):
        import torch.distributed as dist

        n = token_pad_mask.shape[1]
        (r0, r1), (c0, c1) = self.grid.coords.my_rows(n), self.grid.coords.my_cols(n)
        m = self.serial.embed_msa(emb, _local(msa), _local(has_deletion), _local(deletion_value),
                                  _local(msa_paired) if msa_paired is not None else None, tokens=slice(c0, c1))
        tok = token_pad_mask.bool()
        token_mask = (tok[:, r0:r1, None] & tok[:, None, c0:c1]).contiguous()
        mk = _local(msa_mask)
        # global number of MSA rows with at least one valid token: the per-row flags are combined over the row group
        # (token blocks), then counted over the column group (depth slices)
        has_any = mk.bool().any(dim=-1).to(torch.int32)                     # [B, S_r]
        if self.grid.cols > 1:
            dist.all_reduce(has_any, op=dist.ReduceOp.MAX, group=self.grid.row_group)
        count = has_any.sum(dim=1)
        if self.grid.rows > 1:
            dist.all_reduce(count, group=self.grid.col_group)
        for layer in self.layers:
            z, m = layer(z, m, token_mask, mk, count)
        return z


class CPPairMixerSequenceEmbedder(nn.Module):
    """The recycling trunk on an R x C grid (reference: ``PairMixerSequenceEmbedderDistributed``,
    src/bioemu2/context_parallel/modules/pairmixer.py:266-...).  ``forward(s_inputs, feats, num_steps_recycle)`` with
    ``s_inputs`` and ``feats["token_pad_mask"]`` replicated, the MSA features as this rank's ``[B, S_r, n_c, ...]`` block,
    and ``feats["pair_init_terms"]`` (the feature encoders' pair terms) as this rank's ``[B, n_r, n_c, 128]`` block.
    Returns the replicated single representation and this rank's block of the pair representation."""

    def __init__(self, serial, grid, backend=None, local=None) -> None:
        super().__init__()
        self.grid = _grid(grid)
        self.serial = serial
        self.msa_module = CPPairMixerMSAModule(serial.msa_module, self.grid, backend, local)
        self.pairmixer_module = CPPairMixerModule(serial.pairmixer_module, self.grid, backend)

    def forward(self, s_inputs, feats: dict, num_steps_recycle: int = 0):
        from .. import functional as F

        e = self.serial
        if num_steps_recycle < 0:
            raise ValueError("num_steps_recycle must be non-negative")
        n = s_inputs.shape[1]
        (r0, r1), (c0, c1) = self.grid.coords.my_rows(n), self.grid.coords.my_cols(n)
        xb = e._lin["s_init"].operand(s_inputs)
        s_init = e._lin["s_init"](xb)
        a, c = e._lin["z_init_1"](xb), e._lin["z_init_2"](xb)
        terms = feats.get("pair_init_terms")
        z_init = F.pair_outer_sum(a[:, r0:r1].contiguous(), c[:, c0:c1].contiguous(),
                                  _local(terms).float().contiguous() if terms is not None else None)
        tok = feats["token_pad_mask"].bool()
        pair_mask = (tok[:, r0:r1, None] & tok[:, None, c0:c1]).to(torch.uint8).contiguous()
        s, z = torch.zeros_like(s_init), torch.zeros_like(z_init)
        for _ in range(num_steps_recycle + 1):
            s = e._recycle(s, s_init, e.s_norm, "s_recycle")          # replicated: every rank computes the whole track
            z = e._recycle(z, z_init, e.z_norm, "z_recycle")          # per pair: the local block
            z = self.msa_module(z, s_inputs, feats["msa"], feats["msa_mask"], feats["has_deletion"],
                                feats["deletion_value"], feats.get("msa_paired"), feats["token_pad_mask"])
            z = self.pairmixer_module(z, pair_mask)
        return s, z


DistributedPairWeightedAveraging = CPPairWeightedAveraging
DistributedPairMixerMSALayer = CPPairMixerMSALayer
DistributedPairMixerMSAModule = CPPairMixerMSAModule
PairMixerSequenceEmbedderDistributed = CPPairMixerSequenceEmbedder


class CPPairformerBlock(nn.Module):
    """The composite block on sharded inputs: ``(s_rows, z_block, token_mask_rows, token_mask_cols) -> (s_rows, z_block)``."""

    def __init__(self, serial, grid: CPGrid) -> None:
        super().__init__()
        self.grid = grid
        self.tri_mul_out = CPTriangleMultiplication(serial.tri_mul_out, grid)
        self.tri_mul_in = CPTriangleMultiplication(serial.tri_mul_in, grid)
        self.tri_att_start = CPTriangleAttention(serial.tri_att_start, grid)
        self.tri_att_end = CPTriangleAttention(serial.tri_att_end, grid)
        self.transition_z = CPTransition(serial.transition_z, grid)
        self.attention = CPAttentionPairBias(serial.attention, grid)
        self.transition_s = CPTransition(serial.transition_s, grid)

    def forward_(self, s, z, mask_rows, pair_mask_u8):
        """In place on the local blocks, with the pair mask of the block already built (one byte per pair)."""
        self.tri_mul_out(z, pair_mask_u8)
        self.tri_mul_in(z, pair_mask_u8)
        self.tri_att_start(z, pair_mask_u8)
        self.tri_att_end(z, pair_mask_u8)
        self.transition_z.forward_residual_(z)
        s += self.attention(s, z, mask_rows)
        self.transition_s.forward_residual_(s)
        return s, z

    def forward(self, s, z, mask_rows, mask_cols):
        pm = (mask_rows[:, :, None] & mask_cols[:, None, :]).to(torch.uint8)
        return self.forward_(s, z, mask_rows, pm)


class CPPairformerModule(nn.Module):
    """A stack of composite blocks on sharded inputs; adopts a loaded serial ``PairformerModule``.

    ``forward(s_rows, z_block, token_mask_rows, token_mask_cols)`` returns updated copies; ``forward_`` updates the
    given blocks in place.  A kernel-side failure (a bounded wait that ran out) is raised at the end of the stack.
    """

    def __init__(self, serial, grid: CPGrid) -> None:
        super().__init__()
        self.grid = grid
        self.layers = nn.ModuleList(CPPairformerBlock(layer, grid) for layer in serial.layers)

    def forward_(self, s, z, mask_rows, mask_cols):
        from .. import _lib

        pm = (mask_rows[:, :, None] & mask_cols[:, None, :]).to(torch.uint8)
        with torch.no_grad():
            for layer in self.layers:
                layer.forward_(s, z, mask_rows, pm)
        _lib.raise_if_device_wait()
        return s, z

    def forward(self, s, z, mask_rows, mask_cols):
        return self.forward_(s.clone(), z.clone(), mask_rows, mask_cols)


class CPConditionedTransformerLayer(nn.Module):
    """The token block of the diffusion module on sharded inputs
    (``DistributedConditionedTransformerLayer(serial, dist_manager)``,
    src/bioemu2/context_parallel/layers/transformer_layers.py:29-67).

    The token stream ``x[B*M, n_r, dim]``, the conditioning ``c`` and the mask are row-sharded and replicated over the
    grid's columns, ``pairs`` is this rank's block of the pair tensor.  Conditioning, adaptive LayerNorm, gated
    residuals and the transition touch only local rows; the attention is the context-parallel one.
    """

    def __init__(self, serial, grid) -> None:
        super().__init__()
        self.serial = serial
        self.attention = CPAttentionPairBias(serial.attention.pair_bias_attn, _grid(grid))

    def forward(self, x, pairs, c, mask=None, multiplicity: int = 1):
        xl, pl, cl = _local(x), _local(pairs), _local(c)
        ml = _local(mask) if mask is not None else torch.ones(pl.shape[0], pl.shape[1], dtype=torch.bool, device=xl.device)
        out = self.serial._forward(xl, pl, cl, ml, multiplicity, lambda s, z, m, mult: self.attention(s, z, m, mult))
        if hasattr(x, "to_local"):
            from torch.distributed.tensor import DTensor

            return DTensor.from_local(out, x.device_mesh, x.placements, run_check=False)
        return out


DistributedPairMixerLayer = CPPairMixerLayer
DistributedPairMixerModule = CPPairMixerModule
DistributedConditionedTransformerLayer = CPConditionedTransformerLayer
