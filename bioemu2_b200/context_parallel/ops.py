"""The reference's context-parallel wrapper classes, under their own names and constructor signatures.

The reference wraps a loaded serial module for 2D context parallelism by passing it, together with the device mesh
(or the distributed manager that owns it) and a ring communicator, to one of these classes:

    TriangleMultiplicationAddRes(direction, layer, device_mesh, comm)     src/bioemu2/context_parallel/ops/triangle_multiplication.py:45-67
    AttentionPairBias(attention, dist_manager)                            src/bioemu2/context_parallel/ops/attention.py:45-72
    DistributedOuterProductMean(serial, device_mesh, comm)                src/bioemu2/context_parallel/ops/outer_product_mean.py:199-210
    DTensorAwareTransition(serial, device_mesh)                           src/bioemu2/context_parallel/ops/transition.py:19-27
    LayerNormLinearParamsReplicatedTiled(serial, device_mesh)             src/bioemu2/context_parallel/ops/tiled_params_replicated.py:36-81

The classes here take the same arguments, so the reference's wrapping code (``_distributed_trimul`` and the
``Distributed*`` module constructors) keeps working when it imports them from this package instead.  The serial
module may be one of this package's or one of the reference's (its parameters are then adopted through
``load_state_dict``).  The ``DeviceMesh`` supplies the grid and its row / column process groups
(``CPGrid.from_device_mesh``); the ring communicator is accepted and not used, because the exchange here is
all-gather / reduce-scatter / all-to-all over those groups rather than a Cannon ring.  ``forward`` takes ``DTensor``s
with the reference's placements, or plain local blocks, and in-place ops hand back the very object they were given.
"""
from __future__ import annotations

import torch.nn as nn

from ..attention_pair_bias import AttentionPairBias as SerialAttentionPairBias
from ..outer_product_mean import OuterProductMean as SerialOuterProductMean
from ..transition import Transition as SerialTransition
from ..triangle_multiplication import TriangleMultiplication as SerialTriangleMultiplication
from .mesh import CPGrid
from .modules import CPAttentionPairBias, CPOuterProductMean, CPTransition, CPTriangleMultiplication


def grid_of(mesh_or_manager) -> CPGrid:
    """``CPGrid`` from a ``CPGrid``, a ``DeviceMesh``, or an object exposing ``device_mesh_subgroups`` (the
    reference's ``DistributedManager``, src/bioemu2/context_parallel/distributed/manager.py:42)."""
    if isinstance(mesh_or_manager, CPGrid):
        return mesh_or_manager
    mesh = getattr(mesh_or_manager, "device_mesh_subgroups", mesh_or_manager)
    return CPGrid.from_device_mesh(mesh)


def _mode_of(direction) -> str:
    name = getattr(direction, "name", direction)
    mode = str(name).lower()
    if mode not in ("outgoing", "incoming"):
        raise ValueError(f"Invalid direction: {direction}")
    return mode


def adopt_trimul(layer, mode: str):
    if isinstance(layer, SerialTriangleMultiplication) or (hasattr(layer, "packed") and hasattr(layer, "mode")):
        if layer.mode != mode:
            raise ValueError(f"layer is a {layer.mode} triangle multiplication, direction says {mode}")
        return layer
    own = SerialTriangleMultiplication(layer.norm_in.normalized_shape[0], mode).eval()
    own.load_state_dict(layer.state_dict(), strict=True)
    return own.to(layer.p_in.weight.device)


def adopt_apb(attention: nn.Module) -> SerialAttentionPairBias:
    if isinstance(attention, SerialAttentionPairBias):
        return attention
    own = SerialAttentionPairBias(
        c_s=attention.proj_g.in_features, c_z=attention.proj_z.in_features, num_heads=attention.num_heads,
        inf=attention.inf, initial_norm=attention.initial_norm, use_bias_in_layer_norm=attention.norm_z.bias is not None).eval()
    own.load_state_dict(attention.state_dict(), strict=True)
    return own.to(attention.proj_g.weight.device)


def adopt_transition(serial: nn.Module) -> SerialTransition:
    if isinstance(serial, SerialTransition):
        return serial
    own = SerialTransition(serial.fc1.in_features, serial.fc1.out_features, serial.fc3.out_features,
                           use_norm=serial.use_norm).eval()
    own.load_state_dict(serial.state_dict(), strict=True)
    return own.to(serial.fc1.weight.device)


def adopt_opm(serial: nn.Module) -> SerialOuterProductMean:
    if isinstance(serial, SerialOuterProductMean):
        return serial
    own = SerialOuterProductMean(serial.norm.normalized_shape[0], serial.c_hidden, serial.proj_o.out_features).eval()
    own.load_state_dict(serial.state_dict(), strict=True)
    return own.to(serial.proj_o.weight.device)


class TriangleMultiplicationAddRes(CPTriangleMultiplication):
    """``forward(x, mask) -> x``: adds the triangle-multiplication update to the sharded pair tensor in place and
    returns the object it was given (asserted by the reference's
    tests/context_parallel/ops/test_trimul_serial_vs_cp.py:89)."""

    def __init__(self, direction, layer: nn.Module, device_mesh, comm=None, bmm_chunk: int | None = None,
                 tile_size: int | None = None, backend=None) -> None:
        super().__init__(adopt_trimul(layer, _mode_of(direction)), grid_of(device_mesh), backend)
        self.device_mesh = device_mesh
        self.ring_comm = comm


class AttentionPairBias(CPAttentionPairBias):
    """``forward(s, z, mask, multiplicity=1)`` on ``s`` ``(Shard(0), Shard(1), Replicate())``, ``z``
    ``(Shard(0), Shard(1), Shard(2))``, ``mask`` like ``s``; returns the update sharded like ``s``."""

    def __init__(self, attention: nn.Module, dist_manager, local=None) -> None:
        super().__init__(adopt_apb(attention), grid_of(dist_manager), local)


class DistributedOuterProductMean(CPOuterProductMean):
    """``forward(m, mask, row_count)`` with the MSA sharded (depth over cp_axis_0, tokens over cp_axis_1)."""

    def __init__(self, serial: nn.Module, device_mesh, comm=None, local=None) -> None:
        super().__init__(adopt_opm(serial), grid_of(device_mesh), local)
        self.ring_comm = comm


class DTensorAwareTransition(CPTransition):
    """``forward(x)``: the per-position transition on the local shard, placements preserved, no communication."""

    def __init__(self, serial: nn.Module, device_mesh=None) -> None:
        super().__init__(adopt_transition(serial))
        self.device_mesh = device_mesh


def _rewrap(out, like, width: int):
    """``out`` as a DTensor placed like ``like`` (global shape with ``width`` channels), or ``out`` itself."""
    if not hasattr(like, "to_local"):
        return out
    import torch
    from torch.distributed.tensor import DTensor

    shape = torch.Size((*like.shape[:-1], width))
    stride, acc = [], 1
    for n in reversed(shape):
        stride.append(acc)
        acc *= n
    return DTensor.from_local(out, like.device_mesh, like.placements, run_check=False, shape=shape,
                              stride=tuple(reversed(stride)))


class LayerNormLinearParamsReplicatedTiled(nn.Module):
    """``Linear(LayerNorm(cat(*pairs, -1)))`` on the local blocks of one or two pair tensors, no communication and no
    materialised concatenation (src/bioemu2/context_parallel/ops/tiled_params_replicated.py:36-81; the row tiling
    there bounds the intermediates, which do not exist here).  ``serial`` is the ``nn.Sequential(LayerNorm, Linear)``
    of the serial model; its parameters are shared, and sub-module keys ``0`` / ``1`` are kept."""

    def __init__(self, serial: nn.Sequential, device_mesh=None) -> None:
        super().__init__()
        norm, linear = serial
        if linear.bias is not None:
            raise ValueError("the projection is expected to be bias-free (LinearNoBias)")
        self.add_module("0", norm)
        self.add_module("1", linear)
        self.device_mesh = device_mesh
        self._w = None
        self._version = -1

    def forward(self, *pairs):
        import torch

        from .. import functional as F

        if torch.is_grad_enabled():
            raise RuntimeError(f"{type(self).__name__} is forward-only; use torch.no_grad().")
        if not 1 <= len(pairs) <= 2:
            raise ValueError("one or two pair tensors are supported")
        norm, linear = getattr(self, "0"), getattr(self, "1")
        p = linear.weight
        if self._w is None or self._version != p._version or self._w.device != p.device:
            self._w, self._version = p.detach().to(torch.bfloat16).contiguous(), p._version
        loc = [x.to_local() if hasattr(x, "to_local") else x for x in pairs]
        zn = (F.rows_to_bf16(loc[0], norm.weight, norm.bias) if len(loc) == 1
              else F.rows2_to_bf16(loc[0], loc[1].to(loc[0].dtype), norm.weight, norm.bias))
        out = F.linear_bf16(zn, self._w, out_dtype=loc[0].dtype)
        return _rewrap(out, pairs[0], p.shape[0])


class DistributedPairwiseConditioning(nn.Module):
    """``PairwiseConditioning`` on the local blocks of ``z_trunk`` and ``token_rel_pos_feats`` (every pair is
    independent: no communication); DTensors in, a DTensor with the first input's placements out."""

    def __init__(self, serial: nn.Module, device_mesh=None) -> None:
        super().__init__()
        from ..conditioning import PairwiseConditioning
        from ..swap import to_b200

        self.serial = serial if isinstance(serial, PairwiseConditioning) else to_b200(serial)
        self.device_mesh = device_mesh

    def forward(self, z_trunk, token_rel_pos_feats):
        loc = [x.to_local() if hasattr(x, "to_local") else x for x in (z_trunk, token_rel_pos_feats)]
        return _rewrap(self.serial(loc[0], loc[1]), z_trunk, self.serial.a_z)


__all__ = ["grid_of", "TriangleMultiplicationAddRes", "AttentionPairBias", "DistributedOuterProductMean",
           "DTensorAwareTransition", "LayerNormLinearParamsReplicatedTiled", "DistributedPairwiseConditioning"]
