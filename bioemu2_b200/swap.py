"""Replace the reference's pair ops inside a loaded model by this package's modules.

The reference installs its context-parallel wrappers by swapping modules after the checkpoint is loaded
(``wrap_score_model_for_cp``, src/bioemu2/context_parallel/models/__init__.py:29-50); ``swap_into`` does the same
for the single-GPU kernels: it walks the module tree, recognises the reference's op classes by name (the reference
package is never imported here), builds the twin with the same constructor attributes, loads the original's
``state_dict`` strictly, and puts the twin in the original's place on the original's device.

Recognised classes (src/bioemu2/biomoa/ops/):
``TriangleMultiplicationFull / Cueq / CueqTiled / Outgoing / Incoming`` (triangle_multiplication.py:86-395),
``Transition`` (transition.py:17-91), ``AttentionPairBias`` (attention_pair_bias.py:42-225),
``OuterProductMeanVanilla / TritonMemorySaving`` (outer_product_mean.py:32-152),
``PairWeightedAveraging`` (pair_weighted_averaging.py:6-153).
A module whose sizes the kernels are not built for (for example a triangle multiplication of width 64) is left in
place and reported, unless ``strict=True``.
"""
from __future__ import annotations

import torch.nn as nn

from .attention_pair_bias import AttentionPairBias
from .outer_product_mean import OuterProductMean
from .pair_weighted_averaging import PairWeightedAveraging
from .transition import Transition
from .triangle_multiplication import TriangleMultiplication

_TRIMUL = {"TriangleMultiplicationFull", "TriangleMultiplicationCueq", "TriangleMultiplicationCueqTiled",
           "TriangleMultiplicationOutgoing", "TriangleMultiplicationIncoming"}
_OPM = {"OuterProductMeanVanilla", "OuterProductMeanTritonMemorySaving"}
_OWN = (TriangleMultiplication, Transition, AttentionPairBias, OuterProductMean, PairWeightedAveraging)


def _is_reference_op(m: nn.Module) -> bool:
    return type(m).__module__.startswith("bioemu2.biomoa.ops") and not isinstance(m, _OWN)


def to_b200(ref: nn.Module) -> nn.Module:
    """The twin of one reference op, carrying its weights; ``ref`` itself when it is not one of the recognised ops.
    Raises ``ValueError`` when the op is recognised but has sizes the kernels are not built for."""
    if not _is_reference_op(ref):
        return ref
    name = type(ref).__name__
    if name in _TRIMUL:
        new = TriangleMultiplication(ref.norm_in.normalized_shape[0], ref.mode)
    elif name == "Transition":
        new = Transition(ref.fc1.in_features, ref.fc1.out_features, ref.fc3.out_features, use_norm=ref.use_norm,
                         chunk_size=getattr(ref, "chunk_size", None))
    elif name == "AttentionPairBias":
        new = AttentionPairBias(ref.proj_g.in_features, ref.proj_z.in_features, ref.num_heads, inf=ref.inf,
                                initial_norm=ref.initial_norm, tile_size=getattr(ref, "tile_size", 512),
                                use_bias_in_layer_norm=ref.norm_z.bias is not None)
    elif name == "PairWeightedAveraging":
        new = PairWeightedAveraging(ref.c_m, ref.c_z, ref.c_h, ref.num_heads, inf=ref.inf,
                                    use_bias_in_layer_norm=ref.norm_z.bias is not None)
    elif name in _OPM:
        new = OuterProductMean(ref.norm.normalized_shape[0], ref.c_hidden, ref.proj_o.out_features,
                               tile_size=getattr(ref, "tile_size", None))
    else:
        return ref
    new.load_state_dict(ref.state_dict(), strict=True)
    param = next(ref.parameters(), None)
    if param is not None:
        new = new.to(param.device)
    return new.eval()


def swap_into(model: nn.Module, strict: bool = False) -> dict[str, tuple[str, str]]:
    """Swap every recognised op below ``model`` in place.  Returns ``{module path: (old class, new class or reason)}``;
    with ``strict`` an op the kernels cannot serve raises instead of being left in place."""
    report: dict[str, tuple[str, str]] = {}

    def walk(parent: nn.Module, prefix: str) -> None:
        for name, child in list(parent.named_children()):
            path = f"{prefix}.{name}" if prefix else name
            if _is_reference_op(child) and (type(child).__name__ in _TRIMUL | _OPM | {"Transition", "AttentionPairBias", "PairWeightedAveraging"}):
                try:
                    twin = to_b200(child)
                except ValueError as exc:
                    if strict:
                        raise
                    report[path] = (type(child).__name__, f"kept: {exc}")
                    continue
                setattr(parent, name, twin)
                report[path] = (type(child).__name__, type(twin).__name__)
            else:
                walk(child, path)

    walk(model, "")
    return report
