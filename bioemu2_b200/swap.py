"""Replace the reference's pair ops inside a loaded model by this package's modules.

The reference installs its context-parallel wrappers by swapping modules after the checkpoint is loaded
(``wrap_score_model_for_cp``, src/bioemu2/context_parallel/models/__init__.py:29-50); ``swap_into`` does the same
for the single-GPU kernels: it walks the module tree, recognises the reference's op classes by name (the reference
package is never imported here), builds the twin with the same constructor attributes, loads the original's
``state_dict`` strictly, and puts the twin in the original's place on the original's device.

Recognised classes (src/bioemu2/biomoa/ops/):
``TriangleMultiplicationFull / Cueq / CueqTiled / Outgoing / Incoming`` (triangle_multiplication.py:86-395),
``Transition`` (transition.py:17-91), ``AttentionPairBias`` (attention_pair_bias.py:42-225),
``AttentionPairBiasSlidingWindow`` (attention_pair_bias.py:228-340),
``OuterProductMeanVanilla / TritonMemorySaving`` (outer_product_mean.py:32-152),
``PairWeightedAveraging`` (pair_weighted_averaging.py:6-153).
Three of the reference's composite modules are swapped as a whole, glue included (src/bioemu2/biomoa/modules/):
``PairwiseConditioning`` (diffusion.py:464-534), ``PairMixerMSAModule`` (pairmixer.py:459-612) and
``PairMixerSequenceEmbedder`` (pairmixer.py:23-299; its feature encoders are moved across unchanged).
A module whose sizes the kernels are not built for (for example a triangle multiplication of width 64) is left in
place and reported, unless ``strict=True``.
"""
from __future__ import annotations

import torch.nn as nn

from .attention_pair_bias import AttentionPairBias, AttentionPairBiasSlidingWindow
from .conditioning import PairwiseConditioning
from .outer_product_mean import OuterProductMean
from .pair_weighted_averaging import PairWeightedAveraging
from .sequence_trunk import PairMixerMSAModule, PairMixerSequenceEmbedder
from .transition import Transition
from .triangle_multiplication import TriangleMultiplication

_TRIMUL = {"TriangleMultiplicationFull", "TriangleMultiplicationCueq", "TriangleMultiplicationCueqTiled",
           "TriangleMultiplicationOutgoing", "TriangleMultiplicationIncoming"}
_OPM = {"OuterProductMeanVanilla", "OuterProductMeanTritonMemorySaving"}
_COMPOSITE = {"PairwiseConditioning", "PairMixerMSAModule", "PairMixerSequenceEmbedder"}
_ENCODERS = ("rel_pos", "token_bonds", "contact_conditioning", "method_conditioning")
_OWN = (TriangleMultiplication, Transition, AttentionPairBias, OuterProductMean, PairWeightedAveraging,
        PairwiseConditioning, PairMixerMSAModule, PairMixerSequenceEmbedder)


def _is_reference_op(m: nn.Module) -> bool:
    mod = type(m).__module__
    if isinstance(m, _OWN):
        return False
    return mod.startswith("bioemu2.biomoa.ops") or (mod.startswith("bioemu2.biomoa.modules") and
                                                     type(m).__name__ in _COMPOSITE)


def _msa_module_args(ref: nn.Module) -> dict:
    paired = bool(ref.use_paired_feature)
    return dict(msa_s=ref.s_proj.out_features, s_input_dim=ref.s_proj.in_features, msa_blocks=len(ref.layers),
                use_paired_feature=paired, num_tokens=ref.msa_proj.in_features - 2 - int(paired))


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
    elif name == "AttentionPairBiasSlidingWindow":
        new = AttentionPairBiasSlidingWindow(ref.proj_g.in_features, ref.proj_z.in_features, ref.num_heads,
                                             window_queries=ref.window_queries, window_keys=ref.window_keys, inf=ref.inf,
                                             initial_norm=ref.initial_norm, tile_size=getattr(ref, "tile_size", 512),
                                             use_bias_in_layer_norm=ref.norm_z.bias is not None)
    elif name == "PairWeightedAveraging":
        new = PairWeightedAveraging(ref.c_m, ref.c_z, ref.c_h, ref.num_heads, inf=ref.inf,
                                    use_bias_in_layer_norm=ref.norm_z.bias is not None)
    elif name in _OPM:
        new = OuterProductMean(ref.norm.normalized_shape[0], ref.c_hidden, ref.proj_o.out_features,
                               tile_size=getattr(ref, "tile_size", None))
    elif name == "PairwiseConditioning":
        ln, lin = ref.dim_pairwise_init_proj[0], ref.dim_pairwise_init_proj[1]
        t0 = ref.transitions[0] if len(ref.transitions) else None
        a_z = lin.out_features
        token_z = getattr(ref, "token_z", a_z)
        new = PairwiseConditioning(token_z, ln.normalized_shape[0] - token_z, a_z, num_transitions=len(ref.transitions),
                                   transition_expansion_factor=(t0.fc1.out_features // a_z) if t0 is not None else 2)
    elif name == "PairMixerMSAModule":
        a = _msa_module_args(ref)
        new = PairMixerMSAModule(token_s=getattr(ref, "token_s", 384), token_z=ref.layers[0].tri_mul_out.norm_in.normalized_shape[0],
                                 **a)
    elif name == "PairMixerSequenceEmbedder":
        a = _msa_module_args(ref.msa_module)
        new = PairMixerSequenceEmbedder(
            token_s=ref.s_init.out_features, token_z=ref.z_init_1.out_features, s_input_dim=ref.s_init.in_features,
            msa_s=a["msa_s"], msa_blocks=a["msa_blocks"], num_blocks=len(ref.pairmixer_module.layers),
            use_contact_conditioning=ref.use_contact_conditioning, use_method_conditioning=ref.use_method_conditioning,
            use_paired_feature=a["use_paired_feature"], use_unconditional_branch=ref.use_unconditional_branch,
            num_tokens=a["num_tokens"])
        for enc in _ENCODERS:  # input featurisation stays the reference's own modules
            if isinstance(getattr(ref, enc, None), nn.Module):
                setattr(new, enc, getattr(ref, enc))
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
            if _is_reference_op(child) and (type(child).__name__ in _TRIMUL | _OPM | _COMPOSITE | {
                    "Transition", "AttentionPairBias", "AttentionPairBiasSlidingWindow", "PairWeightedAveraging"}):
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
