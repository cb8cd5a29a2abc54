"""B200-native (sm_100a) kernels for BioEmu2's pair-representation hot path behind the reference's
``nn.Module`` contracts.  Importing the package loads the CUDA library; without it the import fails."""
from . import _lib  # noqa: F401  (fails loudly when the library is not built)
from . import context_parallel, functional, ieee, precision
from .attention_pair_bias import AttentionPairBias, AttentionPairBiasSlidingWindow, PairBiasCache
from .conditioning import PairwiseConditioning
from .outer_product_mean import (
    OuterProductMean,
    OuterProductMeanTritonMemorySaving,
    OuterProductMeanVanilla,
)
from .pairformer import PairformerBlock, PairformerModule
from .pair_weighted_averaging import PairWeightedAveraging
from .pairmixer import PairMixerLayer, PairMixerModule, PairMixerMSALayer
from .sequence_trunk import PairMixerMSAModule, PairMixerSequenceEmbedder
from .swap import swap_into, to_b200
from .transformer import AttentionLayer, ConditionedTransformerLayer, SlidingWindowAttentionLayer
from .transition import Transition
from .triangle_attention import (
    TriangleAttention,
    TriangleAttentionEndingNode,
    TriangleAttentionStartingNode,
)
from .triangle_multiplication import (
    TriangleMultiplication,
    TriangleMultiplicationIncoming,
    TriangleMultiplicationOutgoing,
)

__all__ = [
    "context_parallel",
    "functional",
    "ieee",
    "precision",
    "AttentionPairBias",
    "AttentionPairBiasSlidingWindow",
    "PairBiasCache",
    "OuterProductMean",
    "OuterProductMeanTritonMemorySaving",
    "OuterProductMeanVanilla",
    "AttentionLayer",
    "ConditionedTransformerLayer",
    "SlidingWindowAttentionLayer",
    "PairformerBlock",
    "PairformerModule",
    "PairMixerLayer",
    "PairMixerModule",
    "PairMixerMSALayer",
    "PairMixerMSAModule",
    "PairMixerSequenceEmbedder",
    "PairwiseConditioning",
    "PairWeightedAveraging",
    "swap_into",
    "to_b200",
    "Transition",
    "TriangleAttention",
    "TriangleAttentionEndingNode",
    "TriangleAttentionStartingNode",
    "TriangleMultiplication",
    "TriangleMultiplicationIncoming",
    "TriangleMultiplicationOutgoing",
]
