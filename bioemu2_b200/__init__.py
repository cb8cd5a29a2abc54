"""B200-native (sm_100a) kernels for BioEmu2's pair-representation hot path behind the reference's
``nn.Module`` contracts.  Importing the package loads the CUDA library; without it the import fails."""
from . import _lib  # noqa: F401  (fails loudly when the library is not built)
from . import functional
from .attention_pair_bias import AttentionPairBias
from .outer_product_mean import (
    OuterProductMean,
    OuterProductMeanTritonMemorySaving,
    OuterProductMeanVanilla,
)
from .pairmixer import PairMixerLayer, PairMixerModule
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
    "functional",
    "AttentionPairBias",
    "OuterProductMean",
    "OuterProductMeanTritonMemorySaving",
    "OuterProductMeanVanilla",
    "PairMixerLayer",
    "PairMixerModule",
    "Transition",
    "TriangleAttention",
    "TriangleAttentionEndingNode",
    "TriangleAttentionStartingNode",
    "TriangleMultiplication",
    "TriangleMultiplicationIncoming",
    "TriangleMultiplicationOutgoing",
]
