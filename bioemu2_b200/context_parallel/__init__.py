"""2D context parallelism for the pair-representation path: one process per GPU, the pair tensor tiled over an
R x C grid, NCCL all-gather / reduce-scatter over row and column groups around the single-GPU kernels."""
from .mesh import CPGrid, GridCoords, kernel_shard_multiple, pad_amount, shard_multiple, shard_range
from .attention import (cp_attention_pair_bias, cp_outer_product_mean, cp_pair_weighted_averaging,
                        cp_triangle_attention_)
from . import ops
from .modules import (
    CPAttentionPairBias,
    CPConditionedTransformerLayer,
    DistributedConditionedTransformerLayer,
    DistributedPairMixerLayer,
    DistributedPairMixerModule,
    CPOuterProductMean,
    CPPairMixerMSALayer,
    CPPairMixerMSAModule,
    CPPairMixerSequenceEmbedder,
    DistributedPairMixerMSAModule,
    PairMixerSequenceEmbedderDistributed,
    CPPairWeightedAveraging,
    DistributedPairMixerMSALayer,
    DistributedPairWeightedAveraging,
    CPPairformerBlock,
    CPPairformerModule,
    CPPairMixerLayer,
    CPPairMixerModule,
    CPTransition,
    CPTriangleAttention,
    CPTriangleMultiplication,
)
from .trimul import cp_triangle_multiplication_

__all__ = [
    "CPGrid", "GridCoords", "kernel_shard_multiple", "pad_amount", "shard_multiple", "shard_range",
    "ops", "CPConditionedTransformerLayer", "DistributedConditionedTransformerLayer", "DistributedPairMixerLayer",
    "DistributedPairMixerModule", "CPAttentionPairBias", "CPOuterProductMean", "CPPairformerBlock", "CPPairformerModule", "CPPairMixerLayer", "CPPairMixerModule", "CPTransition",
    "CPTriangleAttention", "CPTriangleMultiplication", "cp_attention_pair_bias", "cp_outer_product_mean",
    "cp_triangle_attention_", "cp_triangle_multiplication_", "cp_pair_weighted_averaging", "CPPairMixerMSALayer",
    "CPPairMixerMSAModule", "CPPairMixerSequenceEmbedder", "DistributedPairMixerMSAModule", "PairMixerSequenceEmbedderDistributed",
    "CPPairWeightedAveraging", "DistributedPairMixerMSALayer", "DistributedPairWeightedAveraging",
]
