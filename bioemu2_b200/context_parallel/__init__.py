"""2D context parallelism for the pair-representation path: one process per GPU, the pair tensor tiled over an
R x C grid, NCCL all-gather / reduce-scatter over row and column groups around the single-GPU kernels."""
from .mesh import CPGrid, GridCoords, kernel_shard_multiple, pad_amount, shard_multiple, shard_range
from .modules import (
    CPPairMixerLayer,
    CPPairMixerModule,
    CPTransition,
    CPTriangleMultiplication,
)
from .trimul import cp_triangle_multiplication_

__all__ = [
    "CPGrid", "GridCoords", "kernel_shard_multiple", "pad_amount", "shard_multiple", "shard_range",
    "CPPairMixerLayer", "CPPairMixerModule", "CPTransition", "CPTriangleMultiplication", "cp_triangle_multiplication_",
]
