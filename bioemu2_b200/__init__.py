"""B200-native (sm_100a) kernels for BioEmu2's pair-representation hot path behind the reference's
``nn.Module`` contracts.  Importing the package loads the CUDA library; without it the import fails."""
from . import _lib  # noqa: F401  (fails loudly when the library is not built)
from . import functional
from .pairmixer import PairMixerLayer, PairMixerModule
from .transition import Transition
from .triangle_multiplication import (
    TriangleMultiplication,
    TriangleMultiplicationIncoming,
    TriangleMultiplicationOutgoing,
)

__all__ = [
    "functional",
    "PairMixerLayer",
    "PairMixerModule",
    "Transition",
    "TriangleMultiplication",
    "TriangleMultiplicationIncoming",
    "TriangleMultiplicationOutgoing",
]
