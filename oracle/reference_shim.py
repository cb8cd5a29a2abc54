"""Import the reference's hot-path modules in place, on a machine that has them.

TEST INFRASTRUCTURE ONLY.  The reference package's ``__init__`` pulls
dependencies (mdtraj, rdkit) that this image lacks, so two stub modules are
registered before the hot-path files are imported from the reference checkout.
Used by ``tests/golden/make_golden.py`` and by the pinning tests, both of which
skip when the checkout is absent (it never travels to a GPU box).  The checkout is
found through the environment variable ``BIOEMU2_REFERENCE_SRC`` (the directory that
contains the ``bioemu2`` package) or, failing that, as a checkout named ``reference``
beside this repository; otherwise the shim reports "not available".
"""
from __future__ import annotations

import os
import sys
import types

_SIBLING = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference", "src")
REFERENCE_SRC = os.environ.get("BIOEMU2_REFERENCE_SRC") or (_SIBLING if os.path.isdir(_SIBLING) else "")


def available() -> bool:
    return bool(REFERENCE_SRC) and os.path.isdir(os.path.join(REFERENCE_SRC, "bioemu2", "biomoa", "ops"))


def install() -> None:
    """Register the stub packages; idempotent."""
    if "bioemu2" in sys.modules and getattr(sys.modules["bioemu2"], "_oracle_shim", False):
        return
    if not available():
        raise RuntimeError("reference checkout not found: set BIOEMU2_REFERENCE_SRC to the directory holding the "
                           "bioemu2 package")
    pkg = types.ModuleType("bioemu2")
    pkg.__path__ = [os.path.join(REFERENCE_SRC, "bioemu2")]
    pkg.HAS_TRITON = True  # src/bioemu2/__init__.py exports this flag
    pkg._oracle_shim = True
    sys.modules["bioemu2"] = pkg
    di = types.ModuleType("bioemu2.data_interface")
    di.__path__ = []
    sys.modules["bioemu2.data_interface"] = di
    const = types.ModuleType("bioemu2.data_interface.const")
    const.NUM_TOKENS = 33  # len(Token), src/bioemu2/data_interface/const.py:23,531
    sys.modules["bioemu2.data_interface.const"] = const


def modules():
    """Return the reference classes the oracle is pinned against."""
    install()
    from bioemu2.biomoa.modules.pairmixer import PairMixerLayer, PairMixerModule
    from bioemu2.biomoa.ops.attention_pair_bias import AttentionPairBias
    from bioemu2.biomoa.ops.outer_product_mean import OuterProductMeanVanilla
    from bioemu2.biomoa.ops.transition import Transition
    from bioemu2.biomoa.ops.triangle_multiplication import (
        TriangleMultiplicationFull,
        TriangleMultiplicationIncoming,
        TriangleMultiplicationOutgoing,
    )

    return types.SimpleNamespace(
        PairMixerLayer=PairMixerLayer,
        PairMixerModule=PairMixerModule,
        AttentionPairBias=AttentionPairBias,
        OuterProductMeanVanilla=OuterProductMeanVanilla,
        Transition=Transition,
        TriangleMultiplicationFull=TriangleMultiplicationFull,
        TriangleMultiplicationOutgoing=TriangleMultiplicationOutgoing,
        TriangleMultiplicationIncoming=TriangleMultiplicationIncoming,
    )
