"""CPU oracle for the pair-representation hot path.

TEST INFRASTRUCTURE ONLY.  Nothing under this package is part of the product:
it restates, in plain fp32/fp64 torch on the CPU, the algorithms of the
reference modules so that the CUDA kernels have something to be checked
against.  Only the test-suite, the smoke check and the ``cpu_baseline`` /
``--impl reference`` legs of the benchmark may import it; the package
``bioemu2_b200`` never does and raises when its CUDA library is missing.

Parity status: PINNED for triangle multiplication, transition, pair-bias
attention, outer product mean and the PairMixer layer -- each restatement is
checked against the reference's own torch modules (imported in place through
``oracle.reference_shim``) and against the golden vectors those modules
produced (``tests/golden``).  UNPINNED for triangle attention, which the
reference does not contain.
"""
