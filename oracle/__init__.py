"""CPU oracle for the FP8 transformer inference forward path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this directory; only
the test-suite, the smoke check and the benchmark's CPU-baseline leg may.

The oracle is a NumPy + ``ml_dtypes`` restatement of the reference's JAX code with
*strict per-op dtype semantics*: every array operation produces a value rounded
(round-to-nearest-even) to the dtype JAX's promotion rules give it; dots and reductions
accumulate in float32 and round once.

PARITY UNPINNED: the reference cannot be executed in this environment (JAX, jaxlib and
Equinox are not installed and cannot be installed), and its own tests hold no golden
vectors or known-answer values for this path -- only relational properties, which
``tests/test_oracle_*.py`` re-express against this restatement.  The golden fixtures
under ``tests/golden`` are therefore produced *by this oracle*, not by the reference.
"""

from . import attention, fp8, llm  # noqa: F401
