"""CPU oracle for the fused Pairformer operators.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory; it is used by the test
suite, by the smoke check and by the CPU-baseline leg of the benchmark as the
checker the CUDA path is compared against.
"""
from .pairformer_oracle import *  # noqa: F401,F403
