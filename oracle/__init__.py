"""CPU oracle for the tensor-product / graph-convolution path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this; it is
used by ``tests/``, by the smoke check and by the CPU-baseline leg of the
benchmark as the checker / timed baseline, never as a compute path of the
library.
"""
