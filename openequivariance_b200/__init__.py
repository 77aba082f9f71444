"""B200-native Clebsch-Gordan tensor products and fused graph convolution.

Drop-in for the public surface of OpenEquivariance (reference:
openequivariance/__init__.py:4-10): ``TPProblem``, ``Irreps``,
``TensorProduct`` and ``TensorProductConv`` keep their signatures, weight
layouts and autograd behaviour; the kernels behind them are hand-written
sm_100a CUDA reached through a C-ABI shared library.
"""

from .irreps import Irrep, Irreps
from .problem import (TPProblem, Instruction, FullyConnectedTPProblem, ChannelwiseTPP,
                      SingleInstruction)
from .wigner import wigner_3j

__all__ = ["Irrep", "Irreps", "TPProblem", "Instruction", "FullyConnectedTPProblem",
           "ChannelwiseTPP", "SingleInstruction", "wigner_3j", "TensorProduct",
           "TensorProductConv", "LoopUnrollTP", "LoopUnrollConv", "CoordGraph"]


def __getattr__(name):
    # torch-dependent front ends are imported on first use so that the problem
    # description stays importable without torch, like the reference's e3nn_lite
    if name in ("TensorProduct", "LoopUnrollTP"):
        from .tensor_product import TensorProduct
        return TensorProduct
    if name in ("TensorProductConv", "LoopUnrollConv", "CoordGraph"):
        from . import conv
        return {"TensorProductConv": conv.TensorProductConv, "LoopUnrollConv": conv.TensorProductConv,
                "CoordGraph": conv.CoordGraph}[name]
    raise AttributeError(name)
