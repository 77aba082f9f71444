"""Tensor-product problem description: irreps, instructions, normalisation.

``TPProblem`` keeps the constructor signature, attribute names and numeric
conventions of the reference (reference:
openequivariance/implementations/e3nn_lite.py:365-571), which in turn follow
``e3nn.o3.TensorProduct``:

* an instruction is ``(i_in1, i_in2, i_out, mode, has_weight[, path_weight])``;
* the stored ``Instruction.path_weight`` is ``sqrt(alpha)`` where ``alpha``
  combines the irrep normalisation, the path normalisation, ``out_var`` and the
  user's path weight;
* weights are flattened instruction-major, each instruction's block having
  ``path_shape`` (``(u, v)`` for "uvu", ``(u, v, w)`` for "uvw").

The problem builders below restate the instruction-enumeration rules of the
reference's benchmark helpers (reference:
openequivariance/benchmark/tpp_creation_utils.py:15-36, 118-181).
"""

from __future__ import annotations

from math import prod, sqrt
from typing import List, NamedTuple, Optional, Tuple

import numpy as np

from .irreps import Irrep, Irreps, _MulIr

_MODES = ("uvw", "uvu", "uvv", "uuw", "uuu", "uvuv", "uvu<v", "u<vw")


class Instruction(NamedTuple):
    i_in1: int
    i_in2: int
    i_out: int
    connection_mode: str
    has_weight: bool
    path_weight: float
    path_shape: tuple


def _path_shape(mode: str, m1: int, m2: int, m3: int) -> tuple:
    if mode == "uvw":
        return (m1, m2, m3)
    if mode in ("uvu", "uvv", "uvuv"):
        return (m1, m2)
    if mode == "uuw":
        return (m1, m3)
    if mode == "uuu":
        return (m1,)
    if mode == "uvu<v":
        return (m1 * (m2 - 1) // 2,)
    if mode == "u<vw":
        return (m1 * (m2 - 1) // 2, m3)
    raise ValueError(f"unknown connection mode {mode!r}")


def _fan_in(mode: str, m1: int, m2: int) -> int:
    """Number of input pairs summed into one output element (e3nn's num_elements)."""
    if mode == "uvw":
        return m1 * m2
    if mode == "uvu":
        return m2
    if mode in ("uvv", "uuw"):
        return m1
    if mode in ("uuu", "uvuv", "uvu<v"):
        return 1
    if mode == "u<vw":
        return m1 * (m2 - 1) // 2
    raise ValueError(f"unknown connection mode {mode!r}")


def _variances(values, count: int, what: str) -> List[float]:
    if values is None:
        return [1.0] * count
    values = [float(v) for v in values]
    assert len(values) == count, f"Len of {what} must be equal to len(irreps)"
    return values


class TPProblem:
    """Immutable description of one weighted Clebsch-Gordan tensor product."""

    def __init__(
        self,
        irreps_in1,
        irreps_in2,
        irreps_out,
        instructions: List[tuple],
        in1_var: Optional[List[float]] = None,
        in2_var: Optional[List[float]] = None,
        out_var: Optional[List[float]] = None,
        irrep_normalization: str = "component",
        path_normalization: str = "element",
        internal_weights: Optional[bool] = None,
        shared_weights: Optional[bool] = None,
        label: Optional[str] = None,
        irrep_dtype=np.float32,
        weight_dtype=np.float32,
    ) -> None:
        assert irrep_normalization in ["component", "norm", "none"]
        assert path_normalization in ["element", "path", "none"]
        assert issubclass(irrep_dtype, np.generic)
        assert issubclass(weight_dtype, np.generic)

        self.irreps_in1 = Irreps(irreps_in1)
        self.irreps_in2 = Irreps(irreps_in2)
        self.irreps_out = Irreps(irreps_out)
        self.instructions_raw = instructions
        self.in1_var, self.in2_var, self.out_var = in1_var, in2_var, out_var
        self.irrep_normalization = irrep_normalization
        self.path_normalization = path_normalization
        self.label = label

        v1 = _variances(in1_var, len(self.irreps_in1), "ir1_var")
        v2 = _variances(in2_var, len(self.irreps_in2), "ir2_var")
        v3 = _variances(out_var, len(self.irreps_out), "out_var")

        staged = []
        for raw in instructions:
            raw = tuple(raw)
            if len(raw) == 5:
                raw = raw + (1.0,)
            i1, i2, io, mode, has_weight, user_weight = raw
            assert mode in _MODES
            a, b, c = self.irreps_in1[i1], self.irreps_in2[i2], self.irreps_out[io]
            assert a.ir.p * b.ir.p == c.ir.p
            assert abs(a.ir.l - b.ir.l) <= c.ir.l <= a.ir.l + b.ir.l
            staged.append((i1, i2, io, mode, has_weight, user_weight,
                           _path_shape(mode, a.mul, b.mul, c.mul)))

        def fan(entry):
            return _fan_in(entry[3], self.irreps_in1[entry[0]].mul, self.irreps_in2[entry[1]].mul)

        self.instructions: List[Instruction] = []
        for entry in staged:
            i1, i2, io, mode, has_weight, user_weight, shape = entry
            a, b, c = self.irreps_in1[i1], self.irreps_in2[i2], self.irreps_out[io]
            if irrep_normalization == "component":
                alpha = c.ir.dim
            elif irrep_normalization == "norm":
                alpha = a.ir.dim * b.ir.dim
            else:
                alpha = 1
            siblings = [other for other in staged if other[2] == io]
            if path_normalization == "element":
                denom = sum(v1[o[0]] * v2[o[1]] * fan(o) for o in siblings)
            elif path_normalization == "path":
                denom = v1[i1] * v2[i2] * fan(entry) * len(siblings)
            else:
                denom = 1
            if denom > 0.0:
                alpha /= denom
            alpha *= v3[io]
            alpha *= user_weight
            self.instructions.append(Instruction(i1, i2, io, mode, has_weight, sqrt(alpha), shape))

        self._in1_dim = self.irreps_in1.dim
        self._in2_dim = self.irreps_in2.dim

        if shared_weights is False and internal_weights is None:
            internal_weights = False
        if shared_weights is None:
            shared_weights = True
        if internal_weights is None:
            internal_weights = shared_weights and any(i.has_weight for i in self.instructions)
        assert shared_weights or not internal_weights
        self.internal_weights = internal_weights
        self.shared_weights = shared_weights

        self.weight_numel = sum(prod(i.path_shape) for i in self.instructions if i.has_weight)
        self.output_mask = None
        self.irrep_dtype = irrep_dtype
        self.weight_dtype = weight_dtype

    def weight_range_and_shape_for_instruction(self, instruction: int) -> Tuple[int, int, tuple]:
        ins = self.instructions[instruction]
        if not ins.has_weight:
            raise ValueError(f"Instruction {instruction} has no weights.")
        start = sum(prod(i.path_shape) for i in self.instructions[:instruction])
        return start, start + prod(ins.path_shape), ins.path_shape

    def __str__(self) -> str:
        return (f"{self.__class__.__name__}({self.irreps_in1.simplify()} x "
                f"{self.irreps_in2.simplify()}) -> {self.irreps_out.simplify()}")

    def __repr__(self) -> str:
        lines = [str(self)]
        for name in ("irrep_normalization", "path_normalization", "internal_weights",
                     "shared_weights", "in1_var", "in2_var", "out_var"):
            lines.append(f"{name} = {getattr(self, name)!r}")
        lines.append(f"num weights {self.weight_numel}")
        lines.append("| in1 | in2 | out | l1 | l2 | l3 | m1 | m2 | m3 | mode | weight | path |")
        for ins in self.instructions:
            a = self.irreps_in1[ins.i_in1]
            b = self.irreps_in2[ins.i_in2]
            c = self.irreps_out[ins.i_out]
            lines.append(
                f"| {ins.i_in1:3} | {ins.i_in2:3} | {ins.i_out:3} | {a.ir.l:2} | {b.ir.l:2} | {c.ir.l:2} |"
                f" {a.mul:3} | {b.mul:3} | {c.mul:3} | {ins.connection_mode:<4} |"
                f" {str(ins.has_weight):<5} | {ins.path_weight:<4.2f} |")
        return "\n".join(lines) + "\n"


class FullyConnectedTPProblem(TPProblem):
    """Every selection-rule-allowed (in1, in2, out) triple as a weighted "uvw" path."""

    def __init__(self, irreps_in1, irreps_in2, irreps_out, **kwargs) -> None:
        in1, in2, out = Irreps(irreps_in1), Irreps(irreps_in2), Irreps(irreps_out)
        paths = []
        for i1, (_, ir1) in enumerate(in1):
            for i2, (_, ir2) in enumerate(in2):
                allowed = list(ir1 * ir2)
                for io, (_, ir3) in enumerate(out):
                    if ir3 in allowed:
                        paths.append((i1, i2, io, "uvw", True, 1.0))
        super().__init__(in1, in2, out, paths, **kwargs)


class ChannelwiseTPP(TPProblem):
    """MACE/Nequip-style channel-wise "uvu" product with per-row weights.

    One output block (of the in1 multiplicity) per allowed (in1, in2, l_out)
    triple whose irrep occurs in ``irreps_out``; blocks sorted by (l, p) and
    instructions ordered by output block.
    """

    def __init__(self, irreps_in1, irreps_in2, irreps_out, label: Optional[str] = None,
                 irrep_dtype=np.float32, weight_dtype=np.float32):
        in1, in2, wanted = Irreps(irreps_in1), Irreps(irreps_in2), Irreps(irreps_out)
        blocks, paths = [], []
        for i1, (mul, ir1) in enumerate(in1):
            for i2, (_, ir2) in enumerate(in2):
                for ir3 in ir1 * ir2:
                    if ir3 in wanted:
                        paths.append((i1, i2, len(blocks), "uvu", True))
                        blocks.append((mul, ir3))
        out, new_position, _ = Irreps(blocks).sort()
        paths = sorted(((i1, i2, new_position[io], mode, w) for i1, i2, io, mode, w in paths),
                       key=lambda path: path[2])
        super().__init__(in1, in2, out, paths, internal_weights=False, shared_weights=False,
                         label=label, irrep_dtype=irrep_dtype, weight_dtype=weight_dtype)


class SingleInstruction(TPProblem):
    """One weighted instruction (0, 0, 0, mode) with per-row weights."""

    def __init__(self, irreps_in1, irreps_in2, irreps_in3, mode: str, label: Optional[str] = None,
                 irrep_dtype=np.float32, weight_dtype=np.float32):
        super().__init__(Irreps(irreps_in1), Irreps(irreps_in2), Irreps(irreps_in3),
                         [(0, 0, 0, mode, True)], internal_weights=False, shared_weights=False,
                         label=label, irrep_dtype=irrep_dtype, weight_dtype=weight_dtype)


__all__ = ["Instruction", "TPProblem", "FullyConnectedTPProblem", "ChannelwiseTPP",
           "SingleInstruction", "Irrep", "Irreps", "_MulIr"]
