"""Real-basis Clebsch-Gordan (Wigner 3j) tensors, in e3nn's conventions.

``wigner_3j(l1, l2, l3)`` returns the tensor ``C[2l1+1, 2l2+1, 2l3+1]`` that is
invariant under simultaneous rotation of its three indices in the real
spherical-harmonic basis, with unit Frobenius norm.  Values, signs and index
order equal the reference's generator (reference:
openequivariance/implementations/e3nn_lite.py:573-771), which the kernels bake
in as compile-time constants: the SU(2) coefficients come from Racah's closed
form evaluated in exact rational arithmetic, and are rotated to the real basis
with the change-of-basis matrix of the real spherical harmonics times
``(-i)**l`` (which is what makes the result real).
"""

from __future__ import annotations

import functools
from fractions import Fraction
from math import factorial

import numpy as np


def _racah_cg(j1: int, m1: int, j2: int, m2: int, j3: int, m3: int) -> float:
    """<j1 m1; j2 m2 | j3 m3> for integer spins (Racah's formula)."""
    if m3 != m1 + m2:
        return 0.0
    norm2 = (2 * j3 + 1) * Fraction(
        factorial(j3 + j1 - j2) * factorial(j3 - j1 + j2) * factorial(j1 + j2 - j3)
        * factorial(j3 + m3) * factorial(j3 - m3),
        factorial(j1 + j2 + j3 + 1) * factorial(j1 - m1) * factorial(j1 + m1)
        * factorial(j2 - m2) * factorial(j2 + m2),
    )
    lo = max(-j1 + j2 + m3, -j1 + m1, 0)
    hi = min(j2 + j3 + m1, j3 - j1 + j2, j3 + m3)
    total = Fraction(0)
    for v in range(lo, hi + 1):
        sign = -1 if (v + j2 + m2) % 2 else 1
        total += sign * Fraction(
            factorial(j2 + j3 + m1 - v) * factorial(j1 - m1 + v),
            factorial(v) * factorial(j3 - j1 + j2 - v) * factorial(j3 + m3 - v)
            * factorial(v + j1 - j2 - m3),
        )
    return float(norm2) ** 0.5 * float(total)


def _complex_cg(l1: int, l2: int, l3: int) -> np.ndarray:
    """SU(2) coupling tensor indexed ``[l1+m1, l2+m2, l3+m3]``."""
    out = np.zeros((2 * l1 + 1, 2 * l2 + 1, 2 * l3 + 1), dtype=np.float64)
    if not abs(l1 - l2) <= l3 <= l1 + l2:
        return out
    for m1 in range(-l1, l1 + 1):
        for m2 in range(-l2, l2 + 1):
            m3 = m1 + m2
            if abs(m3) <= l3:
                out[l1 + m1, l2 + m2, l3 + m3] = _racah_cg(l1, m1, l2, m2, l3, m3)
    return out


def real_to_complex_basis(l: int) -> np.ndarray:
    """Unitary ``Q[2l+1, 2l+1]`` taking real SH components to complex ones.

    Includes the global phase ``(-i)**l`` used by e3nn (reference:
    e3nn_lite.py:573-591).
    """
    q = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
    s = 2.0 ** -0.5
    q[l, l] = 1.0
    for m in range(1, l + 1):
        sign = (-1) ** m
        # row for -m
        q[l - m, l + m] = s
        q[l - m, l - m] = -1j * s
        # row for +m
        q[l + m, l + m] = sign * s
        q[l + m, l - m] = 1j * sign * s
    return (-1j) ** l * q


@functools.lru_cache(maxsize=None)
def _real_cg(l1: int, l2: int, l3: int) -> np.ndarray:
    q1 = real_to_complex_basis(l1)
    q2 = real_to_complex_basis(l2)
    q3 = real_to_complex_basis(l3)
    coupling = _complex_cg(l1, l2, l3).astype(np.complex128)
    rotated = np.einsum("ij,kl,mn,ikn->jlm", q1, q2, np.conj(q3.T), coupling)
    if not np.all(np.abs(rotated.imag) < 1e-5):
        raise ArithmeticError(f"Clebsch-Gordan tensor ({l1},{l2},{l3}) is not real")
    real = np.ascontiguousarray(rotated.real)
    real /= np.linalg.norm(real.ravel())
    real.setflags(write=False)
    return real


def wigner_3j(l1: int, l2: int, l3: int, dtype=np.float64) -> np.ndarray:
    """Real Wigner 3j tensor of shape ``(2l1+1, 2l2+1, 2l3+1)``, a fresh copy."""
    assert isinstance(l1, int) and isinstance(l2, int) and isinstance(l3, int)
    assert abs(l2 - l3) <= l1 <= l2 + l3
    return np.array(_real_cg(l1, l2, l3), dtype=dtype)


def cg_nonzeros(l1: int, l2: int, l3: int, tol: float = 1e-12):
    """Sparse form ``[(i, j, k, value), ...]`` of ``wigner_3j`` in row-major order.

    Entries that the change of basis leaves at round-off level are structural
    zeros and are dropped.
    """
    dense = _real_cg(l1, l2, l3)
    return [(int(i), int(j), int(k), float(dense[i, j, k]))
            for i, j, k in zip(*np.nonzero(np.abs(dense) > tol))]
