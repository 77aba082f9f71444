"""Irreducible representations of O(3) and direct sums of them.

Drop-in for the ``Irrep`` / ``Irreps`` types of the reference's torch-free e3nn
clone (reference: openequivariance/implementations/e3nn_lite.py:53-352).  The
classes are tuple subclasses so that ``(mul, (l, p))`` unpacking, hashing and
comparison behave exactly like e3nn's, which the problem builders rely on.

Data-layout contract that every kernel in this package follows: a feature row
is the concatenation, over the entries of an ``Irreps``, of a ``[mul][2l+1]``
block (multiplicity-major, "mul_ir"), and a batch of rows is row-major
``[batch][dim]``.
"""

from __future__ import annotations

import collections
import itertools
from typing import Iterator, List, Tuple

_PARITY_CHAR = {1: "e", -1: "o"}


def _inverse_permutation(perm):
    inv = [0] * len(perm)
    for position, value in enumerate(perm):
        inv[value] = position
    return tuple(inv)


class Irrep(tuple):
    """One irrep ``(l, p)`` of O(3): degree ``l >= 0`` and parity ``p = +-1``.

    Accepts ``Irrep("1o")``, ``Irrep(1, -1)``, ``Irrep((1, -1))`` or another
    ``Irrep``; the string suffix ``y`` means spherical-harmonic parity
    ``(-1)**l`` (reference: e3nn_lite.py:54-78).
    """

    def __new__(cls, l, p=None):
        if p is None:
            if isinstance(l, Irrep):
                return l
            if isinstance(l, str):
                text = l.strip()
                try:
                    degree = int(text[:-1])
                    if degree < 0:
                        raise ValueError
                    suffix = text[-1]
                    if suffix == "e":
                        parity = 1
                    elif suffix == "o":
                        parity = -1
                    elif suffix == "y":
                        parity = (-1) ** degree
                    else:
                        raise ValueError
                except Exception:
                    raise ValueError(f'unable to convert string "{text}" into an Irrep')
                l, p = degree, parity
            elif isinstance(l, tuple):
                l, p = l
        if not isinstance(l, int) or l < 0:
            raise ValueError(f"l must be positive integer, got {l}")
        if p not in (-1, 1):
            raise ValueError(f"parity must be on of (-1, 1), got {p}")
        return super().__new__(cls, (l, p))

    @property
    def l(self) -> int:
        return self[0]

    @property
    def p(self) -> int:
        return self[1]

    @property
    def dim(self) -> int:
        return 2 * self[0] + 1

    def is_scalar(self) -> bool:
        return self[0] == 0 and self[1] == 1

    def __repr__(self) -> str:
        return f"{self[0]}{_PARITY_CHAR[self[1]]}"

    @classmethod
    def iterator(cls, lmax=None) -> Iterator["Irrep"]:
        """All irreps in the order 0e, 0o, 1o, 1e, 2e, 2o, ..."""
        for degree in itertools.count():
            natural = (-1) ** degree
            yield Irrep(degree, natural)
            yield Irrep(degree, -natural)
            if degree == lmax:
                return

    def __mul__(self, other):
        """Irreps contained in the product of two irreps (selection rule)."""
        other = Irrep(other)
        parity = self.p * other.p
        for degree in range(abs(self.l - other.l), self.l + other.l + 1):
            yield Irrep(degree, parity)

    def __rmul__(self, other):
        assert isinstance(other, int)
        return Irreps([(other, self)])

    def __add__(self, other):
        return Irreps(self) + Irreps(other)

    # tuple methods that make no sense for an irrep
    def count(self, _value):
        raise NotImplementedError

    def index(self, _value):
        raise NotImplementedError

    def __contains__(self, _object):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError


class _MulIr(tuple):
    """``mul`` copies of one irrep (reference: e3nn_lite.py:157-188)."""

    def __new__(cls, mul, ir=None):
        if ir is None:
            mul, ir = mul
        assert isinstance(mul, int)
        assert isinstance(ir, Irrep)
        return super().__new__(cls, (mul, ir))

    @property
    def mul(self) -> int:
        return self[0]

    @property
    def ir(self) -> Irrep:
        return self[1]

    @property
    def dim(self) -> int:
        return self[0] * self[1].dim

    def __repr__(self) -> str:
        return f"{self[0]}x{self[1]}"

    def count(self, _value):
        raise NotImplementedError

    def index(self, _value):
        raise NotImplementedError


def _parse_irreps_string(text: str) -> List[_MulIr]:
    entries = []
    if text.strip() == "":
        return entries
    for term in text.split("+"):
        if "x" in term:
            mul_text, ir_text = term.split("x")
            mul = int(mul_text)
        else:
            mul, ir_text = 1, term
        if mul < 0:
            raise ValueError
        entries.append(_MulIr(mul, Irrep(ir_text)))
    return entries


class Irreps(tuple):
    """A direct sum of irreps with multiplicities, e.g. ``"128x0e+128x1o"``.

    Also accepts an e3nn ``Irreps`` object or any iterable of ``(mul, ir)`` /
    ``(mul, (l, p))`` / irrep strings (reference: e3nn_lite.py:191-238).
    """

    def __new__(cls, irreps=None):
        if isinstance(irreps, Irreps):
            return super().__new__(cls, irreps)
        entries: List[_MulIr] = []
        if irreps is None:
            pass
        elif isinstance(irreps, Irrep):
            entries.append(_MulIr(1, irreps))
        elif isinstance(irreps, str):
            try:
                entries = _parse_irreps_string(irreps)
            except Exception:
                raise ValueError(f'Unable to convert string "{irreps}" into an Irreps')
        else:
            for item in irreps:
                mul, ir = None, None
                if isinstance(item, str):
                    mul, ir = 1, Irrep(item)
                elif isinstance(item, Irrep):
                    mul, ir = 1, item
                elif isinstance(item, _MulIr):
                    mul, ir = item
                elif len(item) == 2:
                    mul, ir = item
                    ir = Irrep(tuple(ir)) if not isinstance(ir, (Irrep, str, int)) else Irrep(ir)
                if not (isinstance(mul, int) and mul >= 0 and ir is not None):
                    raise ValueError(f'Unable to interpret "{item}" as an irrep.')
                entries.append(_MulIr(mul, ir))
        return super().__new__(cls, entries)

    @staticmethod
    def spherical_harmonics(lmax: int, p: int = -1) -> "Irreps":
        return Irreps([(1, (l, p**l)) for l in range(lmax + 1)])

    def slices(self) -> List[slice]:
        """Column range of each entry inside a feature row."""
        out, start = [], 0
        for mul_ir in self:
            out.append(slice(start, start + mul_ir.dim))
            start += mul_ir.dim
        return out

    def offsets(self) -> List[int]:
        """First column of each entry inside a feature row."""
        return [s.start for s in self.slices()]

    def __getitem__(self, i):
        item = super().__getitem__(i)
        if isinstance(i, slice):
            return Irreps(item)
        return item

    def __contains__(self, ir) -> bool:
        ir = Irrep(ir)
        return any(ir == entry_ir for _, entry_ir in self)

    def count(self, ir) -> int:
        ir = Irrep(ir)
        return sum(mul for mul, entry_ir in self if entry_ir == ir)

    def index(self, _object):
        raise NotImplementedError

    def __add__(self, irreps) -> "Irreps":
        return Irreps(super().__add__(Irreps(irreps)))

    def __mul__(self, other) -> "Irreps":
        if isinstance(other, Irreps):
            raise NotImplementedError("Use o3.TensorProduct for this, see the documentation")
        return Irreps(super().__mul__(other))

    def __rmul__(self, other) -> "Irreps":
        return Irreps(super().__rmul__(other))

    def simplify(self) -> "Irreps":
        """Merge neighbouring entries with the same irrep, drop empty ones."""
        merged: List[Tuple[int, Irrep]] = []
        for mul, ir in self:
            if merged and merged[-1][1] == ir:
                merged[-1] = (merged[-1][0] + mul, ir)
            elif mul > 0:
                merged.append((mul, ir))
        return Irreps(merged)

    def remove_zero_multiplicities(self) -> "Irreps":
        return Irreps([(mul, ir) for mul, ir in self if mul > 0])

    def sort(self):
        """Stable sort by (l, p); returns ``(irreps, p, inv)`` like e3nn.

        ``inv[j]`` is the old position of the entry now at ``j`` and ``p`` is
        its inverse (reference: e3nn_lite.py:321-328).
        """
        Ret = collections.namedtuple("sort", ["irreps", "p", "inv"])
        keyed = sorted((ir, position, mul) for position, (mul, ir) in enumerate(self))
        inv = tuple(position for _, position, _ in keyed)
        return Ret(Irreps([(mul, ir) for ir, _, mul in keyed]), _inverse_permutation(inv), inv)

    def regroup(self) -> "Irreps":
        return self.sort().irreps.simplify()

    @property
    def dim(self) -> int:
        return sum(mul * ir.dim for mul, ir in self)

    @property
    def num_irreps(self) -> int:
        return sum(mul for mul, _ in self)

    @property
    def ls(self) -> List[int]:
        return [ir.l for mul, ir in self for _ in range(mul)]

    @property
    def lmax(self) -> int:
        if len(self) == 0:
            raise ValueError("Cannot get lmax of empty Irreps")
        return max(self.ls)

    def __repr__(self) -> str:
        return "+".join(repr(mul_ir) for mul_ir in self)
