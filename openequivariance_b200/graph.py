"""Synthetic atomistic graphs for benchmarks and tests.

The reference's convolution benchmarks read three graph pickles that are
downloaded at run time (reference: test/benchmark.py:158-177) and are not
available offline; the benchmark here uses seeded random point clouds of the
same kind instead: points uniform in a periodic unit cube, an edge in both
directions for every pair closer than a cutoff chosen for a target mean degree,
edges ordered exactly as the reference's ``CoordGraph`` orders them
(reference: openequivariance/implementations/convolution/ConvolutionBase.py:45-70),
and real spherical harmonics of the unit edge vectors as edge features.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np


@dataclass
class PeriodicGraph:
    coords: np.ndarray          # [N, 3] in [0, 1)
    rows: np.ndarray            # [E] receiver of each edge, non-decreasing
    cols: np.ndarray            # [E] sender of each edge
    sender_perm: np.ndarray     # [E] k-th edge in (sender, receiver) order
    vectors: np.ndarray         # [E, 3] minimum-image vector receiver -> sender, unit length
    cutoff: float

    @property
    def node_count(self):
        return self.coords.shape[0]

    @property
    def nnz(self):
        return self.rows.shape[0]


def morton_order(coords: np.ndarray, bits: int = 10) -> np.ndarray:
    """Permutation that sorts points along a Z-order curve (spatial locality of node ids)."""
    q = np.minimum((coords * (1 << bits)).astype(np.uint64), (1 << bits) - 1)
    code = np.zeros(coords.shape[0], dtype=np.uint64)
    for b in range(bits):
        for axis in range(3):
            code |= ((q[:, axis] >> np.uint64(b)) & np.uint64(1)) << np.uint64(3 * b + axis)
    return np.argsort(code, kind="stable")


def cutoff_for_degree(nodes: int, degree: float) -> float:
    """Radius whose ball holds ``degree`` other points on average at unit density ``nodes``."""
    return (3.0 * degree / (4.0 * math.pi * nodes)) ** (1.0 / 3.0)


def periodic_radius_graph(nodes: int, degree: float, seed: int = 11111, numbering: str = "morton") -> PeriodicGraph:
    """Points ~ U[0,1)^3 with periodic boundaries; both directions of every pair within the cutoff."""
    from scipy.spatial import cKDTree

    rng = np.random.default_rng(seed)
    coords = rng.uniform(size=(nodes, 3))
    if numbering == "morton":
        coords = coords[morton_order(coords)]
    elif numbering != "random":
        raise ValueError("numbering must be 'morton' or 'random'")
    cutoff = cutoff_for_degree(nodes, degree)
    tree = cKDTree(coords, boxsize=1.0)
    pairs = tree.query_pairs(cutoff, output_type="ndarray").astype(np.int64)
    rows = np.concatenate([pairs[:, 0], pairs[:, 1]])
    cols = np.concatenate([pairs[:, 1], pairs[:, 0]])
    order = np.lexsort((cols, rows))
    rows, cols = rows[order], cols[order]
    sender_perm = np.lexsort((rows, cols)).astype(np.int64)
    delta = coords[cols] - coords[rows]
    delta -= np.round(delta)                                  # minimum image
    norm = np.linalg.norm(delta, axis=1, keepdims=True)
    vectors = delta / np.maximum(norm, 1e-30)
    return PeriodicGraph(coords, rows, cols, sender_perm, vectors, cutoff)


def spherical_harmonics(lmax: int, vectors, normalization: str = "component"):
    """Real spherical harmonics ``[E, (lmax+1)^2]`` of unit vectors for ``lmax <= 3``.

    Component ordering within each l is m = -l..l in the (y, z, x) axis
    convention of e3nn; "component" normalisation gives every l block squared
    norm ``2l+1``.  Works on numpy arrays and torch tensors.  The harmonics are
    only an *input* of the tensor product, so the convention cannot affect
    parity between kernels and oracle.
    """
    if lmax > 3:
        raise ValueError("closed forms are provided up to l = 3")
    x, y, z = vectors[..., 0], vectors[..., 1], vectors[..., 2]
    one = x * 0 + 1
    out = [one]
    if lmax >= 1:
        s = math.sqrt(3.0)
        out += [s * y, s * z, s * x]
    if lmax >= 2:
        s5, s15 = math.sqrt(5.0), math.sqrt(15.0)
        out += [s15 * x * y, s15 * y * z, 0.5 * s5 * (3 * z * z - 1), s15 * x * z, 0.5 * s15 * (x * x - y * y)]
    if lmax >= 3:
        s7 = math.sqrt(7.0)
        a, b, c = math.sqrt(5.0 / 8.0), math.sqrt(15.0), math.sqrt(3.0 / 8.0)
        out += [s7 * a * y * (3 * x * x - y * y), s7 * b * x * y * z, s7 * c * y * (5 * z * z - 1),
                s7 * 0.5 * z * (5 * z * z - 3), s7 * c * x * (5 * z * z - 1), s7 * 0.5 * b * z * (x * x - y * y),
                s7 * a * x * (x * x - 3 * y * y)]
    if isinstance(x, np.ndarray):
        return np.stack(out, axis=-1)
    import torch
    return torch.stack(out, dim=-1)


def receiver_shards(rows: np.ndarray, nodes: int, world: int):
    """Node range and edge slice of every rank when receivers are split evenly.

    Returns ``[(node_lo, node_hi, edge_lo, edge_hi), ...]``; ``rows`` must be sorted.
    """
    out = []
    for rank in range(world):
        lo, hi = nodes * rank // world, nodes * (rank + 1) // world
        e_lo, e_hi = np.searchsorted(rows, lo, side="left"), np.searchsorted(rows, hi, side="left")
        out.append((lo, hi, int(e_lo), int(e_hi)))
    return out
