"""Shared helpers of the GPU parity tests: seeded inputs, error norms, graphs."""
import numpy as np

from oracle import tp_oracle as orc

# Tolerances of the parity tests: max-norm error relative to the max norm of the oracle's
# result, oracle evaluated in float64 on the same (float32- or float64-valued) inputs.
REL_TOL = {np.float32: 1e-5, np.float64: 1e-12}


def rel_err(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if want.size == 0:
        return 0.0
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def tp_inputs(problem, batch, seed, dist="normal"):
    """X, Y, W (e3nn order), dZ as numpy arrays of the problem's dtype."""
    rng = np.random.default_rng(seed)
    dt = problem.irrep_dtype
    draw = (lambda s: rng.normal(size=s)) if dist == "normal" else (lambda s: rng.uniform(size=s))
    x = draw((batch, problem.irreps_in1.dim)).astype(dt)
    y = draw((batch, problem.irreps_in2.dim)).astype(dt)
    wshape = (problem.weight_numel,) if problem.shared_weights else (batch, problem.weight_numel)
    w = draw(wshape).astype(dt)
    dz = draw((batch, problem.irreps_out.dim)).astype(dt)
    return x, y, w, dz


def random_graph(nodes, edges, seed, symmetric=False):
    rng = np.random.default_rng(seed)
    rows = rng.integers(0, nodes, size=edges).astype(np.int64)
    cols = rng.integers(0, nodes, size=edges).astype(np.int64)
    if symmetric:
        rows, cols = np.concatenate([rows, cols]), np.concatenate([cols, rows])
    return rows, cols


def conv_inputs(problem, nodes, edges, seed):
    rng = np.random.default_rng(seed)
    dt = problem.irrep_dtype
    x = rng.normal(size=(nodes, problem.irreps_in1.dim)).astype(dt)
    y = rng.normal(size=(edges, problem.irreps_in2.dim)).astype(dt)
    w = rng.normal(size=(edges, problem.weight_numel)).astype(dt)
    dz = rng.normal(size=(nodes, problem.irreps_out.dim)).astype(dt)
    return x, y, w, dz


def to_oeq(problem, w):
    return orc.e3nn_to_oeq(problem, w)


def to_e3nn(problem, w):
    return orc.oeq_to_e3nn(problem, w)
