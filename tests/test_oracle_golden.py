"""The CPU oracle vs outputs of the reference's own CPU code (tests/golden)."""
import numpy as np
import pytest
import torch

from oracle import tp_oracle as orc
from conftest import load_golden, problem_by_name, golden_problems, build_problem


@pytest.mark.parametrize("name", ["nequip_32", "cw_mixed", "mace_128", "mace_large_128"])
def test_forward_matches_reference_numpy(name):
    g = load_golden("numpy_tp_forward.npz")
    p = problem_by_name(name)
    x, y, w, ref = (g[f"{name}__{k}"] for k in ("in1", "in2", "w", "out"))
    got = orc.tp_forward(p, x, y, w)
    # reference ran its einsum on float32 data; ours runs in float64
    np.testing.assert_allclose(got, ref, rtol=2e-5, atol=2e-5)
    rel = np.abs(got - ref).max() / np.abs(ref).max()
    assert rel < 5e-6


def test_readme_shape_known_answer():
    g = load_golden("numpy_tp_forward.npz")
    p = problem_by_name("readme")
    rng = np.random.default_rng(12345)      # draw order of the reference: in1, in2, weights
    x = rng.uniform(size=(1000, 5)).astype(np.float32)
    y = rng.uniform(size=(1000, 7)).astype(np.float32)
    w = rng.uniform(size=(1000, 1)).astype(np.float32)
    z = orc.tp_forward(p, x, y, w)
    assert np.linalg.norm(z) == pytest.approx(float(g["readme__norm"][0]), rel=1e-6)
    np.testing.assert_allclose(z[:4], g["readme__head"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(z[::50], g["readme__out_every_50"], rtol=1e-5, atol=1e-6)
    assert p.instructions[0].path_weight == pytest.approx(np.sqrt(5.0))


@pytest.mark.parametrize("entry", golden_problems(), ids=lambda e: e["name"])
def test_loop_permutation_matches_reference(entry):
    p = build_problem(entry)
    assert np.array_equal(orc.oeq_from_e3nn_index(p), load_golden("weight_perm.npz")[entry["name"]])
    w = np.random.default_rng(1).normal(size=(2, p.weight_numel))
    assert np.array_equal(orc.oeq_to_e3nn(p, orc.e3nn_to_oeq(p, w)), w)


def test_coord_graph_matches_reference():
    g = load_golden("coord_graph.npz")
    rows, cols, order, perm = orc.coord_graph(g["rows_in"], g["cols_in"])
    assert np.array_equal(rows, g["rows"]) and np.array_equal(cols, g["cols"])
    assert np.array_equal(perm, g["transpose_perm"])
    # the permutation visits the sorted list in (sender, receiver) order
    assert np.all(np.diff(cols[perm]) >= 0)


def test_scatter_sum_matches_reference():
    g = load_golden("scatter_sum.npz")
    out = orc.scatter_sum_rows(torch.as_tensor(g["src"]), torch.as_tensor(g["index"]), g["out"].shape[0])
    np.testing.assert_allclose(out.numpy(), g["out"], rtol=0, atol=1e-14)


def test_conv_is_gather_tp_scatter():
    p = problem_by_name("cw_mixed")
    rng = np.random.default_rng(3)
    n, e = 7, 40
    rows, cols = rng.integers(0, n, e), rng.integers(0, n, e)
    x = rng.normal(size=(n, p.irreps_in1.dim))
    y = rng.normal(size=(e, p.irreps_in2.dim))
    w = rng.normal(size=(e, p.weight_numel))
    z = orc.conv_forward(p, x, y, w, rows, cols)
    msg = orc.tp_forward(p, x[cols], y, w)
    ref = np.zeros_like(z)
    np.add.at(ref, rows, msg)
    np.testing.assert_allclose(z, ref, atol=1e-12)


@pytest.mark.parametrize("name", ["uvw_small", "uvu_v2", "uvu_shared", "uvw_rowweights"])
def test_backward_is_consistent_with_finite_differences(name):
    p = problem_by_name(name)
    rng = np.random.default_rng(5)
    b = 3
    x = rng.normal(size=(b, p.irreps_in1.dim))
    y = rng.normal(size=(b, p.irreps_in2.dim))
    w = rng.normal(size=(p.weight_numel,) if p.shared_weights else (b, p.weight_numel))
    dz = rng.normal(size=(b, p.irreps_out.dim))
    dx, dy, dw = orc.tp_backward(p, x, y, w, dz)
    eps = 1e-6
    for arr, grad in ((x, dx), (y, dy), (w, dw)):
        idx = tuple(rng.integers(0, s) for s in arr.shape)
        plus, minus = arr.copy(), arr.copy()
        plus[idx] += eps
        minus[idx] -= eps
        args_p = [plus if a is arr else a for a in (x, y, w)]
        args_m = [minus if a is arr else a for a in (x, y, w)]
        fd = ((orc.tp_forward(p, *args_p) - orc.tp_forward(p, *args_m)) * dz).sum() / (2 * eps)
        assert grad[idx] == pytest.approx(fd, rel=1e-6, abs=1e-8)


def test_e3nn_style_pairing_is_the_same_function():
    p = problem_by_name("uvw_small")
    rng = np.random.default_rng(6)
    x = torch.as_tensor(rng.normal(size=(4, p.irreps_in1.dim)))
    y = torch.as_tensor(rng.normal(size=(4, p.irreps_in2.dim)))
    w = torch.as_tensor(rng.normal(size=(p.weight_numel,)))
    a = orc.tp_torch(p, x, y, w)
    b = orc.tp_torch(p, x, y, w, e3nn_style_pairs=True)
    np.testing.assert_allclose(a.numpy(), b.numpy(), atol=1e-12)


def test_folded_contraction_order_is_the_same_function():
    p = problem_by_name("cw_mixed")
    rng = np.random.default_rng(16)
    x = torch.as_tensor(rng.normal(size=(6, p.irreps_in1.dim)))
    y = torch.as_tensor(rng.normal(size=(6, p.irreps_in2.dim)))
    w = torch.as_tensor(rng.normal(size=(6, p.weight_numel)))
    a = orc.tp_torch(p, x, y, w)
    b = orc.tp_torch(p, x, y, w, fold_second_input=True)
    np.testing.assert_allclose(a.numpy(), b.numpy(), atol=1e-12)
