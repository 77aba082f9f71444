"""The CPU oracle vs outputs of the reference's own CPU code (tests/golden)."""
import numpy as np
import pytest
import torch

from oracle import tp_oracle as orc
from conftest import load_golden, problem_by_name, golden_problems, build_problem


@pytest.mark.parametrize("name", ["nequip_32", "cw_mixed", "mace_128", "mace_large_128", "roofline_5e_3e",
                                  "roofline_6e", "roofline_7e_7e"])
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


# --------------------------------------------------------------------------- closed forms for "uvw"
#
# The reference's stored CPU code covers "uvu" only, so the dense "uvw" contraction and shared weights are
# pinned here by answers that can be written down: the Wigner 3j tensors of l <= 1 are, up to sign, the
# identity / sqrt(2l+1), the dot product / sqrt(3) and the cross product / sqrt(6), and a "uvw" path is
# Z[b, w, k] = path_weight * sum_{u,v} W[u, v, w] * sum_ij C_ijk x[b, u, i] y[b, v, j].

def _uvw_problem(in1, in2, out, instr, shared=True):
    import openequivariance_b200 as oeq
    return oeq.TPProblem(in1, in2, out, instr, shared_weights=shared, internal_weights=False,
                         irrep_dtype=np.float64, weight_dtype=np.float64)


def _closed_form_cases():
    rng = np.random.default_rng(77)
    b, nu, nv, nw = 5, 3, 2, 4
    cases = []
    # scalar x vector -> vector: C_{0jk} = delta_jk / sqrt(3)
    x, y = rng.normal(size=(b, nu, 1)), rng.normal(size=(b, nv, 3))
    w = rng.normal(size=(nu, nv, nw))
    p = _uvw_problem(f"{nu}x0e", f"{nv}x1o", f"{nw}x1o", [(0, 0, 0, "uvw", True)])
    want = np.einsum("uvw,bu,bvk->bwk", w, x[:, :, 0], y) / np.sqrt(3.0)
    cases.append(("scalar_times_vector", p, x, y, w, want))
    # vector . vector -> scalar: C_{ij0} = delta_ij / sqrt(3)
    x, y = rng.normal(size=(b, nu, 3)), rng.normal(size=(b, nv, 3))
    p = _uvw_problem(f"{nu}x1o", f"{nv}x1o", f"{nw}x0e", [(0, 0, 0, "uvw", True)])
    want = np.einsum("uvw,bui,bvi->bw", w, x, y)[:, :, None] / np.sqrt(3.0)
    cases.append(("dot_product", p, x, y, w, want))
    # vector x vector -> axial vector: C_ijk = eps_ijk / sqrt(6) (the sign is fixed by the stored tensor)
    p = _uvw_problem(f"{nu}x1o", f"{nv}x1o", f"{nw}x1e", [(0, 0, 0, "uvw", True)])
    eps = np.zeros((3, 3, 3))
    for i, j, k in ((0, 1, 2), (1, 2, 0), (2, 0, 1)):
        eps[i, j, k], eps[j, i, k] = 1.0, -1.0
    sign = np.sign(orc.cg(1, 1, 1)[0, 1, 2])
    want = sign * np.einsum("uvw,ijk,bui,bvj->bwk", w, eps, x, y) / np.sqrt(6.0)
    cases.append(("cross_product", p, x, y, w, want))
    return cases


@pytest.mark.parametrize("index", [0, 1, 2], ids=["scalar_times_vector", "dot_product", "cross_product"])
def test_uvw_closed_forms_forward_and_weight_gradient(index):
    name, p, x, y, w, want = _closed_form_cases()[index]
    pw = p.instructions[0].path_weight
    b = x.shape[0]
    xf, yf, wf = x.reshape(b, -1), y.reshape(b, -1), w.reshape(-1)
    got = orc.tp_forward(p, xf, yf, wf).reshape(want.shape)
    np.testing.assert_allclose(got, pw * want, rtol=1e-12, atol=1e-13)
    # the path weight itself: "component" irrep normalisation, "element" path normalisation, one path:
    # alpha = (2 l_out + 1) / (mul_in1 * mul_in2)
    mul1, mul2 = p.irreps_in1[0].mul, p.irreps_in2[0].mul
    assert pw == pytest.approx(np.sqrt(p.irreps_out[0].ir.dim / (mul1 * mul2)), rel=1e-14)
    # weight gradient: Z is linear in W, so dW[u,v,w] = d/dW <dZ, Z> has the same closed form with dZ inserted
    rng = np.random.default_rng(78)
    dz = rng.normal(size=want.shape)
    _, _, dw = orc.tp_backward(p, xf, yf, wf, dz.reshape(b, -1))
    if name == "scalar_times_vector":
        ref = np.einsum("bwk,bu,bvk->uvw", dz, x[:, :, 0], y) / np.sqrt(3.0)
    elif name == "dot_product":
        ref = np.einsum("bw,bui,bvi->uvw", dz[:, :, 0], x, y) / np.sqrt(3.0)
    else:
        eps = np.zeros((3, 3, 3))
        for i, j, k in ((0, 1, 2), (1, 2, 0), (2, 0, 1)):
            eps[i, j, k], eps[j, i, k] = 1.0, -1.0
        ref = np.sign(orc.cg(1, 1, 1)[0, 1, 2]) * np.einsum("bwk,ijk,bui,bvj->uvw", dz, eps, x, y) / np.sqrt(6.0)
    np.testing.assert_allclose(dw.reshape(ref.shape), pw * ref, rtol=1e-12, atol=1e-13)


def test_uvw_per_row_weights_are_the_same_contraction_row_by_row():
    """Per-row weights: row b of the result equals the shared-weight result with W = W[b]."""
    p_rows = problem_by_name("diffdock_l1", irrep_dtype=np.float64, weight_dtype=np.float64)
    import openequivariance_b200 as oeq
    p_shared = oeq.FullyConnectedTPProblem(str(p_rows.irreps_in1), str(p_rows.irreps_in2), str(p_rows.irreps_out),
                                           irrep_dtype=np.float64, weight_dtype=np.float64)
    assert not p_rows.shared_weights and p_shared.shared_weights
    rng = np.random.default_rng(79)
    x = rng.normal(size=(3, p_rows.irreps_in1.dim))
    y = rng.normal(size=(3, p_rows.irreps_in2.dim))
    w = rng.normal(size=(3, p_rows.weight_numel))
    z = orc.tp_forward(p_rows, x, y, w)
    for b in range(3):
        np.testing.assert_allclose(z[b], orc.tp_forward(p_shared, x[b:b + 1], y[b:b + 1], w[b])[0], atol=1e-12)
