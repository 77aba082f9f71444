"""Problem description, Clebsch-Gordan generator and weight layout vs the
reference's own outputs (tests/golden, produced by make_golden.py)."""
import numpy as np
import pytest

import openequivariance_b200 as oeq
from openequivariance_b200 import weights as wl
from openequivariance_b200.wigner import cg_nonzeros
from conftest import load_golden, golden_problems, build_problem


def test_wigner_3j_matches_reference_generator():
    data = load_golden("wigner_3j.npz")
    assert len(data.files) > 60
    for key in data.files:
        l1, l2, l3 = map(int, key.split("_"))
        ours = oeq.wigner_3j(l1, l2, l3)
        ref = data[key]
        assert ours.shape == ref.shape
        # same formula in float64: agree to round-off, zeros in the same places
        np.testing.assert_allclose(ours, ref, rtol=0, atol=1e-14)
        assert abs(np.sum(ours ** 2) - 1.0) < 1e-13
        nz = cg_nonzeros(l1, l2, l3)
        assert len(nz) == np.count_nonzero(np.abs(ref) > 1e-12)


def test_cg_nonzero_counts_of_known_triples():
    expect = {(1, 1, 0): 3, (1, 1, 1): 6, (1, 2, 1): 11, (2, 2, 2): 25, (2, 3, 3): 41, (3, 3, 2): 41}
    for triple, n in expect.items():
        assert len(cg_nonzeros(*triple)) == n


def test_closed_forms_dot_and_cross():
    # 1o x 1o -> 0e is the dot product / sqrt(3); 1o x 1o -> 1e is the cross product / sqrt(6)
    c0 = oeq.wigner_3j(1, 1, 0)[:, :, 0]
    np.testing.assert_allclose(np.abs(c0), np.eye(3) / np.sqrt(3), atol=1e-14)
    c1 = oeq.wigner_3j(1, 1, 1)
    x, y = np.array([0.3, -1.2, 0.7]), np.array([1.1, 0.4, -0.5])
    got = np.einsum("ijk,i,j->k", c1, x, y)
    np.testing.assert_allclose(np.abs(got), np.abs(np.cross(x, y)) / np.sqrt(6), atol=1e-14)


@pytest.mark.parametrize("entry", golden_problems(), ids=lambda e: e["name"])
def test_problem_matches_reference(entry):
    p = build_problem(entry)
    assert str(p.irreps_in1) == entry["irreps_in1"]
    assert str(p.irreps_in2) == entry["irreps_in2"]
    assert str(p.irreps_out) == entry["irreps_out"]
    assert (p.irreps_in1.dim, p.irreps_in2.dim, p.irreps_out.dim) == (
        entry["in1_dim"], entry["in2_dim"], entry["out_dim"])
    assert p.weight_numel == entry["weight_numel"]
    assert p.shared_weights == entry["shared_weights"]
    assert p.internal_weights == entry["internal_weights"]
    assert len(p.instructions) == len(entry["instructions"])
    for ours, ref in zip(p.instructions, entry["instructions"]):
        assert [ours.i_in1, ours.i_in2, ours.i_out, ours.connection_mode, ours.has_weight] == ref[:5]
        assert ours.path_weight == pytest.approx(ref[5], rel=1e-15)
        assert list(ours.path_shape) == ref[6]


@pytest.mark.parametrize("entry", golden_problems(), ids=lambda e: e["name"])
def test_weight_permutation_matches_reference(entry):
    p = build_problem(entry)
    ref = load_golden("weight_perm.npz")[entry["name"]]
    ours = wl.oeq_from_e3nn_index(p)
    assert np.array_equal(ours, ref)
    # round trip through the public reorder entry point, with and without a batch axis
    src = np.random.default_rng(0).normal(size=(3, p.weight_numel))
    dst = np.zeros_like(src)
    wl.reorder_weights(p, src, dst, "forward", True)
    assert np.array_equal(dst, src[:, ref])
    back = np.zeros_like(src)
    wl.reorder_weights(p, dst, back, "backward", True)
    assert np.array_equal(back, src)
    one = np.zeros(p.weight_numel)
    wl.reorder_weights(p, src[0], one, "forward", False)
    assert np.array_equal(one, src[0, ref])


def test_uvu_unit_second_multiplicity_is_identity_layout():
    for name in ("mace_128", "nequip_32", "mace_large_128", "readme"):
        p = build_problem(next(e for e in golden_problems() if e["name"] == name))
        assert np.array_equal(wl.oeq_from_e3nn_index(p), np.arange(p.weight_numel))


def test_irreps_behaviour():
    ir = oeq.Irreps("2x0e + 1e")
    assert [s.start for s in ir.slices()] == [0, 2] and ir.dim == 5
    assert str(oeq.Irreps("0e+1o+2e")) == "1x0e+1x1o+1x2e"
    assert str((oeq.Irreps("2x1e") * 3).simplify()) == "6x1e"
    assert str(oeq.Irreps([(3, (1, -1)), (2, "0e")])) == "3x1o+2x0e"
    assert str(oeq.Irreps.spherical_harmonics(2)) == "1x0e+1x1o+1x2e"
    s = oeq.Irreps("1x2e+3x0e+2x1o").sort()
    assert str(s.irreps) == "3x0e+2x1o+1x2e" and s.inv == (1, 2, 0) and s.p == (2, 0, 1)
    assert [str(i) for i in oeq.Irrep("1o") * oeq.Irrep("2e")] == ["1o", "2o", "3o"]
    with pytest.raises(ValueError):
        oeq.Irrep("1x")
    with pytest.raises(ValueError):
        oeq.Irreps("3y0e")


def test_problem_rejects_bad_paths():
    with pytest.raises(AssertionError):
        oeq.TPProblem("1x1o", "1x1o", "1x1o", [(0, 0, 0, "uvu", True)])  # parity
    with pytest.raises(AssertionError):
        oeq.TPProblem("1x1o", "1x1o", "1x3e", [(0, 0, 0, "uvu", True)])  # triangle
