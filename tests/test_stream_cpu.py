"""Slab streaming of the convolution over host tensors: the slab plan and the slab sequence, on CPU.

The local kernel is replaced by the CPU oracle so that only the host-side logic is under test; the
streamed CUDA path is covered by the gpu-marked tests."""
import numpy as np
import pytest
import torch

from oracle import tp_oracle as orc
from conftest import problem_by_name
from helpers import conv_inputs, random_graph, rel_err
from openequivariance_b200.stream import StreamedTensorProductConv, plan_slabs
from test_dist_cpu import OracleLocalConv


@pytest.mark.parametrize("slab_edges", [1, 7, 64, 10_000])
def test_slabs_partition_edges_and_receivers(slab_edges):
    nodes = 41
    rows, cols = random_graph(nodes, 350, seed=5)
    rows, cols, _, _ = orc.coord_graph(rows, cols)
    slabs = plan_slabs(rows, cols, nodes, slab_edges)
    assert slabs[0].e0 == 0 and slabs[-1].e1 == len(rows)
    assert slabs[0].r0 == 0 and slabs[-1].r1 == nodes
    for a, b in zip(slabs, slabs[1:]):
        assert a.e1 == b.e0 and a.r1 == b.r0
        assert rows[a.e1 - 1] != rows[b.e0]                # cuts fall on receiver boundaries
    for s in slabs:
        assert s.edges >= 1
        assert np.array_equal(s.rows + s.r0, rows[s.e0:s.e1]) and np.array_equal(s.cols, cols[s.e0:s.e1])
        assert np.all((s.rows >= 0) & (s.rows < s.receivers))
        # perm visits the slab's edges by (sender, receiver)
        keys = list(zip(s.cols[s.perm].tolist(), s.rows[s.perm].tolist()))
        assert keys == sorted(keys)
        if slab_edges >= 7:
            assert s is slabs[-1] or s.edges >= slab_edges


def test_slab_plan_edge_cases():
    one = plan_slabs(np.zeros(0, np.int64), np.zeros(0, np.int64), 5, 16)
    assert len(one) == 1 and one[0].edges == 0 and (one[0].r0, one[0].r1) == (0, 5)
    with pytest.raises(ValueError):
        plan_slabs(np.array([1, 0]), np.array([0, 0]), 2, 4)
    with pytest.raises(ValueError):
        plan_slabs(np.array([0, 1]), np.array([0]), 2, 4)
    with pytest.raises(ValueError):
        plan_slabs(np.array([0, 1]), np.array([0, 0]), 2, 0)


@pytest.mark.parametrize("lazy", [False, True])
def test_streamed_matches_whole_graph(lazy):
    p = problem_by_name("cw_mixed", irrep_dtype=np.float64, weight_dtype=np.float64)
    nodes = 23
    rows, cols = random_graph(nodes, 160, seed=9)
    rows, cols, _, _ = orc.coord_graph(rows, cols)
    x, y, w, dz = (torch.from_numpy(a) for a in conv_inputs(p, nodes, len(rows), 4))
    ref = OracleLocalConv(p)
    r, c = torch.from_numpy(rows), torch.from_numpy(cols)
    z_ref = ref._forward_impl(x, y, w, r, c, n_out=nodes)
    dx_ref, dy_ref, dw_ref = ref._backward_impl(x, y, w, dz, r, c)

    conv = StreamedTensorProductConv(p, rows, cols, nodes, slab_edges=37, device="cpu", local_conv=ref)
    assert len(conv.slabs) > 2
    z, dx, dy, dw = torch.empty_like(z_ref), torch.empty_like(x), torch.empty_like(y), torch.empty_like(w)
    calls = []
    if lazy:      # edge arrays handed over slab by slab
        view = lambda t: (lambda i, lo, hi: (calls.append((i, lo, hi)), t[lo:hi])[1])
        conv.forward_backward_host(x, view(y), view(w), dz, z, dx, view(dy), view(dw))
        assert {c_[0] for c_ in calls} == set(range(len(conv.slabs)))
    else:
        conv.forward_backward_host(x, y, w, dz, z, dx, dy, dw)
    for got, want in ((z, z_ref), (dx, dx_ref), (dy, dy_ref), (dw, dw_ref)):
        assert rel_err(got.numpy(), want.numpy()) < 1e-12
    elem = 8
    assert conv.h2d_bytes(elem) == (x.numel() + dz.numel() + y.numel() + w.numel()) * elem + 24 * len(rows)
    assert conv.d2h_bytes(elem) == (z.numel() + dx.numel() + dy.numel() + dw.numel()) * elem
