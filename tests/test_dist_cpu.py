"""Receiver-sharded convolution: partition logic and the two exchange steps, on CPU ranks (gloo).

The local kernel is replaced by the CPU oracle so that only the host-side plan and the
collectives are under test; the GPU kernels are covered by the gpu-marked tests."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import tp_oracle as orc
from conftest import problem_by_name
from helpers import conv_inputs, random_graph, rel_err
from openequivariance_b200.dist import ShardPlan, ShardedTensorProductConv


class OracleLocalConv:
    """Stand-in with the two methods the sharded layer calls on its local convolution."""

    def __init__(self, problem):
        self.problem = problem

    def _forward_impl(self, x, y, w, rows, cols, perm=None, n_out=None):
        msg = orc.tp_torch(self.problem, x[cols], y, w)
        return torch.zeros(n_out, msg.shape[1], dtype=x.dtype).index_add(0, rows, msg)

    def _backward_impl(self, x, y, w, dz, rows, cols, perm=None):
        with torch.enable_grad():    # called from inside autograd's backward, where grad mode is off
            x, y, w = (t.detach().clone().requires_grad_(True) for t in (x, y, w))
            z = self._forward_impl(x, y, w, rows, cols, n_out=dz.shape[0])
            z.backward(dz)
        return x.grad, y.grad, w.grad


def test_plan_partitions_nodes_and_edges():
    rows, cols = random_graph(37, 400, seed=1)
    rows, cols, _, _ = orc.coord_graph(rows, cols)
    for world in (1, 2, 3, 8):
        plans = ShardPlan.build_all(rows, cols, 37, world)
        assert plans[0].node_lo == 0 and plans[-1].node_hi == 37
        assert sum(p.owned for p in plans) == 37
        assert plans[0].edge_lo == 0 and plans[-1].edge_hi == len(rows)
        for a, b in zip(plans, plans[1:]):
            assert a.node_hi == b.node_lo and a.edge_hi == b.edge_lo
        for p in plans:
            assert np.all((p.local_rows >= 0) & (p.local_rows < max(p.owned, 1)))
            assert np.all(np.diff(p.local_cols[p.local_perm]) >= 0)      # sender order
            # the compact sender numbering maps back to the global ids: owned rows first, then the halo
            to_global = np.concatenate([np.arange(p.node_lo, p.node_hi), p.halo])
            assert np.array_equal(to_global[p.local_cols], cols[p.edge_lo:p.edge_hi])
            assert np.all((p.halo < p.node_lo) | (p.halo >= p.node_hi)) and np.all(np.diff(p.halo) > 0)
            assert sum(p.recv_counts) == p.halo.size and p.recv_counts[p.rank] == 0
        # what rank a sends to rank b is exactly what b expects from a, in b's halo order
        for a in plans:
            for b in plans:
                assert len(a.send_rows[b.rank]) == b.recv_counts[a.rank]
                if a.rank != b.rank:
                    first = sum(b.recv_counts[:a.rank])
                    assert np.array_equal(a.send_rows[b.rank] + a.node_lo,
                                          b.halo[first:first + b.recv_counts[a.rank]])
        # a rank can build its own plan (with its send lists) without building its peers'
        for p in plans:
            one = ShardPlan.build_one(rows, cols, 37, p.rank, world)
            assert np.array_equal(one.halo, p.halo) and np.array_equal(one.local_cols, p.local_cols)
            assert np.array_equal(one.local_perm, p.local_perm) and one.recv_counts == p.recv_counts
            assert len(one.send_rows) == world
            for a, b in zip(one.send_rows, p.send_rows):
                assert np.array_equal(a, b)
    with pytest.raises(ValueError):
        ShardPlan(rows[::-1], cols, 37, 0, 2)
    with pytest.raises(ValueError):
        ShardPlan(rows, cols, 37, 2, 2)


def _worker(rank, world, port, nodes, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        p = problem_by_name("cw_mixed", irrep_dtype=np.float64, weight_dtype=np.float64)
        rows, cols = random_graph(nodes, 300, seed=2)
        rows, cols, order, _ = orc.coord_graph(rows, cols)
        x, y, w, dz = conv_inputs(p, nodes, len(rows), 3)
        conv = ShardedTensorProductConv(p, rows, cols, nodes, device="cpu", local_conv=OracleLocalConv(p))
        plan = conv.plan
        xs = torch.from_numpy(x[plan.node_lo:plan.node_hi]).requires_grad_(True)
        ys = torch.from_numpy(y[plan.edge_lo:plan.edge_hi]).requires_grad_(True)
        ws = torch.from_numpy(w[plan.edge_lo:plan.edge_hi]).requires_grad_(True)
        dzs = torch.from_numpy(dz[plan.node_lo:plan.node_hi])
        z = conv(xs, ys, ws)
        z.backward(dzs)
        z_ref = orc.conv_forward(p, x, y, w, rows, cols)
        rx, ry, rw = orc.conv_backward(p, x, y, w, dz, rows, cols)
        errs = [rel_err(z.detach().numpy(), z_ref[plan.node_lo:plan.node_hi]),
                rel_err(xs.grad.numpy(), rx[plan.node_lo:plan.node_hi]),
                rel_err(ys.grad.numpy(), ry[plan.edge_lo:plan.edge_hi]),
                rel_err(ws.grad.numpy(), rw[plan.edge_lo:plan.edge_hi])]
        z2, dx2, dy2, dw2 = conv.forward_backward(xs.detach(), ys.detach(), ws.detach(), dzs)
        errs.append(rel_err(dx2.numpy(), rx[plan.node_lo:plan.node_hi]))
        # two forward passes on the same module before either backward pass (gradient accumulation, a layer
        # applied twice): the second gather must not overwrite what the first saved
        xa = torch.from_numpy(x[plan.node_lo:plan.node_hi]).requires_grad_(True)
        xb = torch.from_numpy(2.0 * x[plan.node_lo:plan.node_hi]).requires_grad_(True)
        za, zb = conv(xa, ys.detach(), ws.detach()), conv(xb, ys.detach(), ws.detach())
        za.backward(dzs)
        zb.backward(dzs)
        errs.append(rel_err(xa.grad.numpy(), rx[plan.node_lo:plan.node_hi]))
        errs.append(rel_err(xb.grad.numpy(), rx[plan.node_lo:plan.node_hi]))     # dX does not depend on X
        errs.append(rel_err(zb.detach().numpy(), 2.0 * z_ref[plan.node_lo:plan.node_hi]))
        result[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("nodes", [40, 41])          # even split and a padded last shard
def test_two_rank_conv_matches_the_single_process_oracle(nodes):
    world = 2
    port = 29600 + nodes
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, nodes, result)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=240)
        assert pr.exitcode == 0
    assert len(result) == world and max(result.values()) < 1e-12


def _host_worker(rank, world, port, nodes, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        p = problem_by_name("cw_mixed", irrep_dtype=np.float64, weight_dtype=np.float64)
        rows, cols = random_graph(nodes, 300, seed=4)
        rows, cols, order, _ = orc.coord_graph(rows, cols)
        x, y, w, dz = conv_inputs(p, nodes, len(rows), 5)
        conv = ShardedTensorProductConv(p, rows, cols, nodes, device="cpu", local_conv=OracleLocalConv(p))
        plan = conv.plan
        n_lo, n_hi, e_lo, e_hi = plan.node_lo, plan.node_hi, plan.edge_lo, plan.edge_hi
        xs, dzs = torch.from_numpy(x[n_lo:n_hi]), torch.from_numpy(dz[n_lo:n_hi])
        ys, ws = torch.from_numpy(y[e_lo:e_hi]), torch.from_numpy(w[e_lo:e_hi])
        z_h = torch.zeros(plan.owned, p.irreps_out.dim, dtype=torch.float64)
        dx_h, dy_h, dw_h = torch.zeros_like(xs), torch.zeros_like(ys), torch.zeros_like(ws)
        # several slabs per rank; the weights are handed over lazily, slab by slab
        conv.forward_backward_host(xs, ys, lambda i, lo, hi: ws[lo:hi], dzs, z_h, dx_h, dy_h, dw_h, slab_edges=40)
        assert len(conv.slab_plan(40).slabs) > 1
        z_ref = orc.conv_forward(p, x, y, w, rows, cols)
        rx, ry, rw = orc.conv_backward(p, x, y, w, dz, rows, cols)
        result[rank] = max(rel_err(z_h.numpy(), z_ref[n_lo:n_hi]), rel_err(dx_h.numpy(), rx[n_lo:n_hi]),
                           rel_err(dy_h.numpy(), ry[e_lo:e_hi]), rel_err(dw_h.numpy(), rw[e_lo:e_hi]))
        h2d, d2h = conv.host_bytes(8)
        assert h2d - d2h == 24 * (e_hi - e_lo)
    finally:
        dist.destroy_process_group()


def test_two_rank_host_tensor_step_streams_slabs_and_matches_the_oracle():
    world, nodes = 2, 41
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    procs = [ctx.Process(target=_host_worker, args=(r, world, 29671, nodes, result)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=240)
        assert pr.exitcode == 0
    assert len(result) == world and max(result.values()) < 1e-12


# ---------------------------------------------------------------------------------------------------
# batch tensor product sharded by rows


class OracleLocalTP:
    """Stand-in with the two methods the row-sharded layer calls on its local tensor product."""

    def __init__(self, problem):
        self.problem = problem

    def _forward_impl(self, x, y, w):
        return orc.tp_torch(self.problem, x, y, w)

    def _backward_impl(self, x, y, w, dz):
        with torch.enable_grad():
            x, y, w = (t.detach().clone().requires_grad_(True) for t in (x, y, w))
            self._forward_impl(x, y, w).backward(dz)
        return x.grad, y.grad, w.grad


def test_row_ranges_partition_the_batch():
    from openequivariance_b200.dist import row_range
    for batch in (0, 1, 7, 64, 1000):
        for world in (1, 2, 3, 8):
            ranges = [row_range(batch, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            assert all(lo <= hi for lo, hi in ranges)
    with pytest.raises(ValueError):
        row_range(10, 2, 2)


def _tp_worker(rank, world, port, batch, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from helpers import tp_inputs
        from openequivariance_b200.dist import ShardedTensorProduct, row_range
        out = {}
        for name in ("uvw_small", "cw_mixed"):       # shared weights (all-reduce of dW) and per-row weights
            p = problem_by_name(name, irrep_dtype=np.float64, weight_dtype=np.float64)
            x, y, w, dz = (torch.from_numpy(a) for a in tp_inputs(p, batch, 5))
            lo, hi = row_range(batch, rank, world)
            tp = ShardedTensorProduct(p, local_tp=OracleLocalTP(p))
            xs, ys = x[lo:hi].clone().requires_grad_(True), y[lo:hi].clone().requires_grad_(True)
            ws = (w if p.shared_weights else w[lo:hi]).clone().requires_grad_(True)
            z = tp(xs, ys, ws)
            z.backward(dz[lo:hi])
            out[name] = (lo, hi, z.detach(), xs.grad, ys.grad, ws.grad)
        result[rank] = out
    finally:
        dist.destroy_process_group()


def test_row_sharded_tensor_product_two_ranks():
    from helpers import tp_inputs
    batch, world = 37, 2
    with mp.Manager() as manager:
        result = manager.dict()
        mp.spawn(_tp_worker, args=(world, 29533, batch, result), nprocs=world, join=True)
        got = dict(result)
    for name in ("uvw_small", "cw_mixed"):
        p = problem_by_name(name, irrep_dtype=np.float64, weight_dtype=np.float64)
        x, y, w, dz = (torch.from_numpy(a) for a in tp_inputs(p, batch, 5))
        ref = OracleLocalTP(p)
        z_ref = ref._forward_impl(x, y, w)
        dx_ref, dy_ref, dw_ref = ref._backward_impl(x, y, w, dz)
        for rank in range(world):
            lo, hi, z, dx, dy, dw = got[rank][name]
            assert rel_err(z.numpy(), z_ref[lo:hi].numpy()) < 1e-12
            assert rel_err(dx.numpy(), dx_ref[lo:hi].numpy()) < 1e-12
            assert rel_err(dy.numpy(), dy_ref[lo:hi].numpy()) < 1e-12
            want = dw_ref if p.shared_weights else dw_ref[lo:hi]
            assert rel_err(dw.numpy(), want.numpy()) < 1e-12       # every rank holds the full sum of a shared gradient



def test_bind_host_to_device_node(tmp_path):
    """The helper that keeps a streaming process on the GPU's NUMA node, against a made-up sysfs tree."""
    import os
    from openequivariance_b200.stream import bind_host_to_device_node, _parse_cpulist
    assert _parse_cpulist("0-2,5,8-9\n") == {0, 1, 2, 5, 8, 9}
    before = os.sched_getaffinity(0)
    first = min(before)
    bus = "0000:66:00.0"
    dev = tmp_path / "bus" / "pci" / "devices" / bus
    dev.mkdir(parents=True)
    node = tmp_path / "devices" / "system" / "node" / "node1"
    node.mkdir(parents=True)
    try:
        (dev / "numa_node").write_text("-1\n")
        assert bind_host_to_device_node(0, sysfs=str(tmp_path), bus_id=bus) is None      # single-node machine
        (dev / "numa_node").write_text("1\n")
        (node / "cpulist").write_text("100000-100003\n")
        assert bind_host_to_device_node(0, sysfs=str(tmp_path), bus_id=bus) is None      # none of them allowed
        assert os.sched_getaffinity(0) == before
        (node / "cpulist").write_text(f"{first}\n")
        assert bind_host_to_device_node(0, sysfs=str(tmp_path), bus_id=bus) == 1
        assert os.sched_getaffinity(0) == {first}
        assert bind_host_to_device_node(0, sysfs=str(tmp_path / "missing"), bus_id=bus) is None
    finally:
        os.sched_setaffinity(0, before)


def test_owned_buffer_alias_and_in_place_scatter():
    """World size 1 on CPU tensors: the helpers that save copies keep their contracts (the first owned rows of
    the gather buffer, and the owned rows of the local gradient returned as a view)."""
    from openequivariance_b200.dist import ShardedTensorProductConv
    rows = np.array([0, 0, 1, 2, 2], dtype=np.int64)
    cols = np.array([1, 2, 0, 0, 1], dtype=np.int64)

    class _NoKernels:           # the exchange steps never touch the local convolution
        pass

    conv = ShardedTensorProductConv(None, rows, cols, 3, device="cpu", local_conv=_NoKernels())
    buf = conv.owned_buffer(4, torch.float64)
    assert buf.shape == (3, 4) and buf.data_ptr() == conv.owned_buffer(4, torch.float64).data_ptr()
    dx_local = torch.arange(12, dtype=torch.float64).reshape(3, 4)
    out = conv.scatter_sender_grads(dx_local)
    assert out.data_ptr() == dx_local.data_ptr() and torch.equal(out, dx_local)
