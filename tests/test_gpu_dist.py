"""The receiver-sharded convolution on real ranks: two processes, one GPU each, NCCL.

Skipped on a machine with fewer than two GPUs.  Each rank runs the CUDA kernels on its shard of a periodic
radius graph with Morton-ordered ids (the benchmark's graph class), the halo rows cross NVLink through
NCCL, and every rank checks its rows of Z, dX, dY, dW against the float64 oracle of the whole graph, then
repeats the step and wants the same bits.  NVLS is switched off: a test rank that dies must not take its
peer's GPU down with it."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from oracle import tp_oracle as orc
    from conftest import problem_by_name
    from helpers import conv_inputs, rel_err
    from openequivariance_b200.dist import ShardedTensorProductConv
    from openequivariance_b200.graph import periodic_radius_graph, spherical_harmonics
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        errs = {}
        for name, nodes, lmax in (("nequip_32", 1200, 2), ("mace_large_128", 300, 3)):
            p = problem_by_name(name)
            g = periodic_radius_graph(nodes, 30.0, seed=7, numbering="morton")
            x, _, w, dz = conv_inputs(p, nodes, g.nnz, 51)
            y = spherical_harmonics(lmax, g.vectors).astype(np.float32)
            conv = ShardedTensorProductConv(p, g.rows, g.cols, nodes, device=device)
            plan = conv.plan
            assert plan.halo.size > 0                      # the exchange is exercised
            dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
            xs, dzs = dev(x[plan.node_lo:plan.node_hi]), dev(dz[plan.node_lo:plan.node_hi])
            ys, ws = dev(y[plan.edge_lo:plan.edge_hi]), dev(w[plan.edge_lo:plan.edge_hi])
            z, dx, dy, dw = conv.forward_backward(xs, ys, ws, dzs)
            torch.cuda.synchronize()
            conv.conv.check_device_status()
            z_ref = orc.conv_forward(p, x, y, w, g.rows, g.cols)
            rx, ry, rw = orc.conv_backward(p, x, y, w, dz, g.rows, g.cols)
            errs[name] = max(rel_err(z.cpu().numpy(), z_ref[plan.node_lo:plan.node_hi]),
                             rel_err(dx.cpu().numpy(), rx[plan.node_lo:plan.node_hi]),
                             rel_err(dy.cpu().numpy(), ry[plan.edge_lo:plan.edge_hi]),
                             rel_err(dw.cpu().numpy(), rw[plan.edge_lo:plan.edge_hi]))
            z2, dx2, dy2, dw2 = conv.forward_backward(xs, ys, ws, dzs)
            same = all(torch.equal(a, b) for a, b in ((z, z2), (dx, dx2), (dy, dy2), (dw, dw2)))
            errs[name + "_bits"] = 0.0 if same else 1.0
            # the autograd path (fresh gather buffer) gives the same numbers
            xg = xs.clone().requires_grad_(True)
            conv(xg, ys, ws).backward(dzs)
            errs[name + "_autograd"] = rel_err(xg.grad.cpu().numpy(), dx.cpu().numpy())
        result[rank] = errs
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpu_ranks_match_the_oracle_and_repeat_bit_for_bit():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, 29731
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, result)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=600)
        assert pr.exitcode == 0
    assert len(result) == world
    for rank in range(world):
        for key, err in result[rank].items():
            assert err < 1e-5, (rank, key, err)
