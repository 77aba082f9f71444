"""Shared-weight 'uvw' graph convolution (edge sum with unit weights, then the dense contraction per node)
against the CPU oracle's gather - 'uvw' product - scatter-sum."""
import numpy as np
import pytest
import torch

import openequivariance_b200 as oeq
from oracle import tp_oracle as orc
from conftest import problem_by_name
from helpers import REL_TOL, rel_err, random_graph, to_oeq, to_e3nn

pytestmark = pytest.mark.gpu


def _cuda(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


def _inputs(p, nodes, edges, seed):
    rng = np.random.default_rng(seed)
    dt = p.irrep_dtype
    x = rng.normal(size=(nodes, p.irreps_in1.dim)).astype(dt)
    y = rng.normal(size=(edges, p.irreps_in2.dim)).astype(dt)
    w = (rng.normal(size=(p.weight_numel,)) / 8).astype(dt)
    dz = rng.normal(size=(nodes, p.irreps_out.dim)).astype(dt)
    return x, y, w, dz


@pytest.mark.parametrize("deterministic", [False, True], ids=["atomic", "deterministic"])
@pytest.mark.parametrize("name,dtype", [("uvw_64", np.float32), ("uvw_mul40", np.float32), ("tetris_poly_2", np.float32),
                                        ("uvw_64", np.float64)], ids=["uvw_64", "uvw_mul40", "tetris_poly_2", "uvw_64_f64"])
def test_forward_and_gradients(name, dtype, deterministic):
    p = problem_by_name(name, irrep_dtype=dtype, weight_dtype=dtype)
    nodes = 31
    rows, cols = random_graph(nodes, 260, seed=3)
    rows, cols, order, perm = orc.coord_graph(rows, cols)
    x, y, w, dz = _inputs(p, nodes, len(rows), 4)
    conv = oeq.TensorProductConv(p, torch_op=True, deterministic=deterministic)
    xt, yt, dzt, r, c, pm = _cuda(x, y, dz, rows, cols, perm)
    wt = torch.from_numpy(to_oeq(p, w)).cuda()
    index = (r, c, pm) if deterministic else (r, c)
    xt.requires_grad_(True); yt.requires_grad_(True); wt.requires_grad_(True)
    z = conv.forward(xt, yt, wt, *index)
    z.backward(dzt)
    torch.cuda.synchronize()
    conv.check_device_status()
    tol = REL_TOL[dtype]
    z_ref = orc.conv_forward(p, x, y, w, rows, cols)
    rx, ry, rw = orc.conv_backward(p, x, y, w, dz, rows, cols)
    assert rel_err(z.detach().cpu().numpy(), z_ref) < tol
    assert rel_err(xt.grad.cpu().numpy(), rx) < tol
    assert rel_err(yt.grad.cpu().numpy(), ry) < tol
    assert rel_err(to_e3nn(p, wt.grad.cpu().numpy()), rw) < tol
    # the explicit gradient entry point agrees with autograd
    dx, dy, dw = conv.backward_helper(xt.detach(), yt.detach(), wt.detach(), dzt, *index)
    assert rel_err(dx.cpu().numpy(), rx) < tol and rel_err(dy.cpu().numpy(), ry) < tol
    assert rel_err(to_e3nn(p, dw.cpu().numpy()), rw) < tol
    if deterministic:
        z2 = conv.forward(xt.detach(), yt.detach(), wt.detach(), *index)
        assert torch.equal(z2, z.detach())


def test_second_derivatives():
    p = problem_by_name("uvw_mul40", irrep_dtype=np.float64, weight_dtype=np.float64)
    nodes = 9
    rows, cols = random_graph(nodes, 40, seed=5)
    rows, cols, order, perm = orc.coord_graph(rows, cols)
    x, y, w, dz = _inputs(p, nodes, len(rows), 6)
    conv = oeq.TensorProductConv(p, torch_op=True, deterministic=True)
    r, c, pm = _cuda(rows, cols, perm)
    xt, yt, dzt = (t.requires_grad_(True) for t in _cuda(x, y, dz))
    wt = torch.from_numpy(to_oeq(p, w)).cuda().requires_grad_(True)
    z = conv.forward(xt, yt, wt, r, c, pm)
    dx, dy, dw = torch.autograd.grad(z, (xt, yt, wt), dzt, create_graph=True)
    rng = np.random.default_rng(7)
    gx, gy = (torch.from_numpy(rng.normal(size=a.shape)).cuda() for a in (x, y))
    gw_e3nn = rng.normal(size=w.shape)
    gw = torch.from_numpy(to_oeq(p, gw_e3nn)).cuda()
    scalar = (dx * gx).sum() + (dy * gy).sum() + (dw * gw).sum()
    got = torch.autograd.grad(scalar, (xt, yt, wt, dzt))
    cx, cy, cw, cdz = (torch.from_numpy(a).requires_grad_(True) for a in (x, y, w, dz))
    zz = orc.conv_torch(p, cx, cy, cw, torch.from_numpy(rows), torch.from_numpy(cols))
    ex, ey, ew = torch.autograd.grad(zz, (cx, cy, cw), cdz, create_graph=True)
    s = (ex * gx.cpu()).sum() + (ey * gy.cpu()).sum() + (ew * torch.from_numpy(gw_e3nn)).sum()
    want = torch.autograd.grad(s, (cx, cy, cw, cdz))
    assert rel_err(got[0].cpu().numpy(), want[0].numpy()) < 1e-11
    assert rel_err(got[1].cpu().numpy(), want[1].numpy()) < 1e-11
    assert rel_err(to_e3nn(p, got[2].cpu().numpy()), want[2].numpy()) < 1e-11
    assert rel_err(got[3].cpu().numpy(), want[3].numpy()) < 1e-11


def test_rejects_per_edge_uvw_weights():
    with pytest.raises(AssertionError):
        oeq.TensorProductConv(problem_by_name("diffdock_l1"), torch_op=True)
