"""The torch custom ops: schema, fake-tensor kernels and autograd registration (``torch.library.opcheck``), and
a ``torch.compile(fullgraph=True)`` call of each front end, as the reference's registration promises
(reference: openequivariance/implementations/TensorProductBase.py:236-298,
openequivariance/implementations/convolution/ConvolutionBase.py:560-709)."""
import numpy as np
import pytest
import torch

import openequivariance_b200 as oeq
from oracle import tp_oracle as orc
from conftest import problem_by_name
from helpers import conv_inputs, random_graph, tp_inputs

pytestmark = pytest.mark.gpu

CHECKS = ("test_schema", "test_faketensor", "test_autograd_registration")


def _cuda(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


@pytest.mark.parametrize("name", ["nequip_32", "uvu_shared", "uvw_small"])
def test_tensor_product_ops(name):
    p = problem_by_name(name)
    tp = oeq.TensorProduct(p, torch_op=True)
    x, y, w, dz = tp_inputs(p, 9, 3)
    xt, yt, wt, dzt = _cuda(x, y, w, dz)
    torch.library.opcheck(tp.forward, (xt, yt, wt), test_utils=CHECKS)
    torch.library.opcheck(tp.backward_helper, (xt, yt, wt, dzt), test_utils=CHECKS)
    # fake tensors: shapes and dtypes without running a kernel
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode(allow_non_fake_inputs=False) as mode:
        fx, fy, fw = (mode.from_tensor(t) for t in (xt, yt, wt))
        fz = tp.forward(fx, fy, fw)
        assert tuple(fz.shape) == (9, p.irreps_out.dim) and fz.dtype == xt.dtype
    # compiled call: one graph, same numbers, gradients flow
    xg = xt.clone().requires_grad_(True)
    compiled = torch.compile(lambda a, b, c: tp.forward(a, b, c), fullgraph=True)
    z_c = compiled(xg, yt, wt)
    z_e = tp.forward(xt, yt, wt)
    assert torch.equal(z_c.detach(), z_e)
    z_c.backward(dzt)
    dx_e = tp.backward_helper(xt, yt, wt, dzt)[0]
    assert torch.equal(xg.grad, dx_e)


@pytest.mark.parametrize("deterministic", [False, True], ids=["atomic", "deterministic"])
def test_convolution_ops(deterministic):
    p = problem_by_name("nequip_32")
    nodes = 17
    rows, cols = random_graph(nodes, 90, seed=4)
    rows, cols, order, perm = orc.coord_graph(rows, cols)
    x, y, w, dz = conv_inputs(p, nodes, len(rows), 5)
    conv = oeq.TensorProductConv(p, torch_op=True, deterministic=deterministic)
    xt, yt, wt, dzt, r, c, pm = _cuda(x, y, w, dz, rows, cols, perm)
    index = (r, c, pm) if deterministic else (r, c)
    torch.library.opcheck(conv.forward, (xt, yt, wt, *index), test_utils=CHECKS)
    torch.library.opcheck(conv.backward_helper, (xt, yt, wt, dzt, *index), test_utils=CHECKS)
    xg = xt.clone().requires_grad_(True)
    compiled = torch.compile(lambda a, b, c_, *idx: conv.forward(a, b, c_, *idx), fullgraph=True)
    z_c = compiled(xg, yt, wt, *index)
    z_e = conv.forward(xt, yt, wt, *index)
    if deterministic:
        assert torch.equal(z_c.detach(), z_e)
    else:
        assert (z_c.detach() - z_e).abs().max().item() <= 1e-5 * z_e.abs().max().item()
    z_c.backward(dzt)
    dx_e = conv.backward_helper(xt, yt, wt, dzt, *index)[0]
    assert (xg.grad - dx_e).abs().max().item() <= 1e-5 * dx_e.abs().max().item()
