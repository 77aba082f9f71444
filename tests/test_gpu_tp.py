"""Batch tensor product on the GPU (through the C ABI) vs the CPU oracle."""
import os

import numpy as np
import pytest
import torch

import openequivariance_b200 as oeq
from oracle import tp_oracle as orc
from conftest import load_golden, problem_by_name
from helpers import REL_TOL, rel_err, tp_inputs, to_oeq, to_e3nn

pytestmark = pytest.mark.gpu

CASES = [
    ("readme", 1000), ("nequip_32", 257), ("cw_mixed", 100), ("mace_128", 64), ("mace_large_128", 33),
    ("uvu_v2", 50), ("uvu_mul40_v3", 37), ("uvu_norm_path", 129), ("uvu_shared", 300),
    # single instructions of the reference's roofline benchmark set (test/benchmark.py:56-70), l up to 7
    ("roofline_1e", 40), ("roofline_5e_3e", 24), ("roofline_6e", 24), ("roofline_7e_4e", 16), ("roofline_7e_7e", 12),
]


def run_case(name, batch, dtype, seed=11111):
    p = problem_by_name(name, irrep_dtype=dtype, weight_dtype=dtype)
    tp = oeq.TensorProduct(p, torch_op=True)
    x, y, w, dz = tp_inputs(p, batch, seed)
    w_oeq = to_oeq(p, w)
    xt, yt, wt, dzt = (torch.from_numpy(a).cuda() for a in (x, y, w_oeq, dz))
    z = tp(xt, yt, wt)
    dx, dy, dw = tp.backward_helper(xt, yt, wt, dzt)
    torch.cuda.synchronize()
    tp.check_device_status()
    z_ref = orc.tp_forward(p, x, y, w)
    dx_ref, dy_ref, dw_ref = orc.tp_backward(p, x, y, w, dz)
    tol = REL_TOL[dtype]
    assert z.dtype == xt.dtype and z.shape == (batch, p.irreps_out.dim)
    assert rel_err(z.cpu().numpy(), z_ref) < tol
    assert rel_err(dx.cpu().numpy(), dx_ref) < tol
    assert rel_err(dy.cpu().numpy(), dy_ref) < tol
    assert rel_err(to_e3nn(p, dw.cpu().numpy()), dw_ref) < tol
    return tp


@pytest.mark.parametrize("name,batch", CASES, ids=[c[0] for c in CASES])
def test_forward_backward_fp32(name, batch):
    run_case(name, batch, np.float32)


@pytest.mark.parametrize("name,batch", [("nequip_32", 65), ("uvu_v2", 31), ("uvu_shared", 77), ("mace_128", 9)],
                         ids=["nequip_32", "uvu_v2", "uvu_shared", "mace_128"])
def test_forward_backward_fp64(name, batch):
    run_case(name, batch, np.float64)


def test_readme_golden_through_host_entry_points():
    """The reference's README shape, seeded like its own buffers, vs its numpy forward."""
    g = load_golden("numpy_tp_forward.npz")
    p = problem_by_name("readme")
    rng = np.random.default_rng(12345)
    x = rng.uniform(size=(1000, 5)).astype(np.float32)
    y = rng.uniform(size=(1000, 7)).astype(np.float32)
    w = rng.uniform(size=(1000, 1)).astype(np.float32)
    z = np.zeros((1000, 5), dtype=np.float32)
    tp = oeq.TensorProduct(p, torch_op=True)
    tp.forward_cpu(x, y, z, w)
    assert np.abs(z[:4] - g["readme__head"]).max() < 5e-5          # the reference's own threshold
    assert rel_err(z[::50], g["readme__out_every_50"]) < 1e-5
    assert np.linalg.norm(z.astype(np.float64)) == pytest.approx(float(g["readme__norm"][0]), rel=1e-6)
    dx, dy, dw = np.zeros_like(x), np.zeros_like(y), np.zeros_like(w)
    dz = rng.uniform(size=z.shape).astype(np.float32)
    tp.backward_cpu(x, dx, y, dy, dz, w, dw)
    rx, ry, rw = orc.tp_backward(p, x, y, w, dz)
    assert rel_err(dx, rx) < 1e-5 and rel_err(dy, ry) < 1e-5 and rel_err(dw, rw) < 1e-5


@pytest.mark.parametrize("name", ["nequip_32", "cw_mixed", "mace_128", "mace_large_128", "roofline_5e_3e",
                                  "roofline_6e", "roofline_7e_7e"])
def test_forward_matches_reference_numpy_golden(name):
    g = load_golden("numpy_tp_forward.npz")
    p = problem_by_name(name)
    x, y, w, ref = (g[f"{name}__{k}"] for k in ("in1", "in2", "w", "out"))
    tp = oeq.TensorProduct(p, torch_op=True)
    z = np.zeros_like(ref)
    tp.forward_cpu(x, y, z, w)
    assert np.abs(z - ref).max() < 5e-5
    assert rel_err(z, ref) < 1e-5


@pytest.mark.parametrize("batch", [0, 1, 2, 31, 4097])
def test_ragged_batches(batch):
    p = problem_by_name("nequip_32")
    tp = oeq.TensorProduct(p, torch_op=True)
    x, y, w, dz = tp_inputs(p, batch, 3)
    xt, yt, wt, dzt = (torch.from_numpy(a).cuda() for a in (x, y, w, dz))
    z = tp(xt, yt, wt)
    dx, dy, dw = tp.backward_helper(xt, yt, wt, dzt)
    assert z.shape == (batch, p.irreps_out.dim)
    if batch:
        assert rel_err(z.cpu().numpy(), orc.tp_forward(p, x, y, w)) < 1e-5
        rx, ry, rw = orc.tp_backward(p, x, y, w, dz)
        assert rel_err(dx.cpu().numpy(), rx) < 1e-5
        assert rel_err(dy.cpu().numpy(), ry) < 1e-5
        assert rel_err(dw.cpu().numpy(), rw) < 1e-5
    tp.check_device_status()


def test_unaligned_views_take_the_element_copy_path():
    """Rows that break the 16-byte rule of the bulk copy (odd offsets into a larger
    allocation) must give the same numbers."""
    p = problem_by_name("nequip_32")
    tp = oeq.TensorProduct(p, torch_op=True)
    batch = 70
    x, y, w, dz = tp_inputs(p, batch, 4)

    def shifted(a):
        flat = torch.zeros(a.size + 1, dtype=torch.float32, device="cuda")
        flat[1:] = torch.from_numpy(a).cuda().reshape(-1)
        return flat[1:].view(a.shape)

    xt, yt, wt, dzt = (shifted(a) for a in (x, y, w, dz))
    assert xt.data_ptr() % 16 != 0
    z = tp(xt, yt, wt)
    dx, dy, dw = tp.backward_helper(xt, yt, wt, dzt)
    assert rel_err(z.cpu().numpy(), orc.tp_forward(p, x, y, w)) < 1e-5
    rx, ry, rw = orc.tp_backward(p, x, y, w, dz)
    assert rel_err(dx.cpu().numpy(), rx) < 1e-5
    assert rel_err(dy.cpu().numpy(), ry) < 1e-5
    assert rel_err(dw.cpu().numpy(), rw) < 1e-5
    tp.check_device_status()


def test_autograd_and_double_backward():
    p = problem_by_name("cw_mixed", irrep_dtype=np.float64, weight_dtype=np.float64)
    tp = oeq.TensorProduct(p, torch_op=True)
    batch = 19
    x, y, w, dz = tp_inputs(p, batch, 5)
    rng = np.random.default_rng(6)
    gx, gy, gw = rng.normal(size=x.shape), rng.normal(size=y.shape), rng.normal(size=w.shape)
    xt, yt, wt, dzt = (torch.from_numpy(a).cuda().requires_grad_(True) for a in (x, y, w, dz))
    z = tp(xt, yt, wt)
    dx, dy, dw = torch.autograd.grad(z, (xt, yt, wt), dzt, create_graph=True)
    rx, ry, rw = orc.tp_backward(p, x, y, w, dz)
    assert rel_err(dx.detach().cpu().numpy(), rx) < 1e-12
    scalar = (dx * torch.from_numpy(gx).cuda()).sum() + (dy * torch.from_numpy(gy).cuda()).sum() + \
             (dw * torch.from_numpy(gw).cuda()).sum()
    ggx, ggy, ggw, ggz = torch.autograd.grad(scalar, (xt, yt, wt, dzt))
    ref = orc.tp_double_backward(p, x, y, w, dz, gx, gy, gw)
    for got, want in zip((ggx, ggy, ggw, ggz), ref):
        assert rel_err(got.cpu().numpy(), want) < 1e-11


@pytest.mark.parametrize("name,dtype,batch", [("readme", np.float64, 77), ("nequip_32", np.float64, 45),
                                              ("uvu_norm_path", np.float64, 19), ("mace_128", np.float32, 40),
                                              ("mace_large_128", np.float32, 11), ("roofline_6e", np.float32, 9)])
def test_one_pass_second_derivatives(name, dtype, batch):
    """The one-pass kernel for the gradient of <ex,dX> + <ey,dY> + <ew,dW> against the oracle (autograd of
    autograd on the CPU) and against the composition of four backward and three forward launches; it is what
    autograd's second backward pass runs when nothing differentiates through its result."""
    p = problem_by_name(name, irrep_dtype=dtype, weight_dtype=dtype)
    tp = oeq.TensorProduct(p, torch_op=True)
    assert tp._has_fused_double_backward
    x, y, w, dz = tp_inputs(p, batch, 15)
    rng = np.random.default_rng(16)
    ex, ey, ew = (rng.normal(size=a.shape).astype(dtype) for a in (x, y, w))
    dev = [torch.from_numpy(a).cuda() for a in (x, y, w, dz, ex, ey, ew)]
    got = tp._double_backward_impl(*dev)
    torch.cuda.synchronize()
    tp.check_device_status()
    ref = orc.tp_double_backward(p, x, y, w, dz, ex, ey, ew)
    tol = REL_TOL[dtype] if dtype == np.float32 else 1e-11
    for g, r in zip(got, ref):
        assert rel_err(g.cpu().numpy(), r) < tol
    # composition, as the reference does it
    xt, yt, wt, dzt, ext, eyt, ewt = dev
    a = tp.backward_helper(ext, eyt, wt, dzt)
    b = tp.backward_helper(xt, yt, ewt, dzt)
    c = tp.backward_helper(ext, yt, wt, dzt)
    d = tp.backward_helper(xt, eyt, wt, dzt)
    gz = tp(ext, yt, wt) + tp(xt, eyt, wt) + tp(xt, yt, ewt)
    for g, r in zip(got, (a[0] + b[0], a[1] + b[1], c[2] + d[2], gz)):
        assert rel_err(g.cpu().numpy(), r.cpu().numpy()) < 10 * tol
    # through autograd: second backward without create_graph takes the one-pass kernel
    xg, yg, wg, dzg = (t.clone().requires_grad_(True) for t in (xt, yt, wt, dzt))
    z = tp(xg, yg, wg)
    dx, dy, dw = torch.autograd.grad(z, (xg, yg, wg), dzg, create_graph=True)
    grads = torch.autograd.grad((dx * ext).sum() + (dy * eyt).sum() + (dw * ewt).sum(), (xg, yg, wg, dzg))
    for g, r in zip(grads, got):
        assert torch.equal(g, r)


def test_second_derivatives_fall_back_to_composition():
    """Shared weights and second inputs of higher multiplicity have no one-pass kernel: the C ABI says so and the
    front end composes."""
    from openequivariance_b200 import _native
    for name in ("uvu_shared", "uvu_v2", "uvw_small"):
        tp = oeq.TensorProduct(problem_by_name(name), torch_op=True)
        assert not tp._has_fused_double_backward
        buf = torch.zeros(1 << 16, device="cuda")
        rc = _native.lib().oeq_tp_double_backward(tp.internal.ptr, 4, *([buf.data_ptr()] * 11), 0)
        assert rc == 2 and b"compose" in _native.lib().oeq_last_error()


def test_shared_weight_gradient_is_reproducible():
    p = problem_by_name("uvu_shared")
    tp = oeq.TensorProduct(p, torch_op=True)
    x, y, w, dz = tp_inputs(p, 5000, 8)
    xt, yt, wt, dzt = (torch.from_numpy(a).cuda() for a in (x, y, w, dz))
    first = tp.backward_helper(xt, yt, wt, dzt)[2].clone()
    for _ in range(4):
        again = tp.backward_helper(xt, yt, wt, dzt)[2]
        assert torch.equal(first, again)


def test_linearity_at_full_mace_batch():
    """Size-independent property at the benchmark's batch size: the product is linear in W."""
    p = problem_by_name("mace_128")
    tp = oeq.TensorProduct(p, torch_op=True)
    batch = 50000
    gen = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(batch, p.irreps_in1.dim, device="cuda", generator=gen)
    y = torch.randn(batch, p.irreps_in2.dim, device="cuda", generator=gen)
    w1 = torch.randn(batch, p.weight_numel, device="cuda", generator=gen)
    w2 = torch.randn(batch, p.weight_numel, device="cuda", generator=gen)
    z1, z2, z12 = tp(x, y, w1), tp(x, y, w2), tp(x, y, w1 + 2 * w2)
    err = (z12 - (z1 + 2 * z2)).abs().max().item() / z12.abs().max().item()
    assert err < 1e-5
    # and a sample of rows against the oracle
    idx = torch.arange(0, batch, 997, device="cuda")
    ref = orc.tp_forward(p, x[idx].cpu().numpy(), y[idx].cpu().numpy(), w1[idx].cpu().numpy())
    assert rel_err(z1[idx].cpu().numpy(), ref) < 1e-5
    tp.check_device_status()


def test_rejects_cpu_tensors_and_bad_shapes():
    p = problem_by_name("readme")
    tp = oeq.TensorProduct(p, torch_op=True)
    with pytest.raises(RuntimeError):
        tp._forward_impl(torch.zeros(3, 5), torch.zeros(3, 7), torch.zeros(3, 1))
    with pytest.raises(ValueError):
        tp._forward_impl(torch.zeros(3, 4, device="cuda"), torch.zeros(3, 7, device="cuda"),
                         torch.zeros(3, 1, device="cuda"))


def test_a_wait_that_runs_out_is_reported_and_the_context_survives():
    """Every staged kernel polls its barriers a bounded number of times and records a code when it gives up.
    The library's probe makes exactly that happen (a barrier that nothing completes, a short poll limit): the
    call must report the device-wait error, and the next launch on the same context must work."""
    from openequivariance_b200 import _native
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.oeq_selftest_bounded_wait(2000, stream) == 5          # OEQ_ERR_DEVICE_WAIT
    assert b"bounded wait" in lib.oeq_last_error()
    assert lib.oeq_selftest_bounded_wait(0, stream) == 1             # rejected argument
    run_case("readme", 100, np.float32)
