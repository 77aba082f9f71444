"""Fully connected ('uvw') batch tensor product on the GPU (through the C ABI) vs the CPU oracle."""
import numpy as np
import pytest
import torch

import openequivariance_b200 as oeq
from oracle import tp_oracle as orc
from conftest import problem_by_name
from helpers import REL_TOL, rel_err, tp_inputs, to_oeq, to_e3nn

pytestmark = pytest.mark.gpu

CASES = [("uvw_small", 100), ("uvw_small", 3), ("uvw_mul40", 37), ("uvw_rowweights", 50), ("uvw_64", 70),
         # the reference's tetris-polynomial and DiffDock benchmark shapes (benchmark_configs.py:38-47): second
         # input of multiplicity 1 with mixed parities; DiffDock carries per-row 'uvw' weights at multiplicity 48
         ("tetris_poly_1", 60), ("tetris_poly_2", 60), ("diffdock_l1", 40), ("diffdock_l2", 24)]


def run_case(name, batch, dtype, seed=11111):
    p = problem_by_name(name, irrep_dtype=dtype, weight_dtype=dtype)
    tp = oeq.TensorProduct(p, torch_op=True)
    x, y, w, dz = tp_inputs(p, batch, seed)
    if p.shared_weights:
        w = (w / 8).astype(dtype)
    w_oeq = to_oeq(p, w)                      # the documented reordering of 'uvw' weights
    xt, yt, wt, dzt = (torch.from_numpy(a).cuda() for a in (x, y, w_oeq, dz))
    z = tp(xt, yt, wt)
    dx, dy, dw = tp.backward_helper(xt, yt, wt, dzt)
    torch.cuda.synchronize()
    tp.check_device_status()
    tol = REL_TOL[dtype]
    assert rel_err(z.cpu().numpy(), orc.tp_forward(p, x, y, w)) < tol
    rx, ry, rw = orc.tp_backward(p, x, y, w, dz)
    assert rel_err(dx.cpu().numpy(), rx) < tol
    assert rel_err(dy.cpu().numpy(), ry) < tol
    assert rel_err(to_e3nn(p, dw.cpu().numpy()), rw) < tol
    return tp, (xt, yt, wt, dzt), dw


@pytest.mark.parametrize("name,batch", CASES, ids=[f"{n}-{b}" for n, b in CASES])
def test_forward_backward_fp32(name, batch):
    run_case(name, batch, np.float32)


@pytest.mark.parametrize("name,batch", [("uvw_small", 41), ("uvw_mul40", 19), ("uvw_rowweights", 23), ("uvw_64", 33)],
                         ids=["uvw_small", "uvw_mul40", "uvw_rowweights", "uvw_64"])
def test_forward_backward_fp64(name, batch):
    run_case(name, batch, np.float64)


def test_shared_weight_gradient_is_reproducible_and_host_entry_points_reorder():
    tp, (xt, yt, wt, dzt), dw = run_case("uvw_64", 1000, np.float32)
    for _ in range(3):
        assert torch.equal(dw, tp.backward_helper(xt, yt, wt, dzt)[2])
    # host entry points take e3nn-ordered weights and return the e3nn-ordered gradient
    p = tp.config
    x, y, w, dz = tp_inputs(p, 64, 5)
    w = (w / 8).astype(np.float32)
    z = np.zeros((64, p.irreps_out.dim), dtype=np.float32)
    tp.forward_cpu(x, y, z, w)
    assert rel_err(z, orc.tp_forward(p, x, y, w)) < 1e-5
    gx, gy, gw = np.zeros_like(x), np.zeros_like(y), np.zeros_like(w)
    tp.backward_cpu(x, gx, y, gy, dz, w, gw)
    assert rel_err(gw, orc.tp_backward(p, x, y, w, dz)[2]) < 1e-5


def test_full_batch_linearity_and_sampled_rows():
    """Benchmark batch size: linear in X, and sampled rows against the oracle."""
    p = problem_by_name("uvw_64")
    tp = oeq.TensorProduct(p, torch_op=True)
    batch = 100000
    gen = torch.Generator(device="cuda").manual_seed(2)
    x1 = torch.randn(batch, p.irreps_in1.dim, device="cuda", generator=gen)
    x2 = torch.randn(batch, p.irreps_in1.dim, device="cuda", generator=gen)
    y = torch.randn(batch, p.irreps_in2.dim, device="cuda", generator=gen)
    w = torch.randn(p.weight_numel, device="cuda", generator=gen) / 8
    z1, z2, z12 = tp(x1, y, w), tp(x2, y, w), tp(x1 - 3 * x2, y, w)
    assert ((z12 - (z1 - 3 * z2)).abs().max() / z12.abs().max()).item() < 1e-5
    idx = torch.arange(0, batch, 1999, device="cuda")
    w_e3nn = to_e3nn(p, w.cpu().numpy())
    ref = orc.tp_forward(p, x1[idx].cpu().numpy(), y[idx].cpu().numpy(), w_e3nn)
    assert rel_err(z1[idx].cpu().numpy(), ref) < 1e-5


TC_SHAPES = [
    ("64x0e+64x1o+64x2e", "0e+1o+2e", "64x0e+64x1o+64x2e", 777),       # the benchmark shape
    ("40x0e+24x1o", "0e+1o", "16x0e+48x1o+32x2e", 301),                 # multiplicities padded to 32-wide K slices
    ("32x1o+96x2e", "1o+2e+3o", "64x0e+16x1o+32x3o", 130),              # l = 3 output: 7 accumulator rows per batch row
    ("8x0e+8x1o", "0e+1o", "128x0e", 50),                                # wide N, very short K
]


@pytest.mark.parametrize("in1,in2,out,batch", TC_SHAPES, ids=[s[2] for s in TC_SHAPES])
def test_tensor_core_forward_matches_oracle_and_fma_path(in1, in2, out, batch, monkeypatch):
    """Shared-weight FP32 problems run their forward pass on tcgen05 with 3xTF32 compensation; it must
    meet the same FP32 tolerance as the FMA path, on full and ragged row chunks."""
    p = oeq.FullyConnectedTPProblem(in1, in2, out)
    tp = oeq.TensorProduct(p, torch_op=True)
    assert tp.internal.launch_info(0)["threads"] == 21 * 32       # tensor-core kernel selected
    x, y, w, dz = tp_inputs(p, batch, 21)
    w = (w / np.sqrt(max(1, p.weight_numel / len(p.instructions)))).astype(np.float32)
    xt, yt, wt = (torch.from_numpy(a).cuda() for a in (x, y, to_oeq(p, w)))
    z = tp(xt, yt, wt)
    torch.cuda.synchronize()
    tp.check_device_status()
    ref = orc.tp_forward(p, x, y, w)
    assert rel_err(z.cpu().numpy(), ref) < 1e-5
    monkeypatch.setenv("OEQ_B200_UVW_TC", "0")
    fma = oeq.TensorProduct(p, torch_op=True)
    assert fma.internal.launch_info(0)["threads"] == 256
    assert rel_err(fma(xt, yt, wt).cpu().numpy(), ref) < 1e-5
    # repeated launches reuse the accumulator ring and the packed weights
    for _ in range(3):
        assert torch.equal(z, tp(xt, yt, wt))


@pytest.mark.parametrize("in1,in2,out,batch", TC_SHAPES + [s[:3] + (9_000,) for s in TC_SHAPES[1:3]],
                         ids=[f"{s[2]}-{s[3]}" for s in TC_SHAPES] + [f"{s[2]}-9000" for s in TC_SHAPES[1:3]])
def test_tensor_core_backward_matches_oracle_and_fma_path(in1, in2, out, batch, monkeypatch):
    """Shared-weight FP32 problems run their backward pass on tcgen05 too (weight gradient; dX and dY):
    same tolerance as the FMA kernel, padded multiplicities, ragged chunks, many chunks per CTA, and a
    bit-reproducible weight gradient."""
    p = oeq.FullyConnectedTPProblem(in1, in2, out)
    tp = oeq.TensorProduct(p, torch_op=True)
    x, y, w, dz = tp_inputs(p, batch, 29)
    w = (w / np.sqrt(max(1, p.weight_numel / len(p.instructions)))).astype(np.float32)
    xt, yt, wt, dzt = (torch.from_numpy(a).cuda() for a in (x, y, to_oeq(p, w), dz))
    dx, dy, dw = tp.backward_helper(xt, yt, wt, dzt)
    torch.cuda.synchronize()
    tp.check_device_status()
    rx, ry, rw = orc.tp_backward(p, x, y, w, dz)
    assert rel_err(dx.cpu().numpy(), rx) < 1e-5
    assert rel_err(dy.cpu().numpy(), ry) < 1e-5
    assert rel_err(to_e3nn(p, dw.cpu().numpy()), rw) < 1e-5
    for _ in range(2):
        dx2, dy2, dw2 = tp.backward_helper(xt, yt, wt, dzt)
        assert torch.equal(dw, dw2) and torch.equal(dx, dx2) and torch.equal(dy, dy2)
    monkeypatch.setenv("OEQ_B200_UVW_TC_BWD", "0")
    fma = oeq.TensorProduct(p, torch_op=True)
    fx, fy, fw = fma.backward_helper(xt, yt, wt, dzt)
    assert rel_err(fx.cpu().numpy(), rx) < 1e-5 and rel_err(fy.cpu().numpy(), ry) < 1e-5
    assert rel_err(to_e3nn(p, fw.cpu().numpy()), rw) < 1e-5


@pytest.mark.parametrize("in1,in2,out,batch", [s[:3] + (40_000,) for s in TC_SHAPES[1:3]], ids=[s[2] for s in TC_SHAPES[1:3]])
def test_tensor_core_forward_many_tiles_mixed_multiplicities(in1, in2, out, batch, monkeypatch):
    """Every CTA walks many row chunks of every output irrep, so the accumulator ring wraps within and
    across output irreps of different multiplicity; compared with the FMA kernel on all rows and with the
    oracle on sampled rows."""
    p = oeq.FullyConnectedTPProblem(in1, in2, out)
    tp = oeq.TensorProduct(p, torch_op=True)
    assert tp.internal.launch_info(0)["threads"] == 21 * 32
    x, y, w, _ = tp_inputs(p, batch, 23)
    w = (w / np.sqrt(max(1, p.weight_numel / len(p.instructions)))).astype(np.float32)
    xt, yt, wt = (torch.from_numpy(a).cuda() for a in (x, y, to_oeq(p, w)))
    z = tp(xt, yt, wt)
    torch.cuda.synchronize()
    tp.check_device_status()
    monkeypatch.setenv("OEQ_B200_UVW_TC", "0")
    fma = oeq.TensorProduct(p, torch_op=True)
    assert rel_err(z.cpu().numpy(), fma(xt, yt, wt).cpu().numpy()) < 1e-5
    rows = np.arange(0, batch, 997)
    assert rel_err(z.cpu().numpy()[rows], orc.tp_forward(p, x[rows], y[rows], w)) < 1e-5


def test_cross_product_closed_form():
    """'uvw' with shared weights against an answer that can be written down: 1o x 1o -> 1e is the cross
    product / sqrt(6) (sign from the stored Wigner tensor), contracted with W[u, v, w] and the path weight."""
    nu, nv, nw, b = 3, 2, 4, 50
    p = oeq.TPProblem(f"{nu}x1o", f"{nv}x1o", f"{nw}x1e", [(0, 0, 0, "uvw", True)], shared_weights=True,
                      internal_weights=False)
    rng = np.random.default_rng(91)
    x = rng.normal(size=(b, nu, 3)).astype(np.float32)
    y = rng.normal(size=(b, nv, 3)).astype(np.float32)
    w = rng.normal(size=(nu, nv, nw)).astype(np.float32)
    dz = rng.normal(size=(b, nw, 3)).astype(np.float32)
    eps = np.zeros((3, 3, 3))
    for i, j, k in ((0, 1, 2), (1, 2, 0), (2, 0, 1)):
        eps[i, j, k], eps[j, i, k] = 1.0, -1.0
    scale = np.sign(orc.cg(1, 1, 1)[0, 1, 2]) / np.sqrt(6.0) * p.instructions[0].path_weight
    want_z = scale * np.einsum("uvw,ijk,bui,bvj->bwk", w.astype(np.float64), eps, x.astype(np.float64), y.astype(np.float64))
    want_dw = scale * np.einsum("bwk,ijk,bui,bvj->uvw", dz.astype(np.float64), eps, x.astype(np.float64), y.astype(np.float64))
    tp = oeq.TensorProduct(p, torch_op=True)
    w_oeq = to_oeq(p, w.reshape(-1))
    xt, yt, wt, dzt = (torch.from_numpy(np.ascontiguousarray(a)).cuda()
                       for a in (x.reshape(b, -1), y.reshape(b, -1), w_oeq, dz.reshape(b, -1)))
    z = tp(xt, yt, wt)
    _, _, dw = tp.backward_helper(xt, yt, wt, dzt)
    torch.cuda.synchronize()
    assert rel_err(z.cpu().numpy().reshape(want_z.shape), want_z) < 1e-5
    assert rel_err(to_e3nn(p, dw.cpu().numpy()).reshape(want_dw.shape), want_dw) < 1e-5
