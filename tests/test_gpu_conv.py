"""Fused graph convolution on the GPU (through the C ABI) vs the CPU oracle."""
import numpy as np
import pytest
import torch

import openequivariance_b200 as oeq
from oracle import tp_oracle as orc
from conftest import problem_by_name
from helpers import REL_TOL, rel_err, conv_inputs, random_graph

pytestmark = pytest.mark.gpu


def cuda(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


def check_conv(problem, nodes, rows, cols, seed, deterministic, dtype=np.float32):
    edges = len(rows)
    x, y, w, dz = conv_inputs(problem, nodes, edges, seed)
    conv = oeq.TensorProductConv(problem, torch_op=True, deterministic=deterministic)
    if deterministic:
        rows, cols, order, perm = orc.coord_graph(rows, cols)
        y, w = y[order], w[order]
        index = cuda(rows, cols, perm)
    else:
        index = cuda(rows, cols)
    xt, yt, wt, dzt = cuda(x, y, w, dz)
    z = conv.forward(xt, yt, wt, *index)
    dx, dy, dw = conv.backward_helper(xt, yt, wt, dzt, *index)
    torch.cuda.synchronize()
    conv.check_device_status()
    tol = REL_TOL[dtype]
    z_ref = orc.conv_forward(problem, x, y, w, rows, cols)
    rx, ry, rw = orc.conv_backward(problem, x, y, w, dz, rows, cols)
    assert rel_err(z.cpu().numpy(), z_ref) < tol
    assert rel_err(dx.cpu().numpy(), rx) < tol
    assert rel_err(dy.cpu().numpy(), ry) < tol
    assert rel_err(dw.cpu().numpy(), rw) < tol
    return conv, (xt, yt, wt, dzt, index), (z, dx, dy, dw)


@pytest.mark.parametrize("deterministic", [False, True], ids=["atomic", "deterministic"])
@pytest.mark.parametrize("name", ["readme", "nequip_32", "cw_mixed", "mace_128", "mace_large_128"])
def test_small_random_graph(name, deterministic):
    p = problem_by_name(name)
    nodes = 23
    rows, cols = random_graph(nodes, 150, seed=2)           # duplicates, self loops, asymmetric
    check_conv(p, nodes, rows, cols, 9, deterministic)


@pytest.mark.parametrize("deterministic", [False, True], ids=["atomic", "deterministic"])
def test_fp64(deterministic):
    p = problem_by_name("nequip_32", irrep_dtype=np.float64, weight_dtype=np.float64)
    rows, cols = random_graph(40, 300, seed=3, symmetric=True)
    check_conv(p, 40, rows, cols, 10, deterministic, dtype=np.float64)


@pytest.mark.parametrize("name,dtype,deterministic,epi", [("nequip_32", np.float32, True, 4), ("nequip_32", np.float32, False, 3),
                                                         ("readme", np.float64, True, 3), ("readme", np.float32, False, 4)])
def test_edges_per_item(name, dtype, deterministic, epi, monkeypatch):
    """Narrow problems stage runs of consecutive edges as one item (two by default); other run lengths, ragged
    runs at chunk ends, rows that do not qualify for bulk copies, and bit-equality with one edge per item in the
    deterministic variant."""
    p = problem_by_name(name, irrep_dtype=dtype, weight_dtype=dtype)
    nodes = 57
    rows, cols = random_graph(nodes, 1003, seed=41)
    monkeypatch.setenv("OEQ_B200_EPI", str(epi))
    monkeypatch.setenv("OEQ_B200_EPI_STAGES", "3")
    conv, inputs, got = check_conv(p, nodes, rows, cols, 42, deterministic, dtype=dtype)
    assert conv.internal.launch_info(0)["stages"] <= 3
    if deterministic:
        monkeypatch.setenv("OEQ_B200_EPI", "1")
        one, _, want = check_conv(p, nodes, rows, cols, 42, deterministic, dtype=dtype)
        for a, b in zip(got, want):
            assert torch.equal(a, b)


@pytest.mark.parametrize("name", ["nequip_32", "mace_128"])
def test_element_copy_staging(name, monkeypatch):
    """Rows staged with element copies instead of bulk copies (what unaligned buffers get), forced for every array."""
    monkeypatch.setenv("OEQ_B200_NO_BULK", "1")
    p = problem_by_name(name)
    rows, cols = random_graph(31, 400, seed=51)
    for deterministic in (True, False):
        check_conv(p, 31, rows, cols, 52, deterministic)


def test_fp64_widest_rows():
    """MACE-large rows in FP64: a backward stage only fits because the output-gradient row is staged in phases."""
    p = problem_by_name("mace_large_128", irrep_dtype=np.float64, weight_dtype=np.float64)
    rows, cols = random_graph(19, 120, seed=5)
    check_conv(p, 19, rows, cols, 12, True, dtype=np.float64)


@pytest.mark.parametrize("deterministic", [False, True], ids=["atomic", "deterministic"])
def test_isolated_nodes_and_hubs(deterministic):
    """Receivers without edges must come out as zero rows; one node receives most edges."""
    p = problem_by_name("nequip_32")
    nodes = 300
    rng = np.random.default_rng(4)
    rows = np.concatenate([np.full(2000, 17), rng.integers(100, 200, 500)]).astype(np.int64)
    cols = np.concatenate([rng.integers(0, nodes, 2000), rng.integers(250, 300, 500)]).astype(np.int64)
    conv, _, (z, dx, _, _) = check_conv(p, nodes, rows, cols, 11, deterministic)
    untouched = np.setdiff1d(np.arange(nodes), rows)
    assert torch.count_nonzero(z[torch.from_numpy(untouched).cuda()]) == 0
    silent = np.setdiff1d(np.arange(nodes), cols)
    assert torch.count_nonzero(dx[torch.from_numpy(silent).cuda()]) == 0


@pytest.mark.parametrize("deterministic", [False, True], ids=["atomic", "deterministic"])
@pytest.mark.parametrize("edges", [0, 1, 5])
def test_tiny_edge_counts(edges, deterministic):
    p = problem_by_name("nequip_32")
    nodes = 6
    rows, cols = random_graph(nodes, edges, seed=5)
    if edges == 0:
        conv = oeq.TensorProductConv(p, torch_op=True, deterministic=deterministic)
        x, y, w, dz = conv_inputs(p, nodes, 0, 1)
        idx = cuda(rows, cols) + (cuda(rows) if deterministic else [])
        xt, yt, wt, dzt = cuda(x, y, w, dz)
        z = conv.forward(xt, yt, wt, *idx)
        dx, dy, dw = conv.backward_helper(xt, yt, wt, dzt, *idx)
        assert z.shape == (nodes, p.irreps_out.dim) and torch.count_nonzero(z) == 0
        assert torch.count_nonzero(dx) == 0 and dy.shape[0] == 0 and dw.shape[0] == 0
    else:
        check_conv(p, nodes, rows, cols, 12, deterministic)


def test_deterministic_is_bit_reproducible_and_matches_atomic():
    p = problem_by_name("nequip_32")
    nodes = 2000
    rows, cols = random_graph(nodes, 30000, seed=6, symmetric=True)
    conv, (xt, yt, wt, dzt, index), (z, dx, dy, dw) = check_conv(p, nodes, rows, cols, 13, True)
    for _ in range(4):
        z2 = conv.forward(xt, yt, wt, *index)
        dx2, dy2, dw2 = conv.backward_helper(xt, yt, wt, dzt, *index)
        assert torch.equal(z, z2) and torch.equal(dx, dx2) and torch.equal(dy, dy2) and torch.equal(dw, dw2)
    atomic = oeq.TensorProductConv(p, torch_op=True, deterministic=False)
    za = atomic.forward(xt, yt, wt, index[0], index[1])
    dxa, dya, dwa = atomic.backward_helper(xt, yt, wt, dzt, index[0], index[1])
    assert rel_err(za.cpu().numpy(), z.cpu().numpy()) < 1e-5
    assert rel_err(dxa.cpu().numpy(), dx.cpu().numpy()) < 1e-5
    assert rel_err(dya.cpu().numpy(), dy.cpu().numpy()) < 1e-5
    assert rel_err(dwa.cpu().numpy(), dw.cpu().numpy()) < 1e-5


def test_autograd_and_double_backward():
    p = problem_by_name("cw_mixed", irrep_dtype=np.float64, weight_dtype=np.float64)
    nodes = 12
    rows, cols = random_graph(nodes, 60, seed=7)
    rows, cols, order, perm = orc.coord_graph(rows, cols)
    x, y, w, dz = conv_inputs(p, nodes, len(rows), 14)
    conv = oeq.TensorProductConv(p, torch_op=True, deterministic=True)
    r, c, pm = cuda(rows, cols, perm)
    xt, yt, wt, dzt = (t.requires_grad_(True) for t in cuda(x, y, w, dz))
    z = conv.forward(xt, yt, wt, r, c, pm)
    dx, dy, dw = torch.autograd.grad(z, (xt, yt, wt), dzt, create_graph=True)
    rng = np.random.default_rng(15)
    gx, gy, gw = (torch.from_numpy(rng.normal(size=a.shape)).cuda() for a in (x, y, w))
    scalar = (dx * gx).sum() + (dy * gy).sum() + (dw * gw).sum()
    got = torch.autograd.grad(scalar, (xt, yt, wt, dzt))
    # oracle: same scalar through autograd on the CPU
    cx, cy, cw, cdz = (torch.from_numpy(a).requires_grad_(True) for a in (x, y, w, dz))
    zz = orc.conv_torch(p, cx, cy, cw, torch.from_numpy(rows), torch.from_numpy(cols))
    ex, ey, ew = torch.autograd.grad(zz, (cx, cy, cw), cdz, create_graph=True)
    s = (ex * gx.cpu()).sum() + (ey * gy.cpu()).sum() + (ew * gw.cpu()).sum()
    want = torch.autograd.grad(s, (cx, cy, cw, cdz))
    for a, b in zip(got, want):
        assert rel_err(a.cpu().numpy(), b.numpy()) < 1e-11


@pytest.mark.parametrize("deterministic", [True, False])
@pytest.mark.parametrize("name,dtype,tol", [("nequip_32", np.float32, 2e-5), ("mace_128", np.float32, 2e-5),
                                            ("readme", np.float64, 1e-11), ("uvu_norm_path", np.float64, 1e-11)])
def test_fused_second_derivatives(name, dtype, tol, deterministic):
    """Second derivatives in two fused launches (taken when nothing differentiates through the result) against
    the oracle's autograd and against the composed path (four backward and three forward launches)."""
    p = problem_by_name(name, irrep_dtype=dtype, weight_dtype=dtype)
    nodes = 40
    rows, cols = random_graph(nodes, 700, seed=21)
    rows, cols, order, perm = orc.coord_graph(rows, cols)
    x, y, w, dz = conv_inputs(p, nodes, len(rows), 22)
    x[5] = 0  # (values only; node 5 still sends)
    conv = oeq.TensorProductConv(p, torch_op=True, deterministic=deterministic)
    assert conv._has_fused_double_backward()
    r, c, pm = cuda(rows, cols, perm)
    index = (r, c, pm) if deterministic else (r, c)
    xt, yt, wt, dzt = (t.requires_grad_(True) for t in cuda(x, y, w, dz))
    rng = np.random.default_rng(23)
    ex, ey, ew = (torch.from_numpy(rng.normal(size=a.shape).astype(dtype)).cuda() for a in (x, y, w))

    def second(create_graph):
        z = conv.forward(xt, yt, wt, *index)
        dx, dy, dw = torch.autograd.grad(z, (xt, yt, wt), dzt, create_graph=True)
        scalar = (dx * ex).sum() + (dy * ey).sum() + (dw * ew).sum()
        return torch.autograd.grad(scalar, (xt, yt, wt, dzt), create_graph=create_graph)

    fused = second(False)
    composed = [t.detach() for t in second(True)]
    conv.check_device_status()
    cx, cy, cw, cdz = (torch.from_numpy(a.astype(np.float64)).requires_grad_(True) for a in (x, y, w, dz))
    zz = orc.conv_torch(p, cx, cy, cw, torch.from_numpy(rows), torch.from_numpy(cols))
    gx, gy, gw = torch.autograd.grad(zz, (cx, cy, cw), cdz, create_graph=True)
    s = (gx * ex.cpu().double()).sum() + (gy * ey.cpu().double()).sum() + (gw * ew.cpu().double()).sum()
    want = torch.autograd.grad(s, (cx, cy, cw, cdz))
    for a, b, cmp in zip(fused, want, composed):
        assert rel_err(a.cpu().numpy(), b.numpy()) < tol
        assert rel_err(a.cpu().numpy(), cmp.cpu().numpy()) < tol
    if deterministic:
        again = second(False)
        for a, b in zip(fused, again):
            assert torch.equal(a, b)


def test_fused_second_derivatives_staging_variants(monkeypatch):
    """Cotangent rows at addresses that rule out bulk copies, and bulk copies switched off altogether: same bits as
    the aligned run of the deterministic variant (only the way rows reach shared memory differs)."""
    p = problem_by_name("mace_128")
    nodes = 50
    rows, cols = random_graph(nodes, 900, seed=61)
    rows, cols, order, perm = orc.coord_graph(rows, cols)
    x, y, w, dz = conv_inputs(p, nodes, len(rows), 62)
    conv = oeq.TensorProductConv(p, torch_op=True, deterministic=True)
    r, c, pm = cuda(rows, cols, perm)
    xt, yt, wt, dzt = cuda(x, y, w, dz)
    rng = np.random.default_rng(63)
    ex, ey, ew = (torch.from_numpy(rng.normal(size=a.shape).astype(np.float32)).cuda() for a in (x, y, w))
    want = conv._double_backward_impl(xt, yt, wt, dzt, ex, ey, ew, r, c, pm)
    assert want is not None

    def shifted(t):           # the same values four bytes off a 16-byte boundary
        buf = torch.empty(t.numel() + 1, dtype=t.dtype, device=t.device)
        out = buf[1:].view(t.shape)
        out.copy_(t)
        assert out.data_ptr() % 16 == 4
        return out

    got = conv._double_backward_impl(xt, yt, wt, dzt, shifted(ex), shifted(ey), shifted(ew), r, c, pm)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    monkeypatch.setenv("OEQ_B200_NO_BULK", "1")
    got = conv._double_backward_impl(xt, yt, wt, dzt, ex, ey, ew, r, c, pm)
    conv.check_device_status()
    for a, b in zip(got, want):
        assert torch.equal(a, b)


def test_fused_second_derivatives_edge_blocks(monkeypatch):
    """Scratch smaller than the edge list: the receiver-order walk runs over blocks of edges."""
    monkeypatch.setenv("OEQ_B200_BWD_SCRATCH_MB", "1")
    monkeypatch.setenv("OEQ_B200_BWD_MIN_BLOCK", "64")
    p = problem_by_name("mace_128")
    nodes = 300
    rows, cols = random_graph(nodes, 6000, seed=31)
    rows, cols, order, perm = orc.coord_graph(rows, cols)
    x, y, w, dz = conv_inputs(p, nodes, len(rows), 32)
    conv = oeq.TensorProductConv(p, torch_op=True, deterministic=True)
    r, c, pm = cuda(rows, cols, perm)
    xt, yt, wt, dzt = cuda(x, y, w, dz)
    assert conv.internal.workspace_bytes(nodes, len(rows)) < len(rows) * p.irreps_in1.dim * 4
    rng = np.random.default_rng(33)
    ex, ey, ew = (torch.from_numpy(rng.normal(size=a.shape).astype(np.float32)).cuda() for a in (x, y, w))
    got = conv._double_backward_impl(xt, yt, wt, dzt, ex, ey, ew, r, c, pm)
    assert got is not None
    a = conv._backward_impl(ex, ey, wt, dzt, r, c, pm)
    b = conv._backward_impl(xt, yt, ew, dzt, r, c, pm)
    cc = conv._backward_impl(ex, yt, wt, dzt, r, c, pm)
    d = conv._backward_impl(xt, ey, wt, dzt, r, c, pm)
    gz = (conv._forward_impl(ex, yt, wt, r, c, pm) + conv._forward_impl(xt, ey, wt, r, c, pm)
          + conv._forward_impl(xt, yt, ew, r, c, pm))
    conv.check_device_status()
    for u, v in zip(got, (a[0] + b[0], a[1] + b[1], cc[2] + d[2], gz)):
        assert rel_err(u.cpu().numpy(), v.cpu().numpy()) < 2e-5


def test_readme_call_sequence():
    """The reference README's convolution example (3 nodes, 4 edges), atomic then deterministic."""
    p = problem_by_name("readme")
    gen = torch.Generator(device="cuda").manual_seed(0)
    rows = torch.tensor([0, 1, 1, 2], device="cuda")
    cols = torch.tensor([1, 0, 2, 1], device="cuda")
    X = torch.rand(3, 5, device="cuda", generator=gen)
    Y = torch.rand(4, 7, device="cuda", generator=gen)
    W = torch.rand(4, p.weight_numel, device="cuda", generator=gen)
    tp_conv = oeq.TensorProductConv(p, torch_op=True, deterministic=False)
    Z = tp_conv.forward(X, Y, W, rows, cols)
    sender_perm = torch.argsort(cols, stable=True)
    det = oeq.TensorProductConv(p, torch_op=True, deterministic=True)
    Z2 = det.forward(X, Y, W, rows, cols, sender_perm)
    ref = orc.conv_forward(p, X.cpu().numpy(), Y.cpu().numpy(), W.cpu().numpy(), rows.cpu().numpy(),
                           cols.cpu().numpy())
    assert rel_err(Z.cpu().numpy(), ref) < 1e-5 and rel_err(Z2.cpu().numpy(), ref) < 1e-5


@pytest.mark.parametrize("name,slab_edges", [("nequip_32", 64), ("mace_128", 500), ("cw_mixed", 10_000)])
def test_streamed_host_tensors(name, slab_edges):
    """Slab streaming over pinned host tensors: same Z, dY, dW as the resident deterministic
    convolution bit for bit (same kernels, same order), dX up to the slab-wise summation order."""
    from openequivariance_b200.stream import StreamedTensorProductConv
    p = problem_by_name(name)
    nodes = 120
    rows, cols = random_graph(nodes, 1500, seed=12)
    conv, (xt, yt, wt, dzt, index), (z, dx, dy, dw) = check_conv(p, nodes, rows, cols, 13, True)
    # the slab pipeline runs the backward pass without scratch memory (sender-order kernel): same bits as that
    dx, dy, dw = conv._backward_impl(xt, yt, wt, dzt, *index, scratch=False)
    rows_s, cols_s = index[0].cpu().numpy(), index[1].cpu().numpy()
    streamed = StreamedTensorProductConv(p, rows_s, cols_s, nodes, slab_edges=slab_edges)
    pin = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
    x_h, y_h, w_h, dz_h = pin(xt), pin(yt), pin(wt), pin(dzt)
    out = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in (z, dx, dy, dw)]
    for _ in range(2):           # the second pass re-uses the device buffers
        for t in out:
            t.fill_(float("nan"))
        streamed.forward_backward_host(x_h, y_h, w_h, dz_h, *out)
        torch.cuda.synchronize()
        conv.check_device_status()
        streamed.conv.check_device_status()
        assert torch.equal(out[0], z.cpu()) and torch.equal(out[2], dy.cpu()) and torch.equal(out[3], dw.cpu())
        assert rel_err(out[1].numpy(), dx.cpu().numpy()) < REL_TOL[np.float32]
    if slab_edges < 1500:
        assert len(streamed.slabs) > 2


def test_sharded_host_tensor_step_on_one_rank():
    """The host-tensor entry point of the sharded convolution (one rank: no halo): owned rows in, edge slabs
    streamed with lazily supplied weight slices, results equal to the resident convolution."""
    from openequivariance_b200.dist import ShardedTensorProductConv
    p = problem_by_name("mace_128")
    nodes = 90
    rows, cols = random_graph(nodes, 1100, seed=31)
    conv, (xt, yt, wt, dzt, index), (z, dx, dy, dw) = check_conv(p, nodes, rows, cols, 32, True)
    dx, dy, dw = conv._backward_impl(xt, yt, wt, dzt, *index, scratch=False)     # what the slab pipeline runs
    sharded = ShardedTensorProductConv(p, index[0].cpu().numpy(), index[1].cpu().numpy(), nodes)
    pin = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
    x_h, y_h, w_h, dz_h = pin(xt), pin(yt), pin(wt), pin(dzt)
    out = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).fill_(float("nan")) for t in (z, dx, dy, dw)]
    sharded.forward_backward_host(x_h, y_h, lambda i, lo, hi: w_h[lo:hi], dz_h, out[0], out[1], out[2],
                                  lambda i, lo, hi: out[3][lo:hi], slab_edges=300)
    torch.cuda.synchronize()
    sharded.conv.check_device_status()
    assert len(sharded.slab_plan(300).slabs) > 2
    assert torch.equal(out[0], z.cpu()) and torch.equal(out[2], dy.cpu()) and torch.equal(out[3], dw.cpu())
    assert rel_err(out[1].numpy(), dx.cpu().numpy()) < REL_TOL[np.float32]
    h2d, d2h = sharded.host_bytes(4)
    assert d2h == sum(t.numel() * 4 for t in out) and h2d == d2h + 24 * len(rows)


@pytest.mark.parametrize("deterministic", [False, True], ids=["atomic", "deterministic"])
@pytest.mark.parametrize("name", ["mace_128", "mace_large_128"])
def test_tensor_core_forward(name, deterministic, monkeypatch):
    """The opt-in tcgen05 forward pass (3xTF32) against the oracle, and against the FMA kernel's launch shape."""
    monkeypatch.setenv("OEQ_B200_UVU_TC", "1")
    p = problem_by_name(name)
    nodes = 61
    rows, cols = random_graph(nodes, 900, seed=21)
    conv, _, _ = check_conv(p, nodes, rows, cols, 22, deterministic)
    info = conv.internal.launch_info(0)
    assert info["threads"] == 320 and info["partitions"] == 2      # 8 consumer warps, staging warp, MMA warp
    if deterministic:                                               # bit-reproducible run to run
        rows_s, cols_s, order, perm = orc.coord_graph(rows, cols)
        x, y, w, _ = conv_inputs(p, nodes, len(rows), 22)
        args = cuda(x, y[order], w[order], rows_s, cols_s, perm)
        first = conv.forward(*args)
        for _ in range(3):
            assert torch.equal(conv.forward(*args), first)


@pytest.mark.parametrize("chunk", [16, 128])
def test_widest_rows_many_chunks_per_group(chunk, monkeypatch):
    """MACE-large rows on a graph large enough that every group walks several work chunks (small chunks make
    that happen at a size the oracle can follow): chunk boundaries moved to node boundaries, the phased
    backward stages and the ring of dY partials all wrap many times."""
    monkeypatch.setenv("OEQ_B200_CHUNK", str(chunk))
    p = problem_by_name("mace_large_128")
    nodes = 700
    rows, cols = random_graph(nodes, 20000, seed=31)
    conv, (xt, yt, wt, dzt, index), (z, dx, dy, dw) = check_conv(p, nodes, rows, cols, 32, True)
    z2 = conv.forward(xt, yt, wt, *index)
    dx2, dy2, dw2 = conv.backward_helper(xt, yt, wt, dzt, *index)
    assert torch.equal(z, z2) and torch.equal(dx, dx2) and torch.equal(dy, dy2) and torch.equal(dw, dw2)
    atomic = oeq.TensorProductConv(p, torch_op=True, deterministic=False)
    za = atomic.forward(xt, yt, wt, index[0], index[1])
    dxa, dya, dwa = atomic.backward_helper(xt, yt, wt, dzt, index[0], index[1])
    atomic.check_device_status()
    assert rel_err(za.cpu().numpy(), z.cpu().numpy()) < 1e-5
    assert rel_err(dxa.cpu().numpy(), dx.cpu().numpy()) < 1e-5
    assert rel_err(dya.cpu().numpy(), dy.cpu().numpy()) < 1e-5
    assert rel_err(dwa.cpu().numpy(), dw.cpu().numpy()) < 1e-5


_periodic_cache = {}


def _periodic_case(name, nodes, lmax):
    """Graph, inputs and oracle results of one periodic-graph case, evaluated once for both variants."""
    from openequivariance_b200.graph import periodic_radius_graph, spherical_harmonics
    key = (name, nodes, lmax)
    if key not in _periodic_cache:
        p = problem_by_name(name)
        g = periodic_radius_graph(nodes, 30.0, seed=5, numbering="morton")
        x, _, w, dz = conv_inputs(p, nodes, g.nnz, 41)
        y = spherical_harmonics(lmax, g.vectors).astype(np.float32)
        z_ref = orc.conv_forward(p, x, y, w, g.rows, g.cols)
        grads = orc.conv_backward(p, x, y, w, dz, g.rows, g.cols)
        _periodic_cache[key] = (p, g, (x, y, w, dz), z_ref, grads)
    return _periodic_cache[key]


@pytest.mark.parametrize("deterministic", [False, True], ids=["atomic", "deterministic"])
@pytest.mark.parametrize("name,nodes,lmax", [("nequip_32", 1500, 2), ("mace_large_128", 400, 3)])
def test_periodic_radius_graph(name, nodes, lmax, deterministic):
    """The benchmark's own graph class: points uniform in a periodic cube, both directions of every pair within
    the cutoff for mean degree 30, Morton-ordered node ids, spherical harmonics of the edge vectors as the
    second input.  (The wide problem runs on fewer nodes so that the float64 oracle's [E, Z.dim] messages fit.)"""
    p, g, (x, y, w, dz), z_ref, (rx, ry, rw) = _periodic_case(name, nodes, lmax)
    edges = g.nnz
    assert abs(edges / nodes - 30.0) < 3.0
    # structurally symmetric: every (r, s) has its (s, r)
    fwd = set(zip(g.rows[:2000].tolist(), g.cols[:2000].tolist()))
    allp = set(zip(g.rows.tolist(), g.cols.tolist()))
    assert all((s, r) in allp for r, s in fwd)
    conv = oeq.TensorProductConv(p, torch_op=True, deterministic=deterministic)
    index = cuda(g.rows, g.cols, g.sender_perm) if deterministic else cuda(g.rows, g.cols)
    xt, yt, wt, dzt = cuda(x, y, w, dz)
    z = conv.forward(xt, yt, wt, *index)
    dx, dy, dw = conv.backward_helper(xt, yt, wt, dzt, *index)
    torch.cuda.synchronize()
    conv.check_device_status()
    tol = REL_TOL[np.float32]
    assert rel_err(z.cpu().numpy(), z_ref) < tol
    assert rel_err(dx.cpu().numpy(), rx) < tol
    assert rel_err(dy.cpu().numpy(), ry) < tol
    assert rel_err(dw.cpu().numpy(), rw) < tol
    if deterministic:
        for _ in range(4):                       # the reference repeats five runs and wants equal bits
            z2 = conv.forward(xt, yt, wt, *index)
            dx2, dy2, dw2 = conv.backward_helper(xt, yt, wt, dzt, *index)
            assert torch.equal(z, z2) and torch.equal(dx, dx2) and torch.equal(dy, dy2) and torch.equal(dw, dw2)


@pytest.mark.parametrize("name", ["nequip_32", "mace_128"])
def test_deterministic_backward_in_edge_blocks(name, monkeypatch):
    """The receiver-order backward pass with scratch for only a part of the edges: it then runs block by block
    (receiver-order launch + row sum per block, later blocks adding into dX).  Same results as the oracle, the
    same bits run to run, and agreement with the scratch-free sender-order kernel."""
    monkeypatch.setenv("OEQ_B200_BWD_SCRATCH_MB", "1")      # 1 MiB of scratch: a few hundred rows per block
    monkeypatch.setenv("OEQ_B200_BWD_MIN_BLOCK", "1")
    if name == "mace_128":
        monkeypatch.setenv("OEQ_B200_PIPELINE_BLOCK_MB", "1")   # blocks of a few hundred edges are pipelined too:
        # each launch's helper warps sum the previous block while the consumers work on the current one
    p = problem_by_name(name)
    nodes = 300
    rows, cols = random_graph(nodes, 4000, seed=41)
    conv, (xt, yt, wt, dzt, index), (z, dx, dy, dw) = check_conv(p, nodes, rows, cols, 42, True)
    assert conv.internal.last_backward_launches() >= 6        # several blocks, two launches each
    dx2, dy2, dw2 = conv.backward_helper(xt, yt, wt, dzt, *index)
    assert torch.equal(dx, dx2) and torch.equal(dy, dy2) and torch.equal(dw, dw2)
    monkeypatch.setenv("OEQ_B200_BWD_SCRATCH_MB", "8192")
    monkeypatch.setenv("OEQ_B200_BWD_RECV", "0")               # a new handle without the receiver-order kernel
    old = oeq.TensorProductConv(p, torch_op=True, deterministic=True)
    dx3, dy3, dw3 = old.backward_helper(xt, yt, wt, dzt, *index)
    assert old.internal.last_backward_launches() == 1
    assert rel_err(dx3.cpu().numpy(), dx.cpu().numpy()) < 1e-5
    assert torch.equal(dy3, dy) or rel_err(dy3.cpu().numpy(), dy.cpu().numpy()) < 1e-5
    assert rel_err(dw3.cpu().numpy(), dw.cpu().numpy()) < 1e-5


def test_backward_without_scratch_uses_the_sender_order_kernel():
    """A caller of the C ABI that passes no workspace still gets the deterministic backward pass."""
    p = problem_by_name("nequip_32")
    nodes = 50
    rows, cols = random_graph(nodes, 600, seed=43)
    rows, cols, order, perm = orc.coord_graph(rows, cols)
    x, y, w, dz = conv_inputs(p, nodes, len(rows), 44)
    conv = oeq.TensorProductConv(p, torch_op=True, deterministic=True)
    xt, yt, wt, dzt, r, c, pm = cuda(x, y, w, dz, rows, cols, perm)
    dx, dy, dw = torch.empty_like(xt), torch.empty_like(yt), torch.empty_like(wt)
    conv.internal.backward(nodes, len(rows), xt.data_ptr(), yt.data_ptr(), wt.data_ptr(), dzt.data_ptr(), r.data_ptr(),
                           c.data_ptr(), pm.data_ptr(), dx.data_ptr(), dy.data_ptr(), dw.data_ptr(), 0, 0,
                           torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert conv.internal.last_backward_launches() == 1
    rx, ry, rw = orc.conv_backward(p, x, y, w, dz, rows, cols)
    assert rel_err(dx.cpu().numpy(), rx) < 1e-5 and rel_err(dy.cpu().numpy(), ry) < 1e-5
    assert rel_err(dw.cpu().numpy(), rw) < 1e-5
