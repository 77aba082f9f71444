"""Benchmark of the fused graph convolution (forward + backward), edges per second.

    python bench.py --gpus N --steps K --warmup W            # this library, N GPUs of one node
    python bench.py --impl reference --steps K --warmup W    # CPU baseline on the host cores

Workloads (``--workload``):
  mace_large  MACE-large irreps 128x(0e+1o+2e+3o), spherical harmonics to l=3, periodic radius
              graph of 200 000 nodes at mean degree 30 (about 6 M edges); deterministic variant.
              The default: it is the configuration the headline metric is quoted on.
  mace        MACE irreps 128x(0e+1o+2e), harmonics to l=3, 100 000 nodes at degree 30.
  nequip      Nequip irreps 32x(0e+1o+2e), harmonics to l=2, 20 000 nodes at degree 40.

One JSON line is printed by rank 0.  ``value`` is edges processed per second by the whole job
for one forward plus one backward pass with inputs resident in HBM; ``e2e`` is the same with
every input copied from pinned host memory and every output copied back inside the timed
region.  For N > 1 the graph is split by receiver range (strong scaling): sender features are
exchanged before the forward kernel and their gradients after the backward kernels, both inside
the timed region (only halo rows -- senders owned by another rank -- move).

Beside the headline the line carries ``parity`` (rows of Z, dX, dY, dW of the benchmark's own inputs
checked against the float64 CPU oracle on rank 0, outside every timed region), ``peaks`` (matmul peaks
measured in this run), ``secondary`` (the other configurations: batch 'uvu', Nequip convolution,
'uvw' in FP32 and FP64) and ``random_numbering`` (the headline workload with random node ids).
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

WORKLOADS = {
    "mace_large": dict(in1="128x0e+128x1o+128x2e+128x3o", in2="1x0e+1x1o+1x2e+1x3o",
                       out="128x0e+128x1o+128x2e+128x3o", lmax=3, nodes=200_000, degree=30.0,
                       cpu_sample_edges=20_000),
    "mace": dict(in1="128x0e+128x1o+128x2e", in2="1x0e+1x1o+1x2e+1x3o", out="128x0e+128x1o+128x2e", lmax=3,
                 nodes=100_000, degree=30.0, cpu_sample_edges=50_000),
    "nequip": dict(in1="32x0e+32x1o+32x2e", in2="0e+1o+2e", out="32x0e+32x1o+32x2e", lmax=2, nodes=20_000,
                   degree=40.0, cpu_sample_edges=100_000),
}


# DRAM read+write bytes per edge of the deterministic backward pass (all its launches), from an ncu
# capture (dram__bytes_read.sum + dram__bytes_write.sum) of a small case of the same workload; the
# capture's case and date are named in the line ("traffic_from").  Only the per-edge arrays scale with
# the edge count, so this is an estimate for other sizes, and it is refreshed when the kernels change.
NCU_BWD_DRAM = {   # (workload, numbering) -> (bytes per edge, "what was captured")
    ("mace_large", "morton"): (12.76e9 / 299832, "ncu dram__bytes_read.sum + dram__bytes_write.sum over all launches of one "
                                                  "backward pass, 10 000 nodes / 299 832 edges, captured 2026-11-25 "
                                                  "(profiles/conv_backward_receiver_order_mace_large.md)"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mace_large", choices=sorted(WORKLOADS))
    ap.add_argument("--numbering", default="morton", choices=["morton", "random"],
                    help="node numbering of the synthetic graph (spatially sorted, or random)")
    ap.add_argument("--nodes", type=int, default=None, help="override the node count (profiling on small cases)")
    ap.add_argument("--variant", default="deterministic", choices=["deterministic", "atomic"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the other configurations, the matmul peaks and the random-numbering run")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--slab-edges", type=int, default=1 << 18,
                    help="edges per slab of the streamed host-tensor path (end-to-end measurement)")
    ap.add_argument("--seed", type=int, default=11111)
    return ap.parse_args()


def make_problem(spec):
    import openequivariance_b200 as oeq
    return oeq.ChannelwiseTPP(spec["in1"], spec["in2"], spec["out"])


def algorithmic_bytes(problem, nodes, edges, elem=4, x_rows=None):
    """Compulsory HBM traffic of one pass: every edge array once, every node array once,
    int64 receiver/sender (and the sender-order permutation in the backward pass).  ``x_rows``:
    rows of X / dX a shard touches (owned + halo) when that differs from its output rows."""
    x, y, z, w = problem.irreps_in1.dim, problem.irreps_in2.dim, problem.irreps_out.dim, problem.weight_numel
    xr = nodes if x_rows is None else x_rows
    fwd = edges * ((w + y) * elem + 16) + (xr * x + nodes * z) * elem
    bwd = edges * (2 * (w + y) * elem + 24) + (2 * xr * x + nodes * z) * elem
    return fwd, bwd


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """SM clock and throttle reasons of one GPU, sampled by `nvidia-smi` in a child process.  The sampler is started
    before the warm-up steps (the tool needs a moment to come up) and every sample carries the tool's time stamp;
    `stop` keeps the samples that fall inside the marked region.  A timed region shorter than a sampling period
    (multi-GPU runs: 10 steps take 0.1 s) falls back to the samples taken since the warm-up began, under the same
    load, and says so in `window`."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu_index, self.proc = gpu_index, None
        self.started = self.begin = self.end = None

    def start(self):
        import datetime
        self.started = datetime.datetime.now()
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def mark_begin(self):
        import datetime
        self.begin = datetime.datetime.now()

    def mark_end(self):
        import datetime
        self.end = datetime.datetime.now()

    @staticmethod
    def parse(text):
        """[(time stamp or None, sm MHz, max MHz, [active throttle reasons])] from the tool's CSV lines."""
        import datetime
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in text.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm, smax = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
            except ValueError:
                stamp = None
            rows.append((stamp, sm, smax, [n for n, flag in zip(names, parts[5:9]) if flag.lower().startswith("active")]))
        return rows

    def summarise(self, rows):
        inside = [r for r in rows if r[0] is not None and self.begin and self.end and self.begin <= r[0] <= self.end]
        window = "timed region"
        if not inside:
            inside = [r for r in rows if r[0] is None or self.started is None or r[0] >= self.started]
            window = "warm-up and timed steps (the timed region is shorter than a sampling period)"
        sm = [r[1] for r in inside]
        reasons = sorted({name for r in inside for name in r[3]})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": inside[-1][2] if inside else None,
                "reasons": reasons, "samples": len(sm), "window": window}

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"], "samples": 0}
        if self.end is None:
            self.mark_end()
        time.sleep(0.12)             # let the sample that covers the end of the region arrive
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        return self.summarise(self.parse(out))


def build_graph(spec, args, numbering=None):
    from openequivariance_b200.graph import periodic_radius_graph
    nodes = args.nodes or spec["nodes"]
    return periodic_radius_graph(nodes, spec["degree"], seed=args.seed, numbering=numbering or args.numbering)


# --------------------------------------------------------------------------- seeded inputs
#
# Every array of the workload is a function of (seed, stream, row): rows are drawn in fixed-size slices,
# each from a generator seeded by the slice index, so any rank -- and the parity check -- can reproduce any
# row of any array without communication and without trusting the exchange it is checking.

SLICE_ROWS = 1 << 14
STREAM_X, STREAM_DZ, STREAM_W = 1, 2, 3


def _slice_seed(seed, stream, index):
    return (seed * 1_000_003 + stream * 100_000_007 + index) % (1 << 62)


def seeded_rows(torch, seed, stream, row_lo, row_hi, width, device):
    """Rows [row_lo, row_hi) of the N(0,1) array `stream`, as a device tensor."""
    out = torch.empty((row_hi - row_lo, width), device=device, dtype=torch.float32)
    gen = torch.Generator(device=device)
    pos = row_lo
    while pos < row_hi:
        index, off = divmod(pos, SLICE_ROWS)
        take = min(SLICE_ROWS - off, row_hi - pos)
        gen.manual_seed(_slice_seed(seed, stream, index))
        block = torch.randn((SLICE_ROWS, width), device=device, dtype=torch.float32, generator=gen)
        out[pos - row_lo:pos - row_lo + take] = block[off:off + take]
        pos += take
    return out


def seeded_rows_at(torch, seed, stream, ids, width, device):
    """The rows `ids` (any order, repeats allowed) of the same array, regenerated slice by slice."""
    ids = np.asarray(ids, dtype=np.int64)
    out = torch.empty((len(ids), width), device=device, dtype=torch.float32)
    gen = torch.Generator(device=device)
    for index in np.unique(ids // SLICE_ROWS):
        sel = np.nonzero(ids // SLICE_ROWS == index)[0]
        gen.manual_seed(_slice_seed(seed, stream, int(index)))
        block = torch.randn((SLICE_ROWS, width), device=device, dtype=torch.float32, generator=gen)
        out[torch.from_numpy(sel).to(device)] = block[torch.from_numpy(ids[sel] - index * SLICE_ROWS).to(device)]
    return out


# --------------------------------------------------------------------------- CPU baseline

def cpu_baseline(problem, spec, graph, steps, warmup, seed):
    """The unfused CPU path (per-instruction einsum as e3nn evaluates it, gather before, scatter-sum
    after; forward + backward by autograd) on a bounded sample of the workload's edges, float32,
    all host threads."""
    import torch
    from oracle import tp_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample = min(spec["cpu_sample_edges"], graph.nnz)
    rows = graph.rows[:sample]
    senders, cols = np.unique(graph.cols[:sample], return_inverse=True)
    n_recv = int(rows.max()) + 1 if sample else 0
    n_send = len(senders)
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(max(n_send, n_recv), problem.irreps_in1.dim, generator=gen)
    y = torch.randn(sample, problem.irreps_in2.dim, generator=gen)
    w = torch.randn(sample, problem.weight_numel, generator=gen)
    dz = torch.randn(max(n_send, n_recv), problem.irreps_out.dim, generator=gen)
    r, c = torch.from_numpy(rows.copy()), torch.from_numpy(cols.astype(np.int64))
    chunk = 5000

    def step():
        x.grad = None
        x.requires_grad_(True)
        for lo in range(0, sample, chunk):
            hi = min(lo + chunk, sample)
            yc, wc = y[lo:hi].requires_grad_(True), w[lo:hi].requires_grad_(True)
            z = orc.conv_torch(problem, x, yc, wc, r[lo:hi], c[lo:hi], fold_second_input=True)
            z.backward(dz)

    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        step()
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    per_step = sum(times) / len(times)
    return {"value": sample / per_step, "unit": "edges/s", "cores": cores, "kind": "port",
            "sample": f"first {sample} receiver-sorted edges of the workload in chunks of {chunk}, "
                      f"{warmup} warm-up and {len(times)} timed passes, torch CPU float32 (gather, per-instruction "
                      f"contraction with the second input folded into the Clebsch-Gordan tensor, index_add), "
                      f"autograd backward",
            "ms_per_step": per_step * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    spec = WORKLOADS[args.workload]
    problem = make_problem(spec)
    graph = build_graph(spec, args)
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    base = cpu_baseline(problem, spec, graph, steps, warmup, args.seed)
    line = {
        "impl": "reference", "metric": "conv_fwd_bwd_edges_per_s", "value": base["value"], "unit": "edges/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": base["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, spec, graph),
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, spec, graph, numbering=None):
    return {"workload": f"{args.workload}: fused conv uvu {spec['in1']} x {spec['in2']} -> l_out<={spec['lmax']}, "
                        f"{args.variant}, fwd+bwd",
            "nodes": graph.node_count, "edges": graph.nnz, "mean_degree": graph.nnz / max(1, graph.node_count),
            "numbering": numbering or args.numbering, "graph": "uniform points in a periodic unit cube, radius cutoff",
            "l2": "inputs larger than L2 (no flush needed)" if graph.nnz > 200_000 else "small case",
            "parallelism": f"receiver-range shards x{args.gpus}" if args.gpus > 1 else "single GPU"}


# --------------------------------------------------------------------------- parity on the benchmark's inputs

def parity_check(torch, args, spec, problem, graph, conv, plan, y, w, outputs, device, rows_wanted=64):
    """Rows of the step's results against the float64 oracle, on rank 0, outside every timed region.

    Receivers: every edge of a receiver is on its owner's rank, so Z, dY and dW rows are checked from the
    rank's own Y and W and from X rows regenerated from the seed (not taken from the exchange).  Senders:
    the edges a node sends may live on any rank; their W and dZ rows are regenerated from the seed and Y
    from the graph's edge vectors, so dX of nodes in other ranks' halos checks the return exchange."""
    from oracle import tp_oracle as orc
    from openequivariance_b200.graph import spherical_harmonics
    z, dx, dy, dw = outputs
    seed = args.seed
    xd, zd, wn = problem.irreps_in1.dim, problem.irreps_out.dim, problem.weight_numel
    rng = np.random.default_rng(seed)
    node_lo, owned, e_lo = plan.node_lo, plan.owned, plan.edge_lo
    half = rows_wanted // 2

    def rel(got, want):
        want = np.asarray(want, dtype=np.float64)
        return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / max(np.abs(want).max(), 1e-30))

    # receivers: those with a sender in the halo first, then random ones
    local_rows, local_cols = plan.local_rows, plan.local_cols
    with_halo = np.unique(local_rows[local_cols >= owned])
    pick = list(rng.choice(with_halo, size=min(half, len(with_halo)), replace=False)) if len(with_halo) else []
    pick += list(rng.choice(owned, size=min(rows_wanted - len(pick), owned), replace=False))
    recv = np.unique(np.asarray(pick, dtype=np.int64))
    lo = np.searchsorted(local_rows, recv, side="left")
    hi = np.searchsorted(local_rows, recv, side="right")
    eidx = np.concatenate([np.arange(a, b) for a, b in zip(lo, hi)]) if len(recv) else np.zeros(0, np.int64)
    out = {"rows": int(len(recv)), "edges": int(len(eidx))}
    if len(eidx):
        glob_cols = graph.cols[e_lo + eidx]
        senders, cols_small = np.unique(glob_cols, return_inverse=True)
        rows_small = np.searchsorted(recv, local_rows[eidx])
        n = max(len(senders), len(recv))
        x_s = np.zeros((n, xd), np.float32)
        x_s[:len(senders)] = seeded_rows_at(torch, seed, STREAM_X, senders, xd, device).cpu().numpy()
        ei = torch.from_numpy(eidx).to(device)
        y_s, w_s = y[ei].cpu().numpy(), w[ei].cpu().numpy()
        dz_s = np.zeros((n, zd), np.float32)
        dz_s[:len(recv)] = seeded_rows_at(torch, seed, STREAM_DZ, node_lo + recv, zd, device).cpu().numpy()
        z_ref = orc.conv_forward(problem, x_s, y_s, w_s, rows_small, cols_small)[:len(recv)]
        _, dy_ref, dw_ref = orc.conv_backward(problem, x_s, y_s, w_s, dz_s, rows_small, cols_small)
        ri = torch.from_numpy(recv).to(device)
        out["z_rel"] = rel(z[ri].cpu().numpy(), z_ref)
        out["dy_rel"] = rel(dy[ei].cpu().numpy(), dy_ref)
        out["dw_rel"] = rel(dw[ei].cpu().numpy(), dw_ref)

    # senders: nodes that other ranks read (their dX sums contributions that came back), then random ones
    shared = np.unique(np.concatenate(plan.send_rows)) if plan.send_rows is not None and len(plan.send_rows) else np.zeros(0, np.int64)
    pick = list(rng.choice(shared, size=min(half, len(shared)), replace=False)) if len(shared) else []
    pick += list(rng.choice(owned, size=min(rows_wanted - len(pick), owned), replace=False))
    send = np.unique(np.asarray(pick, dtype=np.int64))
    by_sender = graph.cols[graph.sender_perm]                     # senders in sender order (non-decreasing)
    lo = np.searchsorted(by_sender, node_lo + send, side="left")
    hi = np.searchsorted(by_sender, node_lo + send, side="right")
    ge = np.concatenate([graph.sender_perm[a:b] for a, b in zip(lo, hi)]) if len(send) else np.zeros(0, np.int64)
    out["sender_rows"], out["sender_edges"] = int(len(send)), int(len(ge))
    if len(ge):
        receivers, rows_small = np.unique(graph.rows[ge], return_inverse=True)
        cols_small = np.searchsorted(send, graph.cols[ge] - node_lo)
        n = max(len(send), len(receivers))
        x_s = np.zeros((n, xd), np.float32)
        x_s[:len(send)] = seeded_rows_at(torch, seed, STREAM_X, node_lo + send, xd, device).cpu().numpy()
        dz_s = np.zeros((n, zd), np.float32)
        dz_s[:len(receivers)] = seeded_rows_at(torch, seed, STREAM_DZ, receivers, zd, device).cpu().numpy()
        w_s = seeded_rows_at(torch, seed, STREAM_W, ge, wn, device).cpu().numpy()
        vec = torch.from_numpy(graph.vectors[ge]).to(device=device, dtype=torch.float32)
        y_s = spherical_harmonics(spec["lmax"], vec).contiguous().cpu().numpy()
        dx_ref = orc.conv_backward(problem, x_s, y_s, w_s, dz_s, rows_small, cols_small)[0][:len(send)]
        si = torch.from_numpy(send).to(device)
        out["dx_rel"] = rel(dx[si].cpu().numpy(), dx_ref)
    out["tolerance"] = 1e-5
    out["ok"] = all(out.get(k, 0.0) < 1e-5 for k in ("z_rel", "dx_rel", "dy_rel", "dw_rel"))
    return out


# --------------------------------------------------------------------------- GPU benchmark

def matmul_peaks(torch):
    """Dense matmul peaks of this GPU (torch.matmul, best of 10, CUDA events): the denominators of the
    'uvw' tensor-pipe and FP64 fractions.  A peak probe, not a product path."""
    def one(dtype, n, tf32):
        old = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = tf32
        try:
            a = torch.randn(n, n, device="cuda", dtype=dtype)
            b = torch.randn(n, n, device="cuda", dtype=dtype)
            for _ in range(3):
                a @ b
            torch.cuda.synchronize()
            best = float("inf")
            for _ in range(10):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                a @ b
                e.record()
                torch.cuda.synchronize()
                best = min(best, s.elapsed_time(e))
            return 2 * n ** 3 / best / 1e9
        finally:
            torch.backends.cuda.matmul.allow_tf32 = old
    return {"tf32_tflops": one(torch.float32, 8192, True), "fp32_tflops": one(torch.float32, 8192, False),
            "fp64_tflops": one(torch.float64, 4096, False),
            "how": "torch.matmul 8192^3 (FP64: 4096^3), best of 10, CUDA events; TF32 with allow_tf32=True"}


def conv_case(torch, args, spec, workload, device, variant, numbering, nodes=None, steps=5, warmup=3):
    """Forward + backward kernel times of one single-GPU convolution workload (inputs resident)."""
    import openequivariance_b200 as oeq
    from openequivariance_b200.graph import periodic_radius_graph, spherical_harmonics
    problem = make_problem(spec)
    g = periodic_radius_graph(nodes or spec["nodes"], spec["degree"], seed=args.seed, numbering=numbering)
    det = variant == "deterministic"
    conv = oeq.TensorProductConv(problem, torch_op=True, deterministic=det)
    idx = [torch.from_numpy(a).to(device) for a in ((g.rows, g.cols, g.sender_perm) if det else (g.rows, g.cols))]
    gen = torch.Generator(device=device).manual_seed(args.seed)
    x = torch.randn(g.node_count, problem.irreps_in1.dim, device=device, generator=gen)
    dz = torch.randn(g.node_count, problem.irreps_out.dim, device=device, generator=gen)
    y = spherical_harmonics(spec["lmax"], torch.from_numpy(g.vectors).to(device=device, dtype=torch.float32)).contiguous()
    w = torch.empty(g.nnz, problem.weight_numel, device=device)
    for lo in range(0, g.nnz, 1 << 19):
        w[lo:lo + (1 << 19)].normal_(generator=gen)
    small = g.nnz * (problem.weight_numel + problem.irreps_in2.dim) * 4 < (256 << 20)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if small else None
    tf, tb = [], []
    for i in range(warmup + steps):
        if flush is not None:
            flush.zero_()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        z = conv._forward_impl(x, y, w, *idx)
        e[1].record()
        out = conv._backward_impl(x, y, w, dz, *idx)
        e[2].record()
        torch.cuda.synchronize()
        del z, out
        if i >= warmup:
            tf.append(e[0].elapsed_time(e[1]))
            tb.append(e[1].elapsed_time(e[2]))
    conv.check_device_status()
    fwd, bwd = statistics.median(tf), statistics.median(tb)
    fb, bb = algorithmic_bytes(problem, g.node_count, g.nnz)
    peak, _ = measured_peak()
    res = {"workload": workload, "variant": variant, "numbering": numbering, "nodes": g.node_count, "edges": g.nnz,
           "forward_ms": fwd, "backward_ms": bwd, "edges_per_s": g.nnz / ((fwd + bwd) * 1e-3),
           "hbm_frac_forward": fb / (fwd * 1e-3) / 1e9 / peak, "hbm_frac_backward": bb / (bwd * 1e-3) / 1e9 / peak,
           "hbm_frac_fwd_bwd": (fb + bb) / ((fwd + bwd) * 1e-3) / 1e9 / peak,
           "l2": "flushed before every step" if small else "inputs larger than L2"}
    del conv, x, y, w, dz, idx
    torch.cuda.empty_cache()
    return res


def second_derivative_case(torch, device, steps=10, warmup=3, batch=50_000):
    """Second derivatives of the batch 'uvu' product (MACE irreps, 50 000 rows): the one-pass kernel against the
    composition of four backward and three forward launches that the reference uses."""
    import openequivariance_b200 as oeq
    p = oeq.ChannelwiseTPP("128x0e+128x1o+128x2e", "1x0e+1x1o+1x2e+1x3o", "128x0e+128x1o+128x2e")
    tp = oeq.TensorProduct(p, torch_op=True)
    gen = torch.Generator(device=device).manual_seed(3)
    mk = lambda n: torch.randn(batch, n, device=device, generator=gen)
    x, y, w, dz = mk(p.irreps_in1.dim), mk(p.irreps_in2.dim), mk(p.weight_numel), mk(p.irreps_out.dim)
    ex, ey, ew = mk(p.irreps_in1.dim), mk(p.irreps_in2.dim), mk(p.weight_numel)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def composed():
        a = tp.backward_helper(ex, ey, w, dz)
        b = tp.backward_helper(x, y, ew, dz)
        c = tp.backward_helper(ex, y, w, dz)
        d = tp.backward_helper(x, ey, w, dz)
        gz = tp(ex, y, w) + tp(x, ey, w) + tp(x, y, ew)
        return a[0] + b[0], a[1] + b[1], c[2] + d[2], gz

    def timed(fn):
        ts = []
        for i in range(warmup + steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if i >= warmup:
                ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    fused = timed(lambda: tp._double_backward_impl(x, y, w, dz, ex, ey, ew))
    comp = timed(composed)
    tp.check_device_status()
    xd, yd, zd, wn = p.irreps_in1.dim, p.irreps_in2.dim, p.irreps_out.dim, p.weight_numel
    bytes_ = batch * (3 * xd + 3 * yd + 3 * wn + 2 * zd) * 4          # seven arrays in, four out
    peak, _ = measured_peak()
    return {"one_pass_ms": fused, "composed_ms": comp, "rows_per_s": batch / (fused * 1e-3),
            "hbm_frac_one_pass": bytes_ / (fused * 1e-3) / 1e9 / peak, "algorithmic_bytes": bytes_}


def conv_second_derivative_case(torch, args, device, nodes=20_000, degree=40.0, steps=5, warmup=3):
    """Second derivatives of the deterministic convolution (MACE irreps to l=2, 20 000 nodes x ~40 neighbours): two
    fused launches (plus the row sum) against the four backward and three forward launches the reference composes."""
    import openequivariance_b200 as oeq
    from openequivariance_b200.graph import periodic_radius_graph
    p = oeq.ChannelwiseTPP("128x0e+128x1o+128x2e", "1x0e+1x1o+1x2e+1x3o", "128x0e+128x1o+128x2e")
    g = periodic_radius_graph(nodes, degree, seed=args.seed, numbering="morton")
    conv = oeq.TensorProductConv(p, torch_op=True, deterministic=True)
    idx = [torch.from_numpy(a).to(device) for a in (g.rows, g.cols, g.sender_perm)]
    gen = torch.Generator(device=device).manual_seed(args.seed + 1)
    n, e = g.node_count, g.nnz
    mk = lambda r, c: torch.randn(r, c, device=device, generator=gen)
    xd, yd, zd, wn = p.irreps_in1.dim, p.irreps_in2.dim, p.irreps_out.dim, p.weight_numel
    x, y, w, dz = mk(n, xd), mk(e, yd), mk(e, wn), mk(n, zd)
    ex, ey, ew = mk(n, xd), mk(e, yd), mk(e, wn)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def composed():
        a = conv._backward_impl(ex, ey, w, dz, *idx)
        b = conv._backward_impl(x, y, ew, dz, *idx)
        c = conv._backward_impl(ex, y, w, dz, *idx)
        d = conv._backward_impl(x, ey, w, dz, *idx)
        gz = conv._forward_impl(ex, y, w, *idx) + conv._forward_impl(x, ey, w, *idx) + conv._forward_impl(x, y, ew, *idx)
        return a[0] + b[0], a[1] + b[1], c[2] + d[2], gz

    def timed(fn):
        ts, out = [], None
        for i in range(warmup + steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = fn()
            b.record()
            torch.cuda.synchronize()
            if i >= warmup:
                ts.append(a.elapsed_time(b))
        return statistics.median(ts), out

    fused_ms, got = timed(lambda: conv._double_backward_impl(x, y, w, dz, ex, ey, ew, *idx))
    comp_ms, want = timed(composed)
    conv.check_device_status()
    err = max(float((a - b).abs().max() / b.abs().max()) for a, b in zip(got, want))
    # per edge: Y, W and their cotangents read twice (once per launch), GY, GW written; per node: X, EX twice, dZ, GX, GdZ
    bytes_ = (e * (4 * yd + 4 * wn + yd + wn) + n * (4 * xd + zd + xd + zd)) * 4
    peak, _ = measured_peak()
    return {"nodes": n, "edges": e, "fused_ms": fused_ms, "composed_ms": comp_ms,
            "edges_per_s": e / (fused_ms * 1e-3), "max_rel_diff_vs_composed": err,
            "hbm_frac_fused": bytes_ / (fused_ms * 1e-3) / 1e9 / peak, "algorithmic_bytes": bytes_}


def uvw_conv_case(torch, args, device, nodes=20_000, degree=40.0, steps=5, warmup=3):
    """Shared-weight 'uvw' convolution (64x(0e+1o+2e), harmonics to l=2) on a Nequip-sized graph: the unit-weight
    edge sum over the edges, then the dense contraction over the nodes; forward and backward (all gradients)."""
    import openequivariance_b200 as oeq
    from openequivariance_b200.graph import periodic_radius_graph, spherical_harmonics
    p = oeq.FullyConnectedTPProblem("64x0e+64x1o+64x2e", "0e+1o+2e", "64x0e+64x1o+64x2e")
    g = periodic_radius_graph(nodes, degree, seed=args.seed, numbering="morton")
    conv = oeq.TensorProductConv(p, torch_op=True, deterministic=True)
    idx = [torch.from_numpy(a).to(device) for a in (g.rows, g.cols, g.sender_perm)]
    gen = torch.Generator(device=device).manual_seed(args.seed)
    x = torch.randn(g.node_count, p.irreps_in1.dim, device=device, generator=gen)
    dz = torch.randn(g.node_count, p.irreps_out.dim, device=device, generator=gen)
    w = torch.randn(p.weight_numel, device=device, generator=gen) / 8
    y = spherical_harmonics(2, torch.from_numpy(g.vectors).to(device=device, dtype=torch.float32)).contiguous()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    tf, tb = [], []
    for i in range(warmup + steps):
        flush.zero_()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        z = conv.forward(x, y, w, *idx)
        e[1].record()
        out = conv.backward_helper(x, y, w, dz, *idx)
        e[2].record()
        torch.cuda.synchronize()
        del z, out
        if i >= warmup:
            tf.append(e[0].elapsed_time(e[1]))
            tb.append(e[1].elapsed_time(e[2]))
    # through autograd the edge sum saved by the forward pass is re-used (no recomputation)
    ta = []
    xg, yg, wg = (t.clone().requires_grad_(True) for t in (x, y, w))
    for i in range(warmup + steps):
        flush.zero_()
        z = conv.forward(xg, yg, wg, *idx)
        e = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        e[0].record()
        grads = torch.autograd.grad(z, (xg, yg, wg), dz)
        e[1].record()
        torch.cuda.synchronize()
        del z, grads
        if i >= warmup:
            ta.append(e[0].elapsed_time(e[1]))
    conv.check_device_status()
    fwd, bwd = statistics.median(tf), statistics.median(tb)
    return {"nodes": g.node_count, "edges": g.nnz, "forward_ms": fwd, "backward_ms": bwd,
            "backward_autograd_ms": statistics.median(ta),
            "edges_per_s": g.nnz / ((fwd + bwd) * 1e-3),
            "note": "backward_ms is the stand-alone backward entry point, which recomputes the edge sum; backward_autograd_ms re-uses the one the forward pass saved; weights applied once per node, not per edge"}


def secondary_block(torch, args, device, peaks):
    """The other configurations, measured in this process with the same protocol (CUDA events, L2 flushed or
    inputs larger than L2): batch 'uvu' (50 000 rows), Nequip convolution both variants, 'uvw' FP32 / FP64."""
    from openequivariance_b200 import bench_tp
    peak, _ = measured_peak()
    out = {}
    r = bench_tp.measure("uvu_mace", "f32", steps=10, warmup=3)
    out["batch_uvu_mace_50k"] = {
        "rows_per_s_fwd_bwd": r["rows_per_s_fwd_bwd"], "forward_ms": r["forward_ms"], "backward_ms": r["backward_ms"],
        "hbm_frac_forward": r["forward_GBps"] / peak, "hbm_frac_backward": r["backward_GBps"] / peak,
        "hbm_frac_fwd_bwd": (r["algorithmic_bytes"]["forward"] + r["algorithmic_bytes"]["backward"])
                            / ((r["forward_ms"] + r["backward_ms"]) * 1e-3) / 1e9 / peak}
    for variant in ("deterministic", "atomic"):
        out[f"conv_nequip_{variant}"] = conv_case(torch, args, WORKLOADS["nequip"], "nequip", device, variant, "morton")
    out["conv_mace_large_atomic_20k_nodes"] = conv_case(torch, args, WORKLOADS["mace_large"], "mace_large", device,
                                                        "atomic", "morton", nodes=20_000)
    out["batch_uvu_mace_50k_second_derivatives"] = second_derivative_case(torch, device)
    out["conv_uvu_mace_20k_nodes_second_derivatives"] = conv_second_derivative_case(torch, args, device)
    out["conv_uvw_fc64_shared_20k_nodes"] = uvw_conv_case(torch, args, device)
    for dt, pk in (("f32", peaks["tf32_tflops"]), ("f64", peaks["fp64_tflops"])):
        r = bench_tp.measure("uvw_fc", dt, steps=10, warmup=3)
        out[f"batch_uvw_fc_100k_{dt}"] = {
            "forward_ms": r["forward_ms"], "backward_ms": r["backward_ms"], "rows_per_s_fwd_bwd": r["rows_per_s_fwd_bwd"],
            "logical_tflops_forward": r["forward_contraction_TFLOPs"],
            "logical_tflops_fwd_bwd": r["fwd_bwd_contraction_TFLOPs"],
            # FP32 runs as 3xTF32: three tensor-core products per logical one
            "frac_of_measured_peak_forward": r["forward_contraction_TFLOPs"] * (3 if dt == "f32" else 1) / pk,
            "frac_of_measured_peak_fwd_bwd": r["fwd_bwd_contraction_TFLOPs"] * (3 if dt == "f32" else 1) / pk,
            "peak": "tf32_tflops (issued = 3 x logical)" if dt == "f32" else "fp64_tflops"}
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    import openequivariance_b200 as oeq
    from openequivariance_b200.dist import ShardedTensorProductConv
    from openequivariance_b200.graph import spherical_harmonics

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    spec = WORKLOADS[args.workload]
    problem = make_problem(spec)
    det = args.variant == "deterministic"
    if not det and world > 1:
        raise SystemExit("the sharded benchmark runs the deterministic variant")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def measure(numbering, steps, with_parity, with_e2e):
        """One workload instance: set-up, warm-up, timed steps, then (untimed) parity and the host-tensor step."""
        graph = build_graph(spec, args, numbering)
        nodes, edges = graph.node_count, graph.nnz
        if det:
            conv = ShardedTensorProductConv(problem, graph.rows, graph.cols, nodes, device=device)
            plan = conv.plan
            e_lo, e_hi, owned = plan.edge_lo, plan.edge_hi, plan.owned
        else:
            conv = oeq.TensorProductConv(problem, torch_op=True, deterministic=False)
            plan = None
            e_lo, e_hi, owned = 0, edges, nodes
            rows_d = torch.from_numpy(graph.rows).to(device)
            cols_d = torch.from_numpy(graph.cols).to(device)
        local_edges = e_hi - e_lo
        node_lo = plan.node_lo if plan is not None else 0
        x = seeded_rows(torch, args.seed, STREAM_X, node_lo, node_lo + owned, problem.irreps_in1.dim, device)
        if det and world > 1:
            # node features live in the rank's gather buffer: the halo exchange copies no owned rows
            x = conv.owned_buffer(x.shape[1], x.dtype).copy_(x)
        dz = seeded_rows(torch, args.seed, STREAM_DZ, node_lo, node_lo + owned, problem.irreps_out.dim, device)
        vec = torch.from_numpy(graph.vectors[e_lo:e_hi]).to(device=device, dtype=torch.float32)
        y = spherical_harmonics(spec["lmax"], vec).contiguous()
        del vec
        w = seeded_rows(torch, args.seed, STREAM_W, e_lo, e_hi, problem.weight_numel, device)

        def step():
            if det:
                return conv.forward_backward(x, y, w, dz)
            z = conv.forward(x, y, w, rows_d, cols_d)
            dx, dy, dw = conv.backward_helper(x, y, w, dz, rows_d, cols_d)
            return z, dx, dy, dw

        sampler = ClockSampler(local_rank if os.environ.get("CUDA_VISIBLE_DEVICES") is None else 0)
        sampler.start()
        for _ in range(max(3, args.warmup)):
            out = step()
            del out
        barrier()

        # -- timed region: device events per step, fwd and bwd passes timed separately on the rank's stream
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
        inner = conv.conv if det else conv
        barrier()
        sampler.mark_begin()
        t0 = time.perf_counter()
        for k in range(steps):
            if det:
                x_full = conv.gather_senders(x)
                ev[k][0].record()
                z = conv.local_forward(x_full, y, w)
                ev[k][1].record()
                dx_all, dy, dw = conv.local_backward(x_full, y, w, dz)
                ev[k][2].record()
                dx = conv.scatter_sender_grads(dx_all)
                ev[k][3].record()
                del z, dx_all, dy, dw, dx
            else:
                ev[k][0].record()
                z = conv.forward(x, y, w, rows_d, cols_d)
                ev[k][1].record()
                dx, dy, dw = conv.backward_helper(x, y, w, dz, rows_d, cols_d)
                ev[k][2].record()
                ev[k][3].record()
                del z, dx, dy, dw
        barrier()
        elapsed = time.perf_counter() - t0
        sampler.mark_end()
        clocks = sampler.stop()
        inner.check_device_status()
        launches_bwd = max(1, inner.internal.last_backward_launches())

        fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
        bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
        t = torch.tensor([elapsed, fwd_ms, bwd_ms], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed, fwd_ms_max, bwd_ms_max = t.tolist()
        res = {"graph": graph, "conv": conv, "plan": plan, "inner": inner, "elapsed": elapsed, "steps": steps,
               "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "fwd_ms_max": fwd_ms_max, "bwd_ms_max": bwd_ms_max,
               "clocks": clocks, "local_edges": local_edges, "owned": owned, "launches_bwd": launches_bwd,
               "halo_fraction": (plan.halo.size / max(1, plan.owned)) if plan is not None else 0.0}

        if with_parity and det:
            outputs = step()
            torch.cuda.synchronize()
            if rank == 0:
                res["parity"] = parity_check(torch, args, spec, problem, graph, conv, plan, y, w, outputs, device)
            del outputs
            barrier()
        if with_e2e:
            # the resident arrays are handed over: the host-tensor path pins what it needs of them and lets them go,
            # so that its own device buffers do not have to be carved out of a full allocator
            resident = [x, y, w, dz]
            del x, y, w, dz
            res["e2e"] = run_e2e(args, torch, dist, world, device, conv, det, resident, edges, local_edges,
                                 (rows_d, cols_d) if not det else None, graph=graph)
            del resident
        else:
            del x, y, w, dz
        return res

    main = measure(args.numbering, args.steps, not args.no_parity, not args.no_e2e)
    graph, plan, inner = main["graph"], main["plan"], main["inner"]
    nodes, edges = graph.node_count, graph.nnz
    ms_per_step = main["elapsed"] / args.steps * 1e3
    value = edges / (main["elapsed"] / args.steps)
    fwd_ms, bwd_ms = main["fwd_ms"], main["bwd_ms"]

    # -- roofline of the dominant pass (backward), rank 0's launches
    fb, bb = algorithmic_bytes(problem, main["owned"] if world > 1 else nodes, main["local_edges"],
                               x_rows=plan.local_nodes if (plan is not None and world > 1) else None)
    peak, peak_kind = measured_peak()
    traffic, traffic_from = None, None
    if (args.workload, args.numbering) in NCU_BWD_DRAM and world == 1 and det:
        per_edge, traffic_from = NCU_BWD_DRAM[(args.workload, args.numbering)]
        traffic = per_edge * main["local_edges"]
    info_b, info_f = inner.internal.launch_info(1), inner.internal.launch_info(0)
    launches_bwd = main["launches_bwd"]
    roofline = {"bound": "hbm", "kernel": "conv backward pass (oeq_uvu_kernel receiver order + oeq_sum_sender_rows per edge block)"
                if launches_bwd > 1 else "oeq_uvu_kernel (conv backward)",
                "achieved": bb / (bwd_ms * 1e-3) / 1e9, "peak": peak, "peak_source": peak_kind, "unit": "GB/s",
                "frac": bb / (bwd_ms * 1e-3) / 1e9 / peak, "traffic": traffic, "traffic_from": traffic_from,
                "algorithmic_bytes": bb, "ms": bwd_ms, "launches": launches_bwd,
                "forward": {"achieved": fb / (fwd_ms * 1e-3) / 1e9, "frac": fb / (fwd_ms * 1e-3) / 1e9 / peak,
                            "algorithmic_bytes": fb, "ms": fwd_ms},
                "fwd_bwd_frac": (fb + bb) / ((fwd_ms + bwd_ms) * 1e-3) / 1e9 / peak}

    line = None
    if rank == 0:
        line = {
            "metric": "conv_fwd_bwd_edges_per_s", "value": value, "unit": "edges/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(args, spec, graph),
            "kernel_ms": {"forward": main["fwd_ms_max"], "backward": main["bwd_ms_max"]},
            "roofline": roofline, "e2e": main.get("e2e"),
            "gpu_launches": (1 + launches_bwd) * args.steps, "clocks": main["clocks"],
            "launch": {"backward": info_b, "forward": info_f},
            "halo_fraction": main["halo_fraction"],
        }
        if "parity" in main:
            line["parity"] = main["parity"]

    # release the main workload before anything else is allocated
    conv_main = main.pop("conv")
    del conv_main, main, inner
    torch.cuda.empty_cache()

    if not args.no_secondary and det and args.workload == "mace_large":
        other = "random" if args.numbering == "morton" else "morton"
        rnd = measure(other, max(2, min(args.steps, 5)), False, False)
        if rank == 0:
            g2 = rnd["graph"]
            line["random_numbering" if other == "random" else "morton_numbering"] = {
                "value": g2.nnz / (rnd["elapsed"] / rnd["steps"]), "unit": "edges/s", "steps": rnd["steps"],
                "ms_per_step": rnd["elapsed"] / rnd["steps"] * 1e3,
                "kernel_ms": {"forward": rnd["fwd_ms_max"], "backward": rnd["bwd_ms_max"]},
                "halo_fraction": rnd["halo_fraction"], "numbering": other,
                "note": "halo_fraction = halo rows / owned rows of rank 0"}
        rnd.pop("conv")
        del rnd
        torch.cuda.empty_cache()
        if rank == 0 and world == 1:
            peaks = matmul_peaks(torch)
            line["peaks"] = peaks
            line["secondary"] = secondary_block(torch, args, device, peaks)

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        base = cpu_baseline(problem, spec, graph, 2, 1, args.seed)
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_e2e(args, torch, dist, world, device, conv, det, resident, edges, local_edges, index, graph=None):
    """Forward + backward with every input copied from pinned host memory and every output copied
    back, inside the timed region.  Host memory stays bounded: the per-edge weight array and its
    gradient move through one pinned tile that is re-used for every slice of the device array (the
    bytes that cross PCIe are the full arrays; a real caller's 70 GB host array would add its own
    page-touch cost).

    Deterministic variant, any number of GPUs: the public host-tensor entry point
    (``ShardedTensorProductConv.forward_backward_host``), which exchanges the halo once and pipelines
    the rank's edge slabs so that the copies in both directions overlap the kernels.  Atomic variant
    (one GPU): copy in, run, copy out."""
    x, y, w, dz = resident
    pin = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
    pinned_like = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True)   # empty_like would not pin
    # pinned buffers on the GPU's own NUMA node (a copy that crosses the socket interconnect is slower)
    numa_node = None
    if os.environ.get("OEQ_B200_NUMA_BIND", "1") != "0":
        from openequivariance_b200.stream import bind_host_to_device_node
        numa_node = bind_host_to_device_node(device.index if device.index is not None else 0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(one, h2d, d2h, note):
        one()
        one()
        barrier()
        retries0 = torch.cuda.memory_stats(device).get("num_alloc_retries", 0)
        t0 = time.perf_counter()
        marks = []
        for _ in range(args.e2e_steps):
            one()
            marks.append(time.perf_counter())
        barrier()
        dt = torch.tensor([(time.perf_counter() - t0) / args.e2e_steps], device=device, dtype=torch.float64)
        step_ms = [round((b - a) * 1e3, 1) for a, b in zip([t0] + marks[:-1], marks)]   # this rank's steps, one by one
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        return {"value": edges / dt.item(), "unit": "edges/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": dt.item() * 1e3, "steps": args.e2e_steps,
                "warmup": 2, "step_ms_rank0": step_ms, "host_numa_node": numa_node,
                "allocator_retries_rank0": torch.cuda.memory_stats(device).get("num_alloc_retries", 0) - retries0,
                "note": note}

    if det:
        # host-tensor entry point of the sharded convolution: X of the rank's nodes goes in, the halo is
        # exchanged, the per-edge arrays stream through the GPU in slabs (copies overlap the kernels)
        elem = x.element_size()
        streamed = conv.slab_plan(args.slab_edges)
        x_h, dz_h = pin(x), pin(dz)
        z_h = torch.empty((x.shape[0], dz.shape[1]), dtype=x.dtype, pin_memory=True)
        dx_h = pinned_like(x_h)
        tile = streamed.max_edges
        y_h, w_h = pin(y[:tile]), pin(w[:tile])
        dy_h, dw_h = pinned_like(y_h), pinned_like(w_h)
        tile_of = lambda t: (lambda i, lo, hi: t[:hi - lo])      # every slab crosses through the same pinned tile
        # nothing below reads the device-resident arrays: release them (and the allocator's cached blocks) so that
        # no step has to wait for the allocator to flush its cache
        resident.clear()
        del x, y, w, dz
        torch.cuda.synchronize()
        torch.cuda.empty_cache()

        def one():
            conv.forward_backward_host(x_h, tile_of(y_h), tile_of(w_h), dz_h, z_h, dx_h, tile_of(dy_h), tile_of(dw_h),
                                       slab_edges=args.slab_edges)
            torch.cuda.synchronize()

        h2d, d2h = conv.host_bytes(elem)
        if world > 1:
            tot = torch.tensor([h2d, d2h], device=device, dtype=torch.float64)
            dist.all_reduce(tot)
            h2d, d2h = tot[0].item(), tot[1].item()
        return timed(one, h2d, d2h,
                     f"{len(streamed.slabs)} edge slabs per rank pipelined (copy in / kernels / copy out overlap); "
                     "per-edge arrays cross PCIe through one re-used pinned tile per array (not a full-size host "
                     "array); bytes summed over ranks")

    tile = min(local_edges, 1 << 19)
    x_h, y_h, dz_h = pin(x), pin(y), pin(dz)
    w_h = pin(w[:tile])
    idx_dev = list(index)
    idx_h = [pin(t) for t in idx_dev]
    z_h = torch.empty((x.shape[0], dz.shape[1]), dtype=x.dtype, pin_memory=True)
    dx_h, dy_h, dw_h = pinned_like(x_h), pinned_like(y_h), pinned_like(w_h)
    x_d, y_d, dz_d, w_d = x, y, dz, w      # copy over the resident tensors: no second device copy
    h2d = sum(t.numel() * t.element_size() for t in (x_h, y_h, dz_h, *idx_h)) + w.numel() * w.element_size()
    d2h = sum(t.numel() * t.element_size() for t in (z_h, dx_h, dy_h)) + w.numel() * w.element_size()

    def one():
        x_d.copy_(x_h, non_blocking=True)
        y_d.copy_(y_h, non_blocking=True)
        dz_d.copy_(dz_h, non_blocking=True)
        for dst, src in zip(idx_dev, idx_h):
            dst.copy_(src, non_blocking=True)
        for lo in range(0, local_edges, tile):
            n = min(tile, local_edges - lo)
            w_d[lo:lo + n].copy_(w_h[:n], non_blocking=True)
        z = conv.forward(x_d, y_d, w_d, *idx_dev)
        dx, dy, dw = conv.backward_helper(x_d, y_d, w_d, dz_d, *idx_dev)
        z_h.copy_(z, non_blocking=True)
        dx_h.copy_(dx, non_blocking=True)
        dy_h.copy_(dy, non_blocking=True)
        for lo in range(0, local_edges, tile):
            n = min(tile, local_edges - lo)
            dw_h[:n].copy_(dw[lo:lo + n], non_blocking=True)
        torch.cuda.synchronize()

    return timed(one, h2d, d2h, "copy in, run, copy out; W and dW cross PCIe through one re-used pinned tile")


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
