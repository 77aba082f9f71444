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
all-gathered before the forward kernel and their gradients reduce-scattered after the backward
kernel, both inside the timed region (only halo rows -- senders owned by another rank -- move).
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


# DRAM read+write bytes per edge of the deterministic backward launch, from a one-pass ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum) of the full-size run; proportional to the edge count
# at fixed degree, so it scales to other --nodes values of the same workload.
NCU_BWD_DRAM_BYTES_PER_EDGE = {("mace_large", "morton"): 377.4e9 / 6004880}


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
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--slab-edges", type=int, default=1 << 18,
                    help="edges per slab of the streamed host-tensor path (end-to-end measurement)")
    ap.add_argument("--seed", type=int, default=11111)
    return ap.parse_args()


def make_problem(spec):
    import openequivariance_b200 as oeq
    return oeq.ChannelwiseTPP(spec["in1"], spec["in2"], spec["out"])


def algorithmic_bytes(problem, nodes, edges, elem=4):
    """Compulsory HBM traffic of one launch: every edge array once, every node array once,
    int64 receiver/sender (and the sender-order permutation in the backward pass)."""
    x, y, z, w = problem.irreps_in1.dim, problem.irreps_in2.dim, problem.irreps_out.dim, problem.weight_numel
    fwd = edges * ((w + y) * elem + 16) + nodes * (x + z) * elem
    bwd = edges * (2 * (w + y) * elem + 24) + nodes * (2 * x + z) * elem
    return fwd, bwd


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu_index, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax = float(parts[2])
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_graph(spec, args):
    from openequivariance_b200.graph import periodic_radius_graph
    nodes = args.nodes or spec["nodes"]
    return periodic_radius_graph(nodes, spec["degree"], seed=args.seed, numbering=args.numbering)


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
                      f"{len(times)} timed passes, torch CPU float32 (gather, per-instruction contraction with the second "
                      f"input folded into the Clebsch-Gordan tensor, index_add), autograd backward",
            "ms_per_step": per_step * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    spec = WORKLOADS[args.workload]
    problem = make_problem(spec)
    graph = build_graph(spec, args)
    base = cpu_baseline(problem, spec, graph, max(1, args.steps), max(0, min(args.warmup, 1)), args.seed)
    line = {
        "impl": "reference", "metric": "conv_fwd_bwd_edges_per_s", "value": base["value"], "unit": "edges/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, spec, graph),
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, spec, graph):
    return {"workload": f"{args.workload}: fused conv uvu {spec['in1']} x {spec['in2']} -> l_out<={spec['lmax']}, "
                        f"{args.variant}, fwd+bwd",
            "nodes": graph.node_count, "edges": graph.nnz, "mean_degree": graph.nnz / max(1, graph.node_count),
            "numbering": args.numbering, "graph": "uniform points in a periodic unit cube, radius cutoff",
            "l2": "inputs larger than L2 (no flush needed)" if graph.nnz > 200_000 else "small case",
            "parallelism": f"receiver-range shards x{args.gpus}" if args.gpus > 1 else "single GPU"}


# --------------------------------------------------------------------------- GPU benchmark

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
    graph = build_graph(spec, args)
    nodes, edges = graph.node_count, graph.nnz
    det = args.variant == "deterministic"
    if not det and world > 1:
        raise SystemExit("the sharded benchmark runs the deterministic variant")

    if det:
        conv = ShardedTensorProductConv(problem, graph.rows, graph.cols, nodes, device=device)
        plan = conv.plan
        e_lo, e_hi, owned = plan.edge_lo, plan.edge_hi, plan.owned
    else:
        conv = oeq.TensorProductConv(problem, torch_op=True, deterministic=False)
        e_lo, e_hi, owned = 0, edges, nodes
        rows_d = torch.from_numpy(graph.rows).to(device)
        cols_d = torch.from_numpy(graph.cols).to(device)
    local_edges = e_hi - e_lo

    gen = torch.Generator(device=device).manual_seed(args.seed + rank)
    x = torch.randn(owned, problem.irreps_in1.dim, device=device, generator=gen)
    dz = torch.randn(owned, problem.irreps_out.dim, device=device, generator=gen)
    vec = torch.from_numpy(graph.vectors[e_lo:e_hi]).to(device=device, dtype=torch.float32)
    y = spherical_harmonics(spec["lmax"], vec).contiguous()
    del vec
    w = torch.empty(local_edges, problem.weight_numel, device=device)
    for lo in range(0, local_edges, 1 << 19):          # fill in slices: no temporary of W's size
        w[lo:lo + (1 << 19)].normal_(generator=gen)

    def step():
        if det:
            return conv.forward_backward(x, y, w, dz)
        z = conv.forward(x, y, w, rows_d, cols_d)
        dx, dy, dw = conv.backward_helper(x, y, w, dz, rows_d, cols_d)
        return z, dx, dy, dw

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        out = step()
        del out
    barrier()

    # -- timed region: device events per step, fwd and bwd kernels timed separately on rank's stream
    sampler = ClockSampler(local_rank if os.environ.get("CUDA_VISIBLE_DEVICES") is None else 0)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    inner = conv.conv if det else conv
    sampler.start()
    barrier()
    t0 = time.perf_counter()
    for k in range(args.steps):
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
    clocks = sampler.stop()
    inner.check_device_status()

    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    t = torch.tensor([elapsed, fwd_ms, bwd_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed, fwd_ms_max, bwd_ms_max = t.tolist()
    ms_per_step = elapsed / args.steps * 1e3
    value = edges / (elapsed / args.steps)

    # -- roofline of the dominant kernel (backward), rank 0's launch
    fb, bb = algorithmic_bytes(problem, owned if world > 1 else nodes, local_edges)
    if world > 1:   # a shard reads/writes its owned and halo rows of X / dX once, owned rows of Z / dZ
        xd, zd = problem.irreps_in1.dim, problem.irreps_out.dim
        fb = local_edges * ((problem.weight_numel + problem.irreps_in2.dim) * 4 + 16) + (plan.local_nodes * xd + owned * zd) * 4
        bb = local_edges * (2 * (problem.weight_numel + problem.irreps_in2.dim) * 4 + 24) + (2 * plan.local_nodes * xd + owned * zd) * 4
    peak, peak_kind = measured_peak()
    per_edge = NCU_BWD_DRAM_BYTES_PER_EDGE.get((args.workload, args.numbering))
    traffic = per_edge * local_edges if (per_edge is not None and world == 1 and det) else None
    roofline = {"bound": "hbm", "kernel": "oeq_uvu_kernel (conv backward)", "achieved": bb / (bwd_ms * 1e-3) / 1e9,
                "peak": peak, "peak_source": peak_kind, "unit": "GB/s", "frac": bb / (bwd_ms * 1e-3) / 1e9 / peak,
                "traffic": traffic, "algorithmic_bytes": bb, "ms": bwd_ms,
                "forward": {"achieved": fb / (fwd_ms * 1e-3) / 1e9, "frac": fb / (fwd_ms * 1e-3) / 1e9 / peak,
                            "algorithmic_bytes": fb, "ms": fwd_ms},
                "fwd_bwd_frac": (fb + bb) / ((fwd_ms + bwd_ms) * 1e-3) / 1e9 / peak}

    # -- end to end through the public API with host buffers
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, torch, dist, world, device, conv, det, x, y, w, dz, edges, local_edges,
                      (rows_d, cols_d) if not det else None, graph=graph)

    base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        base = cpu_baseline(problem, spec, graph, 2, 1, args.seed)

    if rank == 0:
        info = inner.internal.launch_info(1)
        line = {
            "metric": "conv_fwd_bwd_edges_per_s", "value": value, "unit": "edges/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(args, spec, graph),
            "kernel_ms": {"forward": fwd_ms_max, "backward": bwd_ms_max},
            "roofline": roofline, "e2e": e2e, "gpu_launches": 2 * args.steps, "clocks": clocks,
            "launch": {"backward": info, "forward": inner.internal.launch_info(0)},
        }
        if base is not None:
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_e2e(args, torch, dist, world, device, conv, det, x, y, w, dz, edges, local_edges, index, graph=None):
    """Forward + backward with every input copied from pinned host memory and every output copied
    back, inside the timed region.  Host memory stays bounded: the per-edge weight array and its
    gradient move through one pinned tile that is re-used for every slice of the device array (the
    bytes that cross PCIe are the full arrays).

    Deterministic variant, any number of GPUs: the public host-tensor entry point
    (``ShardedTensorProductConv.forward_backward_host``), which exchanges the halo once and pipelines
    the rank's edge slabs so that the copies in both directions overlap the kernels.  Atomic variant
    (one GPU): copy in, run, copy out."""
    pin = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
    pinned_like = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True)   # empty_like would not pin

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(one, h2d, d2h, note):
        one()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            one()
        barrier()
        dt = torch.tensor([(time.perf_counter() - t0) / args.e2e_steps], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        return {"value": edges / dt.item(), "unit": "edges/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": dt.item() * 1e3, "steps": args.e2e_steps,
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
                     "per-edge arrays cross PCIe through one re-used pinned tile per array; bytes summed over ranks")

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
