"""Timing of the batch tensor product (rows per second), the counterpart of the reference's
``test/benchmark.py uvu`` / ``uvw`` drivers (reference: test/benchmark.py:107-134) for two fixed
configurations:

  uvu_mace  channel-wise 128x(0e+1o+2e) x (0e+1o+2e+3o), per-row weights, batch 50 000
  uvw_fc    fully connected 64x(0e+1o+2e) x (0e+1o+2e) -> 64x(0e+1o+2e), shared weights, batch 100 000

    python -m openequivariance_b200.bench_tp --config uvw_fc --dtype f32 --steps 20

CUDA events around each launch, an L2 flush (256 MB memset) before every timed launch, one JSON line.
"""

import argparse
import json
import statistics

import numpy as np
import torch

import openequivariance_b200 as oeq

CONFIGS = {
    "uvu_mace": dict(kind="channelwise", in1="128x0e+128x1o+128x2e", in2="1x0e+1x1o+1x2e+1x3o",
                     out="128x0e+128x1o+128x2e", batch=50_000),
    "uvw_fc": dict(kind="fully_connected", in1="64x0e+64x1o+64x2e", in2="0e+1o+2e", out="64x0e+64x1o+64x2e",
                   batch=100_000),
}


def measure(config="uvw_fc", dtype="f32", steps=20, warmup=5, batch=None, forward_only=False):
    """Time one configuration on the current device; returns the result record (a dict)."""
    args = argparse.Namespace(config=config, dtype=dtype, steps=steps, warmup=warmup, batch=batch,
                              forward_only=forward_only)
    cfg = CONFIGS[args.config]
    np_dt, dt = (np.float32, torch.float32) if args.dtype == "f32" else (np.float64, torch.float64)
    if cfg["kind"] == "channelwise":
        p = oeq.ChannelwiseTPP(cfg["in1"], cfg["in2"], cfg["out"], irrep_dtype=np_dt, weight_dtype=np_dt)
    else:
        p = oeq.FullyConnectedTPProblem(cfg["in1"], cfg["in2"], cfg["out"], irrep_dtype=np_dt, weight_dtype=np_dt)
    tp = oeq.TensorProduct(p, torch_op=True)
    batch = args.batch or cfg["batch"]
    gen = torch.Generator(device="cuda").manual_seed(11111)
    x = torch.randn(batch, p.irreps_in1.dim, device="cuda", dtype=dt, generator=gen)
    y = torch.randn(batch, p.irreps_in2.dim, device="cuda", dtype=dt, generator=gen)
    wshape = (p.weight_numel,) if p.shared_weights else (batch, p.weight_numel)
    w = torch.randn(wshape, device="cuda", dtype=dt, generator=gen) / (8 if p.shared_weights else 1)
    dz = torch.randn(batch, p.irreps_out.dim, device="cuda", dtype=dt, generator=gen)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn):
        times = []
        for i in range(args.warmup + args.steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(a.elapsed_time(b))
        return statistics.median(times)

    fwd = timed(lambda: tp(x, y, w))
    bwd = None if args.forward_only else timed(lambda: tp.backward_helper(x, y, w, dz))
    tp.check_device_status()
    s = x.element_size()
    xd, yd, zd, wn = p.irreps_in1.dim, p.irreps_in2.dim, p.irreps_out.dim, p.weight_numel
    wbytes = wn * s if p.shared_weights else batch * wn * s
    fwd_bytes = batch * (xd + yd + zd) * s + wbytes
    bwd_bytes = batch * (2 * xd + 2 * yd + zd) * s + 2 * wbytes
    flops = 0
    if cfg["kind"] == "fully_connected":     # the dense weight contraction, 2 flop per multiply-add
        for ins in p.instructions:
            u, v, wm = ins.path_shape
            flops += 2 * batch * u * v * wm * p.irreps_out[ins.i_out].ir.dim
    line = {"config": args.config, "dtype": args.dtype, "batch": batch, "forward_ms": fwd, "backward_ms": bwd,
            "rows_per_s_forward": batch / (fwd * 1e-3),
            "rows_per_s_fwd_bwd": None if bwd is None else batch / ((fwd + bwd) * 1e-3),
            "forward_GBps": fwd_bytes / (fwd * 1e-3) / 1e9,
            "backward_GBps": None if bwd is None else bwd_bytes / (bwd * 1e-3) / 1e9,
            "forward_contraction_TFLOPs": flops / (fwd * 1e-3) / 1e12 if flops else None,
            "fwd_bwd_contraction_TFLOPs": None if (bwd is None or not flops) else 3 * flops / ((fwd + bwd) * 1e-3) / 1e12,
            "algorithmic_bytes": {"forward": fwd_bytes, "backward": bwd_bytes},
            "launch": {"forward": tp.internal.launch_info(0), "backward": tp.internal.launch_info(1)}}
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="uvw_fc", choices=sorted(CONFIGS))
    ap.add_argument("--dtype", default="f32", choices=["f32", "f64"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--forward-only", action="store_true")
    args = ap.parse_args()
    print(json.dumps(measure(args.config, args.dtype, args.steps, args.warmup, args.batch, args.forward_only)),
          flush=True)


if __name__ == "__main__":
    main()
