"""Regenerate the golden fixtures in this directory from the reference project.

Run where a checkout of the reference project is available and point
``OEQ_REFERENCE`` at it:

    OEQ_REFERENCE=/path/to/OpenEquivariance python tests/golden/make_golden.py

Only the reference's CPU-runnable pieces are executed: its problem
description and Clebsch-Gordan generator (e3nn_lite.py), its numpy "uvu"
forward (NumpyTensorProduct.py), its weight permutation
(ComputationSchedule.reorder_weights), its edge ordering (CoordGraph), its
scatter-sum, its problem builders and its random-buffer generator.  The
reference package's ``__init__`` builds a CUDA extension on import, so the
package and its ``extlib`` are replaced by empty stand-ins first.

Outputs (all small):
  wigner_3j.npz          real Wigner 3j tensors for every valid l1,l2,l3 <= 7 (the reference's roofline
                         benchmark set, test/benchmark.py:56-70, reaches l = 7)
  problems.json          path weights / shapes / weight_numel of named problems
  numpy_tp_forward.npz   NumpyTensorProduct.forward_cpu on seeded inputs
  weight_perm.npz        reorder_weights applied to arange(weight_numel)
  coord_graph.npz        CoordGraph ordering of a random multigraph
  scatter_sum.npz        scatter_sum on CPU
  bench_conventions.json flop / byte counts of the reference's benchmark records for the named problems
"""

import json
import os
import sys
import types

import numpy as np

REF = os.environ.get("OEQ_REFERENCE")
if not REF:
    raise SystemExit("set OEQ_REFERENCE to the root of a checkout of the reference project")
HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference():
    pkg = types.ModuleType("openequivariance")
    pkg.__path__ = [os.path.join(REF, "openequivariance")]
    sys.modules["openequivariance"] = pkg
    ext = types.ModuleType("openequivariance.extlib")

    class KernelLaunchConfig:  # four plain fields are all the scheduler touches
        num_blocks = 0
        num_threads = 0
        smem = 0
        warp_size = 32

    ext.KernelLaunchConfig = KernelLaunchConfig
    ext.__all__ = ["KernelLaunchConfig"]
    sys.modules["openequivariance.extlib"] = ext
    pkg.extlib = ext


# (name, builder kind, args, kwargs) -- shared with the tests through problems.json
PROBLEMS = [
    ("readme", "tpp", ["1x2e", "1x3e", "1x2e", [[0, 0, 0, "uvu", True]]],
     {"shared_weights": False, "internal_weights": False}),
    ("mace_128", "channelwise", ["128x0e+128x1o+128x2e", "1x0e+1x1o+1x2e+1x3o", "128x0e+128x1o+128x2e"], {}),
    ("nequip_32", "channelwise", ["32x0e+32x1o+32x2e", "0e+1o+2e", "32x0e+32x1o+32x2e"], {}),
    ("uvw_64", "fully_connected", ["64x0e+64x1o+64x2e", "0e+1o+2e", "64x0e+64x1o+64x2e"], {}),
    ("mace_large_128", "channelwise",
     ["128x0e+128x1o+128x2e+128x3o", "1x0e+1x1o+1x2e+1x3o", "128x0e+128x1o+128x2e+128x3o"], {}),
    ("cw_mixed", "channelwise", ["5x0e+3x1o+2x2e+1x3o+4x1e", "1x0e+1x1o+1x2e+1x3o", "0e+0o+1o+1e+2e+2o+3o+3e"], {}),
    ("uvu_v2", "tpp", ["4x1o+3x0e", "2x1o+2x0e", "4x1o+4x0e+3x1o+4x1e",
                       [[0, 0, 1, "uvu", True], [0, 1, 0, "uvu", True], [1, 0, 2, "uvu", True, 0.5],
                        [0, 0, 3, "uvu", True]]],
     {"shared_weights": False, "internal_weights": False}),
    ("uvu_mul40_v3", "tpp", ["40x1e", "3x1e", "40x1e+40x0e",
                             [[0, 0, 0, "uvu", True], [0, 0, 1, "uvu", True]]],
     {"shared_weights": False, "internal_weights": False}),
    ("uvu_norm_path", "tpp", ["5x0e+5x1o", "1x0e+1x1o", "5x0e+5x1o",
                              [[0, 0, 0, "uvu", True], [1, 1, 0, "uvu", True], [0, 1, 1, "uvu", True],
                               [1, 0, 1, "uvu", True, 2.0]]],
     {"shared_weights": False, "internal_weights": False, "irrep_normalization": "norm",
      "path_normalization": "path", "in1_var": [1.0, 2.0], "in2_var": [0.5, 1.0], "out_var": [1.0, 3.0]}),
    ("uvw_small", "fully_connected", ["3x0e+2x1o", "2x0e+1x1o", "4x0e+3x1o+2x1e"], {}),
    ("uvw_mul40", "fully_connected", ["40x0e+8x1o", "0e+1o", "36x0e+33x1o"], {}),
    ("uvw_rowweights", "fully_connected", ["3x0e+2x1o", "2x0e+1x1o", "4x0e+3x1o"],
     {"shared_weights": False, "internal_weights": False}),
    ("uvu_shared", "tpp", ["8x0e+8x1o", "0e+1o", "8x0e+8x1o",
                           [[0, 0, 0, "uvu", True], [1, 1, 0, "uvu", True], [0, 1, 1, "uvu", True],
                            [1, 0, 1, "uvu", True]]],
     {"shared_weights": True, "internal_weights": False}),
    # a small channel-wise problem for the interaction-block test (energies, forces, one training step)
    ("interaction_8", "channelwise", ["8x0e+8x1o", "1x0e+1x1o", "8x0e+8x1o"], {}),
    # the reference's benchmark shapes with mixed parities and second-input multiplicity 1
    # (openequivariance/benchmark/benchmark_configs.py:38-47)
    ("tetris_poly_1", "fully_connected", ["1x0e + 1x1o + 1x2e + 1x3o", "1x0e + 1x1o + 1x2e + 1x3o",
                                          "64x0e + 24x1e + 24x1o + 16x2e + 16x2o"], {}),
    ("tetris_poly_2", "fully_connected", ["64x0e + 24x1e + 24x1o + 16x2e + 16x2o", "1x0e + 1x1o + 1x2e + 1x3o",
                                          "0o + 6x0e"], {}),
    ("diffdock_l1", "fully_connected", ["10x1o + 10x1e + 48x0e + 48x0o", "1x0e + 1x1o",
                                        "10x1o + 10x1e + 48x0e + 48x0o"], {"shared_weights": False}),
    ("diffdock_l2", "fully_connected", ["10x1o + 10x1e + 48x0e + 48x0o", "1x0e + 1x1o + 1x2e",
                                        "10x1o + 10x1e + 48x0e + 48x0o"], {"shared_weights": False}),
    # single instructions of the reference's roofline set (test/benchmark.py:56-70), l up to 7
    ("roofline_1e", "single", ["128x1e", "1x1e", "128x1e", "uvu"], {}),
    ("roofline_5e_3e", "single", ["128x5e", "1x5e", "128x3e", "uvu"], {}),
    ("roofline_6e", "single", ["128x6e", "1x3e", "128x6e", "uvu"], {}),
    ("roofline_7e_4e", "single", ["128x7e", "1x4e", "128x7e", "uvu"], {}),
    ("roofline_7e_7e", "single", ["128x7e", "1x7e", "128x7e", "uvu"], {}),
]


def build(ref_mods, kind, args, kwargs):
    e3, tpp = ref_mods
    if kind == "tpp":
        a, b, c, instr = args
        return e3.TPProblem(e3.Irreps(a), e3.Irreps(b), e3.Irreps(c), [tuple(i) for i in instr], **kwargs)
    if kind == "channelwise":
        return tpp.ChannelwiseTPP(*args, **kwargs)
    if kind == "fully_connected":
        return tpp.FullyConnectedTPProblem(*args, **kwargs)
    if kind == "single":
        return tpp.SingleInstruction(*args, **kwargs)
    raise ValueError(kind)


def main():
    _import_reference()
    import openequivariance.implementations.e3nn_lite as e3
    import openequivariance.benchmark.tpp_creation_utils as tpp
    from openequivariance.benchmark.random_buffer_utils import get_random_buffers_forward
    from openequivariance.implementations.NumpyTensorProduct import NumpyTensorProduct
    from openequivariance.implementations.ComputationSchedule import ComputationSchedule
    from openequivariance.implementations.convolution.ConvolutionBase import CoordGraph
    from openequivariance.implementations.convolution.scatter import scatter_sum
    import torch

    # 1. Wigner 3j
    tensors = {}
    lmax = 7
    for l1 in range(lmax + 1):
        for l2 in range(lmax + 1):
            for l3 in range(abs(l1 - l2), min(l1 + l2, lmax) + 1):
                tensors[f"{l1}_{l2}_{l3}"] = e3.wigner_3j(l1, l2, l3)
    np.savez_compressed(os.path.join(HERE, "wigner_3j.npz"), **tensors)

    # 2. problems
    described = []
    built = {}
    for name, kind, args, kwargs in PROBLEMS:
        p = build((e3, tpp), kind, args, kwargs)
        built[name] = p
        described.append({
            "name": name, "kind": kind, "args": args, "kwargs": kwargs,
            "irreps_in1": str(p.irreps_in1), "irreps_in2": str(p.irreps_in2), "irreps_out": str(p.irreps_out),
            "in1_dim": p.irreps_in1.dim, "in2_dim": p.irreps_in2.dim, "out_dim": p.irreps_out.dim,
            "weight_numel": p.weight_numel, "shared_weights": p.shared_weights,
            "internal_weights": p.internal_weights,
            "instructions": [[i.i_in1, i.i_in2, i.i_out, i.connection_mode, i.has_weight,
                              float(i.path_weight), list(i.path_shape)] for i in p.instructions],
        })
    with open(os.path.join(HERE, "problems.json"), "w") as f:
        json.dump(described, f, indent=1)

    # 3. numpy forward of the reference ("uvu", per-row weights, e3nn weight order)
    fwd = {}
    # (NumpyTensorProduct indexes weights by output block, so it is only valid for
    # channel-wise problems: second-input multiplicity 1, one output block per instruction)
    for name, batch in [("readme", 1000), ("nequip_32", 24), ("cw_mixed", 17), ("mace_128", 3),
                        ("mace_large_128", 2), ("roofline_5e_3e", 2), ("roofline_6e", 2), ("roofline_7e_7e", 2)]:
        p = built[name]
        in1, in2, w, out = get_random_buffers_forward(p, batch, 12345)
        NumpyTensorProduct(p).forward_cpu(in1, in2, out, w)
        if name == "readme":
            # inputs are regenerated from the seed in the test; keep the file small
            fwd[f"{name}__norm"] = np.array([np.linalg.norm(out.astype(np.float64))])
            fwd[f"{name}__head"] = out[:4].copy()
            fwd[f"{name}__out_every_50"] = out[::50].copy()
        else:
            fwd[f"{name}__in1"], fwd[f"{name}__in2"], fwd[f"{name}__w"], fwd[f"{name}__out"] = in1, in2, w, out
    np.savez_compressed(os.path.join(HERE, "numpy_tp_forward.npz"), **fwd)

    # 4. weight permutation (e3nn -> kernel order), applied to arange
    perms = {}
    for name, p in built.items():
        sched = ComputationSchedule(p, smem_limit=232448, warps_per_block=8, block_count=148 * 4,
                                    direction="forward", irrep_dtype=np.float32, weight_dtype=np.float32,
                                    include_scratch=(p.instructions[0].connection_mode == "uvw"),
                                    stream_weights=(p.instructions[0].connection_mode == "uvw"))
        src = np.arange(p.weight_numel, dtype=np.float64)
        dst = np.zeros_like(src)
        sched.reorder_weights(src, dst, "forward", False)
        back = np.zeros_like(src)
        sched.reorder_weights(dst, back, "backward", False)
        assert np.array_equal(back, src)
        perms[name] = dst.astype(np.int64)
        src2 = np.stack([src, src[::-1]])
        dst2 = np.zeros_like(src2)
        sched.reorder_weights(src2, dst2, "forward", True)
        assert np.array_equal(dst2[0], dst)
    np.savez_compressed(os.path.join(HERE, "weight_perm.npz"), **perms)

    # 5. CoordGraph on a random directed multigraph (duplicates + asymmetric edges)
    rng = np.random.default_rng(7)
    n, e = 13, 60
    rows = rng.integers(0, n, size=e).astype(np.int64)
    cols = rng.integers(0, n, size=e).astype(np.int64)
    g = CoordGraph(np.zeros((n, 3)), rows, cols, "golden")
    np.savez_compressed(os.path.join(HERE, "coord_graph.npz"), rows_in=rows, cols_in=cols,
                        rows=g.rows, cols=g.cols, transpose_perm=g.transpose_perm)

    # 6. scatter_sum on CPU
    src = torch.as_tensor(rng.normal(size=(e, 5)))
    idx = torch.as_tensor(rows)
    out = scatter_sum(src=src, index=idx, dim=0, dim_size=n)
    np.savez_compressed(os.path.join(HERE, "scatter_sum.npz"), src=src.numpy(), index=rows, out=out.numpy())
    # 7. flop and byte conventions of the reference's benchmark records
    from openequivariance.benchmark.perf_metrics_utils import (calculate_minimum_flops_forward,
                                                              calculate_minimum_memory_streamed_forward,
                                                              calculate_minimum_memory_streamed_backward)
    from openequivariance.benchmark.e3nn_lite_utils import calculate_total_nnz
    from openequivariance.implementations.convolution.ConvolutionBase import flops_data_per_tp
    conv = {}
    for name, p in built.items():
        entry = {"total_cg_nnz": int(calculate_total_nnz(p)),
                 "minimum_flops_forward": {k: int(v) for k, v in calculate_minimum_flops_forward(p, 7).items()},
                 "memory_forward": {k: int(v) for k, v in calculate_minimum_memory_streamed_forward(p, 7).items()},
                 "memory_backward": {k: int(v) for k, v in calculate_minimum_memory_streamed_backward(p, 7).items()}}
        if not p.shared_weights:
            for direction in ("forward", "backward"):
                ops, data, nnz = flops_data_per_tp(p, direction)
                entry[f"conv_{direction}"] = [int(ops), int(data), int(nnz)]
        conv[name] = entry
    with open(os.path.join(HERE, "bench_conventions.json"), "w") as f:
        json.dump(conv, f, indent=1)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
