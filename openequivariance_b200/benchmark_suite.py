"""Benchmark records in the reference's JSON layout, so that its plotting scripts can read them.

The reference's suite (reference: openequivariance/benchmark/TestBenchmarkSuite.py:18-190) writes a folder
with ``metadata.json`` and one ``{test_ID}_{implementation}.json`` per test; the convolution benchmarks
return one record per graph (reference: openequivariance/implementations/convolution/ConvolutionBase.py:
256-439).  This module produces the same files and keys for this library's operators:

    suite = TestBenchmarkSuite(bench_batch_size=50_000)
    folder = suite.run([TestDefinition(oeq.TensorProduct, problem, "forward", correctness=False)], "out")
    record = benchmark_conv(conv, graph, "backward")

Flop and byte counts follow the reference's own conventions (its per-kernel counts for "uvu", its
"minimum" counts for "uvw"), not the roofline bytes that ``bench.py`` uses, so numbers are comparable
with the reference's published plots.  Correctness needs a reference implementation object with
``forward_cpu`` / ``backward_cpu`` (the reference uses e3nn); when none is given the check is skipped
and recorded as such.  Timing: CUDA events around each launch, L2 flushed before every timed launch.
"""

from __future__ import annotations

import json
import math
import os
import pathlib
import time
from typing import NamedTuple, Optional

import numpy as np

from .wigner import cg_nonzeros, wigner_3j

L2_FLUSH_BYTES = 256 << 20


class TestDefinition(NamedTuple):
    implementation: type
    problem: object
    direction: str
    correctness: bool = True
    benchmark: bool = True


# --------------------------------------------------------------------------- seeded buffers
# draw order of the reference (openequivariance/benchmark/random_buffer_utils.py:11-52)

def get_random_buffers_forward(tpp, batch_size: int, prng_seed: int):
    rng = np.random.default_rng(prng_seed)
    in1 = np.array(rng.uniform(size=(batch_size, tpp.irreps_in1.dim)), dtype=tpp.irrep_dtype)
    in2 = np.array(rng.uniform(size=(batch_size, tpp.irreps_in2.dim)), dtype=tpp.irrep_dtype)
    wshape = (tpp.weight_numel,) if tpp.shared_weights else (batch_size, tpp.weight_numel)
    weights = np.array(rng.uniform(size=wshape), dtype=tpp.weight_dtype)
    out = np.zeros((batch_size, tpp.irreps_out.dim), dtype=tpp.weight_dtype)
    return in1, in2, weights, out


def get_random_buffers_backward(tpp, batch_size: int, prng_seed: int):
    rng = np.random.default_rng(prng_seed)
    in1 = np.array(rng.uniform(size=(batch_size, tpp.irreps_in1.dim)), dtype=tpp.irrep_dtype)
    in2 = np.array(rng.uniform(size=(batch_size, tpp.irreps_in2.dim)), dtype=tpp.irrep_dtype)
    out_grad = np.array(rng.uniform(size=(batch_size, tpp.irreps_out.dim)), dtype=tpp.irrep_dtype)
    wshape = (tpp.weight_numel,) if tpp.shared_weights else (batch_size, tpp.weight_numel)
    weights = np.array(rng.uniform(size=wshape), dtype=tpp.irrep_dtype)
    return in1, in2, out_grad, weights, np.zeros_like(weights), np.zeros_like(in1), np.zeros_like(in2)


# --------------------------------------------------------------------------- flop / byte conventions

def _ls(tpp, ins):
    return tpp.irreps_in1[ins.i_in1].ir.l, tpp.irreps_in2[ins.i_in2].ir.l, tpp.irreps_out[ins.i_out].ir.l


def count_cg_non_zero(l1, l2, l3) -> int:
    return len(cg_nonzeros(l1, l2, l3))


def calculate_total_nnz(tpp) -> int:
    return sum({_ls(tpp, ins): count_cg_non_zero(*_ls(tpp, ins)) for ins in tpp.instructions}.values())


def _is_uvw(tpp) -> bool:
    return tpp.instructions[0].connection_mode == "uvw"


def calculate_minimum_flops_forward(tpp, batch_size: int) -> dict:
    """Reference: perf_metrics_utils.py:49-74 (outer products formed once per Clebsch-Gordan tensor)."""
    count = {"outer_products": 0, "CG_decomposition": 0, "linear_combination": 0}
    for ins in tpp.instructions:
        l1, l2, l3 = _ls(tpp, ins)
        cg = np.asarray(wigner_3j(l1, l2, l3))
        count["outer_products"] += int(np.sum(np.max(cg != 0, axis=2)))
        count["CG_decomposition"] += count_cg_non_zero(l1, l2, l3) * (ins.path_shape[0] * ins.path_shape[1])
        count["linear_combination"] += (2 * l3 + 1) * math.prod(ins.path_shape) if ins.has_weight else 0
    count["outer_products"] *= batch_size
    count["CG_decomposition"] *= 2 * batch_size
    count["linear_combination"] *= 2 * batch_size
    count["total"] = sum(count.values())
    return count


def calculate_flops_forward(tpp, batch_size: int) -> dict:
    """Reference: LoopUnrollTP.calculate_flops_forward (LoopUnrollTP.py:77-91) for "uvu", the "minimum" count
    for "uvw"."""
    if _is_uvw(tpp):
        return calculate_minimum_flops_forward(tpp, batch_size)
    else:
        count = {"CG_decomposition": 0, "linear_combination": 0, "outer_products": 0}
        for ins in tpp.instructions:
            l1, l2, l3 = _ls(tpp, ins)
            count["CG_decomposition"] += count_cg_non_zero(l1, l2, l3) * (ins.path_shape[0] * ins.path_shape[1])
            count["linear_combination"] += (2 * l3 + 1) * math.prod(ins.path_shape) if ins.has_weight else 0
        count["CG_decomposition"] *= 3 * batch_size
        count["linear_combination"] *= batch_size
    count["total"] = sum(count.values())
    return count


def calculate_flops_backward(tpp, batch_size: int) -> dict:
    """Reference: LoopUnrollTP.calculate_flops_backward (LoopUnrollTP.py:93-105); "uvw" falls back to the
    forward "minimum" count as the reference's driver does (benchmark_utils.py:165-173)."""
    if _is_uvw(tpp):
        return calculate_flops_forward(tpp, batch_size)
    count = {"backward": 0}
    for ins in tpp.instructions:
        count["backward"] += count_cg_non_zero(*_ls(tpp, ins)) * (ins.path_shape[0] * ins.path_shape[1])
    count["backward"] *= 9 * batch_size
    count["total"] = sum(count.values())
    return count


def calculate_minimum_memory_streamed_forward(tpp, batch_size: int) -> dict:
    iw, ww = np.dtype(tpp.irrep_dtype).itemsize, np.dtype(tpp.weight_dtype).itemsize
    size = {"input 1": tpp.irreps_in1.dim * batch_size * iw, "input 2": tpp.irreps_in2.dim * batch_size * iw,
            "output": tpp.irreps_out.dim * batch_size * iw, "weights": tpp.weight_numel * batch_size * ww}
    size["total"] = sum(size.values())
    return size


def calculate_minimum_memory_streamed_backward(tpp, batch_size: int) -> dict:
    iw, ww = np.dtype(tpp.irrep_dtype).itemsize, np.dtype(tpp.weight_dtype).itemsize
    size = {"input 1": tpp.irreps_in1.dim * batch_size * iw, "input 1 grad": tpp.irreps_in1.dim * batch_size * iw,
            "input 2": tpp.irreps_in2.dim * batch_size * iw, "input 2 grad": tpp.irreps_in2.dim * batch_size * iw,
            "output grad": tpp.irreps_out.dim * batch_size * iw, "weights": tpp.weight_numel * batch_size * ww,
            "weights grad": tpp.weight_numel * batch_size * ww}
    size["total"] = sum(size.values())
    return size


def calculate_performance_statistics(problem, batch_size, total_flops, total_memory_streamed, time_millis) -> dict:
    """Reference: benchmark_utils.py:17-57 (same keys)."""
    time_millis = np.asarray(time_millis, dtype=np.float64)
    return {
        "total_cg_nnz": calculate_total_nnz(problem),
        "flops_per_tp": total_flops / batch_size,
        "L1": str(problem.irreps_in1), "L2": str(problem.irreps_in2), "L3": str(problem.irreps_out),
        "L1_rep_len": problem.irreps_in1.dim, "L2_rep_len": problem.irreps_in2.dim,
        "L3_rep_len": problem.irreps_out.dim,
        "rep_dtype": str(problem.irrep_dtype), "weight_dtype": str(problem.weight_dtype),
        "arithmetic_intensity (FLOPs / byte)": total_flops / total_memory_streamed,
        "batch_size": batch_size,
        "time_millis": [float(x) for x in time_millis],
        "throughputs_gflops": [float(x) for x in total_flops / (time_millis * 1e6)],
        "bandwidth_gbps": [float(x) for x in total_memory_streamed / (time_millis * 1e6)],
    }


def check_similiarity(name, to_check, ground_truth, correctness_threshold) -> dict:
    """Reference: correctness_utils.py:13-31 (the reference's spelling of the name is kept)."""
    if to_check.shape != ground_truth.shape:
        return {"shape_match": False, "diff_Linf_norm": float("inf"), "pass": False}
    diff = float(np.max(np.abs(ground_truth.astype(np.float64) - to_check.astype(np.float64)))) if to_check.size else 0.0
    return {"shape_match": True, "diff_Linf_norm": diff, "pass": bool(diff < correctness_threshold)}


# --------------------------------------------------------------------------- timing

def _time_launches(fn, num_warmup: int, num_iter: int):
    import torch
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
    for _ in range(num_warmup):
        fn()
    times = np.zeros(num_iter, dtype=np.float32)
    for i in range(num_iter):
        flush.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        times[i] = start.elapsed_time(stop)
    return times


def benchmark_forward(problem, implementation, batch_size, num_warmup, num_iter, prng_seed, torch_op) -> dict:
    import torch
    result = {"tp_direction": "forward", "num_warmup": num_warmup, "num_iter": num_iter, "prng_seed": prng_seed}
    in1, in2, weights, _ = get_random_buffers_forward(problem, batch_size, prng_seed)
    tp = implementation(problem, torch_op=torch_op)
    x, y = (torch.from_numpy(a).cuda() for a in (in1, in2))
    w = tp._weights_to_device(weights)          # the kernels take the reordered layout
    launch = (lambda: tp.forward(x, y, w)) if torch_op else (lambda: tp._forward_impl(x, y, w))
    times = _time_launches(launch, num_warmup, num_iter)
    flops = calculate_flops_forward(problem, batch_size)
    memory = calculate_minimum_memory_streamed_forward(problem, batch_size)
    result |= calculate_performance_statistics(problem, batch_size, flops["total"], memory["total"], times)
    return result


def benchmark_backward(problem, implementation, batch_size, num_warmup, num_iter, prng_seed, torch_op) -> dict:
    import torch
    result = {"tp_direction": "backward", "num_warmup": num_warmup, "num_iter": num_iter, "prng_seed": prng_seed}
    in1, in2, out_grad, weights, _, _, _ = get_random_buffers_backward(problem, batch_size, prng_seed)
    tp = implementation(problem, torch_op=torch_op)
    x, y, dz = (torch.from_numpy(a).cuda() for a in (in1, in2, out_grad))
    w = tp._weights_to_device(weights)
    launch = (lambda: tp.backward_helper(x, y, w, dz)) if torch_op else (lambda: tp._backward_impl(x, y, w, dz))
    times = _time_launches(launch, num_warmup, num_iter)
    flops = calculate_flops_backward(problem, batch_size)
    memory = calculate_minimum_memory_streamed_backward(problem, batch_size)
    result |= calculate_performance_statistics(problem, batch_size, flops["total"], memory["total"], times)
    return result


def correctness_forward(problem, test_implementation, reference_implementation, batch_size, correctness_threshold,
                        prng_seed) -> dict:
    result = {"thresh": correctness_threshold, "batch_size": batch_size}
    in1, in2, weights, out = get_random_buffers_forward(problem, batch_size, prng_seed)
    ref_out, test_out = out.copy(), out.copy()
    reference_implementation(problem).forward_cpu(L1_in=in1.copy(), L2_in=in2.copy(), L3_out=ref_out, weights=weights.copy())
    test_implementation(problem).forward_cpu(L1_in=in1.copy(), L2_in=in2.copy(), L3_out=test_out, weights=weights.copy())
    result["output"] = check_similiarity("output", ref_out, test_out, correctness_threshold)
    return result


def correctness_backward(problem, test_implementation, reference_implementation, batch_size, correctness_threshold,
                         prng_seed) -> dict:
    result = {"thresh": correctness_threshold}
    in1, in2, out_grad, weights, wg, g1, g2 = get_random_buffers_backward(problem, batch_size, prng_seed)
    ref = [wg.copy(), g1.copy(), g2.copy()]
    got = [wg.copy(), g1.copy(), g2.copy()]
    for impl, (wgrad, in1_grad, in2_grad) in ((reference_implementation, ref), (test_implementation, got)):
        impl(problem).backward_cpu(L1_in=in1.copy(), L1_grad=in1_grad, L2_in=in2.copy(), L2_grad=in2_grad,
                                   L3_grad=out_grad.copy(), weights=weights.copy(), weights_grad=wgrad)
    # a shared weight gradient sums over the batch: the reference scales its threshold accordingly
    # (correctness_utils.py:140-146)
    wthresh = correctness_threshold * batch_size if problem.shared_weights else correctness_threshold
    for name, a, b, thresh in (("weight_grad", ref[0], got[0], wthresh), ("in1_grad", ref[1], got[1], correctness_threshold),
                               ("in2_grad", ref[2], got[2], correctness_threshold)):
        result[name] = check_similiarity(name, a, b, thresh)
    return result


# --------------------------------------------------------------------------- the suite

class TestBenchmarkSuite:
    __test__ = False      # not a pytest class

    def __init__(self, num_warmup: int = 10, num_iter: int = 30, correctness_batch_size: int = 10_000,
                 bench_batch_size: int = 10_000_000, prng_seed: int = 12345, reference_implementation=None,
                 correctness_threshold: float = 5e-7, torch_op: bool = False):
        self.num_warmup, self.num_iter = num_warmup, num_iter
        self.correctness_batch_size, self.bench_batch_size = correctness_batch_size, bench_batch_size
        self.prng_seed = prng_seed
        self.reference_implementation = reference_implementation
        self.correctness_threshold = correctness_threshold
        self.torch_op = torch_op

    @staticmethod
    def validate_inputs(test_list) -> None:
        for impl, problem, direction, _, _ in test_list:
            assert isinstance(impl, type)
            assert direction in ("forward", "backward")

    @staticmethod
    def generate_metadata(test_list) -> dict:
        impls, tpps, directions, correctnesses, benchmarks = zip(*test_list)
        try:
            import torch
            gpu_name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "none"
        except Exception:
            gpu_name = "unknown"
        metadata = {
            "config_strs": list(dict.fromkeys(str(t) for t in tpps)),
            "config_reprs": list(dict.fromkeys(repr(t) for t in tpps)),
            "config_labels": list(dict.fromkeys(t.label for t in tpps)),
            "implementations": list(dict.fromkeys(i.name() for i in impls)),
            "directions": list(dict.fromkeys(directions)),
            "did_correctness": any(correctnesses),
            "did_benchmark": any(benchmarks),
            "gpu_name": gpu_name,
        }
        metadata["test details"] = {
            n: {"implementation": t.implementation.name(), "problem": repr(t.problem), "direction": t.direction,
                "correctness": t.correctness, "benchmark": t.benchmark} for n, t in enumerate(test_list)}
        return metadata

    def run(self, test_list, output_folder) -> pathlib.Path:
        """Runs every test and writes ``metadata.json`` plus one record per test into a new sub-folder
        (named by the time in milliseconds, as the reference does) of ``output_folder``."""
        if output_folder is None:
            raise ValueError("output folder must be specified")
        test_list = [t if isinstance(t, TestDefinition) else TestDefinition(*t) for t in test_list]
        output_folder = pathlib.Path(output_folder) / f"{round(time.time() * 1000)}"
        self.validate_inputs(test_list)
        output_folder.mkdir(parents=True)
        with open(os.path.join(output_folder, "metadata.json"), "w") as f:
            json.dump(self.generate_metadata(test_list), f, indent=2)
        for test_id, test in enumerate(test_list):
            impl, tpp = test.implementation, test.problem
            result = {"config_str": str(tpp), "config_repr": repr(tpp), "config_label": tpp.label,
                      "direction": test.direction, "implementation_name": impl.name(),
                      "correctness": str(test.correctness), "benchmark": str(test.benchmark),
                      "torch_overhead_included": self.torch_op}
            fwd = test.direction == "forward"
            if test.correctness:
                if self.reference_implementation is None:
                    result["correctness results"] = {"skipped": "no reference implementation was supplied"}
                else:
                    check = correctness_forward if fwd else correctness_backward
                    result["correctness results"] = check(tpp, impl, self.reference_implementation,
                                                          self.correctness_batch_size, self.correctness_threshold,
                                                          self.prng_seed)
            if test.benchmark:
                bench = benchmark_forward if fwd else benchmark_backward
                result["benchmark results"] = bench(tpp, impl, self.bench_batch_size, self.num_warmup, self.num_iter,
                                                    self.prng_seed, self.torch_op)
            with open(output_folder / f"{test_id}_{impl.name()}.json", "w") as f:
                json.dump(result, f, indent=2)
        return output_folder


# --------------------------------------------------------------------------- convolution records

def flops_data_per_tp(config, direction: str):
    """(flops per edge, bytes per edge, CG nonzeros), the reference's convention
    (ConvolutionBase.py:11-43): node rows are counted once per edge."""
    word = np.dtype(config.irrep_dtype).itemsize
    assert not config.shared_weights
    L1, L2, L3 = config.irreps_in1, config.irreps_in2, config.irreps_out
    ops_per_nz = 3 if direction == "forward" else 9
    words = L1.dim + L2.dim + L3.dim + config.weight_numel
    if direction == "backward":
        words += L1.dim + L2.dim + config.weight_numel
    ops, nnz = 0, 0
    for ins in config.instructions:
        l1, l2, l3 = _ls(config, ins)
        local = count_cg_non_zero(l1, l2, l3)
        nnz += local
        ops += ops_per_nz * local * L1[ins.i_in1].mul * L2[ins.i_in2].mul
        if ins.connection_mode == "uvu":
            ops += L3[ins.i_out].mul * (2 * l3 + 1)
        elif ins.connection_mode == "uvw":
            ops += L1[ins.i_in1].mul * L2[ins.i_in2].mul * L3[ins.i_out].ir.dim * L3[ins.i_out].mul
    return ops, words * word, nnz


def benchmark_conv(conv, graph, direction: str, num_warmup: int = 10, num_iter: int = 30, prng_seed: int = 12345) -> dict:
    """One record of ``ConvolutionBase.test_benchmark_forward`` / ``test_benchmark_backward``
    (ConvolutionBase.py:256-439): ``graph`` has ``rows``, ``cols``, ``nnz``, ``node_count`` and, for the
    deterministic variant, ``transpose_perm`` (a ``CoordGraph`` or ``PeriodicGraph.sender_perm``)."""
    import torch
    config = conv.config
    rng = np.random.default_rng(prng_seed)
    dt = config.irrep_dtype
    x = torch.from_numpy(np.array(rng.uniform(size=(graph.node_count, config.irreps_in1.dim)), dtype=dt)).cuda()
    y = torch.from_numpy(np.array(rng.uniform(size=(graph.nnz, config.irreps_in2.dim)), dtype=dt)).cuda()
    w = torch.from_numpy(np.array(rng.uniform(size=(graph.nnz, config.weight_numel)), dtype=dt)).cuda()
    index = [torch.from_numpy(np.ascontiguousarray(graph.rows)).cuda(), torch.from_numpy(np.ascontiguousarray(graph.cols)).cuda()]
    if conv.deterministic:
        perm = getattr(graph, "transpose_perm", None)
        perm = graph.sender_perm if perm is None else perm
        index.append(torch.from_numpy(np.ascontiguousarray(perm)).cuda())
    if direction == "forward":
        launch = lambda: conv._forward_impl(x, y, w, *index)
    else:
        dz = torch.from_numpy(np.array(rng.uniform(size=(graph.node_count, config.irreps_out.dim)), dtype=dt)).cuda()
        launch = lambda: conv._backward_impl(x, y, w, dz, *index)
    times = _time_launches(launch, num_warmup, num_iter).astype(np.float64)
    ops, data, _ = flops_data_per_tp(config, direction)
    ops += config.irreps_out.dim
    return {
        "direction": direction, "flops_per_tp": ops, "data_per_tp": data,
        "time_millis": [float(t) for t in times],
        "throughputs_gflops": [float(t) for t in graph.nnz * ops / (times * 1e6)],
        "bandwidth_gbps": [float(t) for t in graph.nnz * data / (times * 1e6)],
        "L1": str(config.irreps_in1), "L2": str(config.irreps_in2), "L3": str(config.irreps_out),
        "graph_node_count": graph.node_count, "graph_adj_nnz": graph.nnz,
        "num_warmup": num_warmup, "num_iter": num_iter, "prng_seed": prng_seed,
    }
