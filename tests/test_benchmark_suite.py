"""Benchmark records in the reference's JSON layout (openequivariance_b200.benchmark_suite)."""
import json
import os

import numpy as np
import pytest

from conftest import problem_by_name
from openequivariance_b200 import benchmark_suite as bs


def test_flop_and_byte_conventions_of_the_reference():
    """Hand-checked counts for the README shape (1x2e x 1x3e -> 1x2e, one 'uvu' path): the reference counts
    3 flops per Clebsch-Gordan nonzero plus one per output component forward, 9 per nonzero backward
    (LoopUnrollTP.py:77-105), and streams every array once (perf_metrics_utils.py:11-44)."""
    p = problem_by_name("readme")
    nnz = bs.count_cg_non_zero(2, 3, 2)
    assert nnz == bs.calculate_total_nnz(p) and nnz > 0
    fwd = bs.calculate_flops_forward(p, 10)
    assert fwd["CG_decomposition"] == 3 * nnz * 10 and fwd["linear_combination"] == 5 * 10
    assert fwd["total"] == fwd["CG_decomposition"] + fwd["linear_combination"]
    assert bs.calculate_flops_backward(p, 10)["total"] == 9 * nnz * 10
    assert bs.calculate_minimum_memory_streamed_forward(p, 10)["total"] == (5 + 7 + 5 + 1) * 4 * 10
    assert bs.calculate_minimum_memory_streamed_backward(p, 10)["total"] == (2 * 5 + 2 * 7 + 5 + 2 * 1) * 4 * 10
    ops, data, n = bs.flops_data_per_tp(p, "forward")
    assert (ops, data, n) == (3 * nnz + 5, (5 + 7 + 5 + 1) * 4, nnz)
    ops, data, n = bs.flops_data_per_tp(p, "backward")
    assert (ops, data) == (9 * nnz + 5, (2 * 5 + 2 * 7 + 5 + 2 * 1) * 4)
    # 'uvw' uses the "minimum" count: outer products + 2 flops per nonzero per (u, v) + 2 per weight and component
    q = problem_by_name("uvw_small")
    f = bs.calculate_flops_forward(q, 1)
    assert f["total"] == f["outer_products"] + f["CG_decomposition"] + f["linear_combination"]
    assert f["linear_combination"] == 2 * sum((2 * q.irreps_out[i.i_out].ir.l + 1) * int(np.prod(i.path_shape))
                                              for i in q.instructions)


def test_conventions_match_numbers_computed_by_the_reference():
    """tests/golden/bench_conventions.json holds the reference's own functions evaluated on the named problems
    (batch 7): total nonzeros, "minimum" forward flops, streamed bytes, per-edge convolution counts."""
    from conftest import GOLDEN, golden_problems, build_problem
    with open(os.path.join(GOLDEN, "bench_conventions.json")) as f:
        want = json.load(f)
    for entry in golden_problems():
        p, ref = build_problem(entry), want[entry["name"]]
        assert bs.calculate_total_nnz(p) == ref["total_cg_nnz"]
        assert bs.calculate_minimum_flops_forward(p, 7) == ref["minimum_flops_forward"]
        assert bs.calculate_minimum_memory_streamed_forward(p, 7) == ref["memory_forward"]
        assert bs.calculate_minimum_memory_streamed_backward(p, 7) == ref["memory_backward"]
        if not p.shared_weights:
            for direction in ("forward", "backward"):
                assert list(bs.flops_data_per_tp(p, direction)) == ref[f"conv_{direction}"]


def test_seeded_buffers_follow_the_reference_draw_order():
    p = problem_by_name("readme")
    in1, in2, w, out = bs.get_random_buffers_forward(p, 1000, 12345)
    rng = np.random.default_rng(12345)
    assert np.array_equal(in1, rng.uniform(size=(1000, 5)).astype(np.float32))
    assert np.array_equal(in2, rng.uniform(size=(1000, 7)).astype(np.float32))
    assert np.array_equal(w, rng.uniform(size=(1000, 1)).astype(np.float32)) and not out.any()


def test_statistics_record_has_the_reference_keys():
    p = problem_by_name("nequip_32")
    rec = bs.calculate_performance_statistics(p, 100, 2.0e6, 4.0e5, np.array([0.5, 1.0]))
    assert set(rec) == {"total_cg_nnz", "flops_per_tp", "L1", "L2", "L3", "L1_rep_len", "L2_rep_len", "L3_rep_len",
                        "rep_dtype", "weight_dtype", "arithmetic_intensity (FLOPs / byte)", "batch_size",
                        "time_millis", "throughputs_gflops", "bandwidth_gbps"}
    assert rec["throughputs_gflops"] == [4.0, 2.0] and rec["bandwidth_gbps"] == [0.8, 0.4]
    assert rec["arithmetic_intensity (FLOPs / byte)"] == 5.0
    sim = bs.check_similiarity("output", np.zeros(3), np.array([0.0, 1e-8, 0.0]), 5e-7)
    assert sim == {"shape_match": True, "diff_Linf_norm": 1e-8, "pass": True}
    assert bs.check_similiarity("output", np.zeros(3), np.zeros(4), 1.0)["pass"] is False


class OracleTP:
    """Reference implementation for the suite's correctness checks: the float64 CPU oracle behind the
    host-array entry points of the reference's classes."""

    def __init__(self, problem, torch_op=False):
        self.p = problem

    @staticmethod
    def name():
        return "OracleTP"

    def forward_cpu(self, L1_in, L2_in, L3_out, weights):
        from oracle import tp_oracle as orc
        L3_out[:] = orc.tp_forward(self.p, L1_in, L2_in, weights)

    def backward_cpu(self, L1_in, L1_grad, L2_in, L2_grad, L3_grad, weights, weights_grad):
        from oracle import tp_oracle as orc
        dx, dy, dw = orc.tp_backward(self.p, L1_in, L2_in, weights, L3_grad)
        L1_grad[:], L2_grad[:], weights_grad[:] = dx, dy, dw


@pytest.mark.gpu
def test_suite_writes_the_reference_layout(tmp_path):
    import openequivariance_b200 as oeq
    from openequivariance_b200.graph import periodic_radius_graph
    problems = [problem_by_name("nequip_32"), problem_by_name("uvw_small")]
    tests = [bs.TestDefinition(oeq.TensorProduct, p, d, True, True) for p in problems for d in ("forward", "backward")]
    suite = bs.TestBenchmarkSuite(num_warmup=2, num_iter=3, correctness_batch_size=64, bench_batch_size=2000,
                                  reference_implementation=OracleTP, correctness_threshold=5e-5, torch_op=True)
    folder = suite.run(tests, tmp_path)
    names = sorted(os.listdir(folder))
    assert names == ["0_LoopUnrollTP.json", "1_LoopUnrollTP.json", "2_LoopUnrollTP.json", "3_LoopUnrollTP.json",
                     "metadata.json"]
    meta = json.load(open(folder / "metadata.json"))
    assert meta["implementations"] == ["LoopUnrollTP"] and meta["directions"] == ["forward", "backward"]
    assert meta["did_correctness"] and meta["did_benchmark"] and len(meta["test details"]) == 4
    for n, direction in enumerate(["forward", "backward", "forward", "backward"]):
        rec = json.load(open(folder / f"{n}_LoopUnrollTP.json"))
        assert rec["direction"] == direction and rec["implementation_name"] == "LoopUnrollTP"
        bench = rec["benchmark results"]
        assert bench["tp_direction"] == direction and len(bench["time_millis"]) == 3 and bench["batch_size"] == 2000
        assert all(t > 0 for t in bench["time_millis"])
        checks = rec["correctness results"]
        keys = ["output"] if direction == "forward" else ["weight_grad", "in1_grad", "in2_grad"]
        assert all(checks[k]["pass"] for k in keys), checks
    # convolution record (ConvolutionBase.calculate_bench_stats)
    g = periodic_radius_graph(500, 20.0, seed=3)
    for det in (False, True):
        conv = oeq.TensorProductConv(problems[0], torch_op=True, deterministic=det)
        for direction in ("forward", "backward"):
            rec = bs.benchmark_conv(conv, g, direction, num_warmup=1, num_iter=2)
            assert set(rec) == {"direction", "flops_per_tp", "data_per_tp", "time_millis", "throughputs_gflops",
                                "bandwidth_gbps", "L1", "L2", "L3", "graph_node_count", "graph_adj_nnz", "num_warmup",
                                "num_iter", "prng_seed"}
            assert rec["graph_adj_nnz"] == g.nnz and len(rec["time_millis"]) == 2 and min(rec["time_millis"]) > 0
