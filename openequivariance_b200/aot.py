"""Ahead-of-time specialisation of the kernels of well-known problems.

Kernels are normally specialised the first time a problem is used and cached on
disk; doing it for the benchmark configurations and the test problems at build
time means a fresh machine does not pay for it.  The cache lives beside the
library (``_kcache/``) and is keyed by a hash of the problem tables and of the
kernel headers, so stale entries are simply never hit.
"""

from __future__ import annotations

import os
from concurrent.futures import ProcessPoolExecutor

import numpy as np

from . import _native
from .problem import ChannelwiseTPP, FullyConnectedTPProblem, SingleInstruction, TPProblem

BATCH, DET, ATOMIC = _native.KIND_BATCH, _native.KIND_CONV_DET, _native.KIND_CONV_ATOMIC


def named_problems():
    """(label, constructor, kinds) of the benchmark configurations."""
    return [
        ("readme", lambda dt: TPProblem("1x2e", "1x3e", "1x2e", [(0, 0, 0, "uvu", True)], shared_weights=False,
                                        internal_weights=False, irrep_dtype=dt, weight_dtype=dt), BATCH | DET | ATOMIC),
        ("mace_128", lambda dt: ChannelwiseTPP("128x0e+128x1o+128x2e", "1x0e+1x1o+1x2e+1x3o",
                                               "128x0e+128x1o+128x2e", irrep_dtype=dt, weight_dtype=dt),
         BATCH | DET | ATOMIC),
        ("nequip_32", lambda dt: ChannelwiseTPP("32x0e+32x1o+32x2e", "0e+1o+2e", "32x0e+32x1o+32x2e",
                                                irrep_dtype=dt, weight_dtype=dt), BATCH | DET | ATOMIC),
        ("uvw_64", lambda dt: FullyConnectedTPProblem("64x0e+64x1o+64x2e", "0e+1o+2e", "64x0e+64x1o+64x2e",
                                                      irrep_dtype=dt, weight_dtype=dt), BATCH),
        ("mace_large_128", lambda dt: ChannelwiseTPP("128x0e+128x1o+128x2e+128x3o", "1x0e+1x1o+1x2e+1x3o",
                                                     "128x0e+128x1o+128x2e+128x3o", irrep_dtype=dt,
                                                     weight_dtype=dt), BATCH | DET | ATOMIC),
    ]


def _build_entry(entry, dt):
    """A problem from a description ``{"kind", "args", "kwargs"}`` (kinds: tpp, channelwise, fully_connected,
    single)."""
    kind, args, kwargs = entry["kind"], entry["args"], dict(entry["kwargs"])
    kwargs.update(irrep_dtype=dt, weight_dtype=dt)
    if kind == "tpp":
        a, b, c, instr = args
        return TPProblem(a, b, c, [tuple(i) for i in instr], **kwargs)
    if kind == "channelwise":
        return ChannelwiseTPP(*args, **kwargs)
    if kind == "single":
        return SingleInstruction(*args, **kwargs)
    return FullyConnectedTPProblem(*args, **kwargs)


def _jobs(extra):
    jobs = []
    for n, (_, make, kinds) in enumerate(named_problems()):
        jobs.append(("named", n, None, "f32", kinds))
    for entry in extra:
        conv_ok = entry["kind"] == "channelwise" or entry.get("name") == "readme"
        for dt in ("f32", "f64"):
            jobs.append(("extra", 0, entry, dt, BATCH | ((DET | ATOMIC) if conv_ok else 0)))
    return jobs


def _run(job):
    source, n, entry, dt_name, kinds = job
    dt = np.float32 if dt_name == "f32" else np.float64
    problem = named_problems()[n][1](dt) if source == "named" else _build_entry(entry, dt)
    for bit in (BATCH, DET, ATOMIC):
        if kinds & bit:
            try:
                # convolutions: with the two second-derivative kernels, where the problem has them
                _native.precompile(problem, bit if bit == BATCH else bit | _native.KIND_CONV_SECOND)
            except _native.OeqError as err:
                if err.code != 2:  # "unsupported problem" is a property of the problem, not a build failure
                    raise
    # shared-weight 'uvw' problems with a second input of multiplicity 1 also serve as graph convolutions:
    # the unit-weight edge sum and the dense stage (conv.UVWConvPlan)
    if (problem.shared_weights and all(i.connection_mode == "uvw" for i in problem.instructions)
            and all(mul == 1 for mul, _ in problem.irreps_in2)):
        from .conv import UVWConvPlan
        plan = UVWConvPlan(problem)
        try:
            _native.precompile(plan.edge_sum, DET | ATOMIC, unit_weights=True)
            _native.precompile(plan.dense, BATCH)
        except _native.OeqError as err:
            if err.code != 2:
                raise
    return job


def precompile_all(extra_problems=(), workers: int | None = None):
    """Specialise the kernels of the benchmark configurations and of ``extra_problems`` (problem descriptions
    as in ``_build_entry``; the build entry point hands in the test suite's list)."""
    _native.lib()  # build/load once in the parent so the children find the library
    jobs = _jobs(list(extra_problems))
    workers = workers or min(len(jobs), os.cpu_count() or 1)
    import multiprocessing
    # spawn: the children must not inherit the parent's loaded compiler library across a fork
    with ProcessPoolExecutor(max_workers=workers, mp_context=multiprocessing.get_context("spawn")) as pool:
        list(pool.map(_run, jobs))
    return len(jobs)
