import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def golden_problems():
    with open(os.path.join(GOLDEN, "problems.json")) as f:
        return json.load(f)


def build_problem(entry, **overrides):
    """Build one of the named golden problems with this package's classes."""
    import openequivariance_b200 as oeq
    kind, args, kwargs = entry["kind"], entry["args"], dict(entry["kwargs"])
    kwargs.update(overrides)
    if kind == "tpp":
        a, b, c, instr = args
        return oeq.TPProblem(a, b, c, [tuple(i) for i in instr], **kwargs)
    if kind == "channelwise":
        return oeq.ChannelwiseTPP(*args, **kwargs)
    if kind == "fully_connected":
        return oeq.FullyConnectedTPProblem(*args, **kwargs)
    if kind == "single":
        return oeq.SingleInstruction(*args, **kwargs)
    raise ValueError(kind)


def problem_by_name(name, **overrides):
    for entry in golden_problems():
        if entry["name"] == name:
            return build_problem(entry, **overrides)
    raise KeyError(name)


@pytest.fixture(scope="session")
def problems():
    return {e["name"]: e for e in golden_problems()}
