"""Builds ``liboeq_b200.so`` (the C-ABI runtime) in-tree with nvcc for sm_100a.

The library holds the host runtime and the fixed kernels; the problem-specific
kernels are specialised at run time from ``csrc/*.cuh`` and cached under
``_kcache/``.  ``python -m openequivariance_b200.build`` rebuilds the library.
"""

from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "liboeq_b200.so")
SOURCES = ["oeq_runtime.cu"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the CUDA toolkit is required to build liboeq_b200.so")


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + [os.path.join(HERE, "..", "include", "oeq_b200.h")]
    return any(os.path.getmtime(d) > built for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Build the library if it is missing or older than its sources.

    Several processes may get here at once (one rank per GPU under ``torch.distributed.run``): the build
    runs under an exclusive lock on a sidecar file, writes to a temporary name and is renamed into place,
    so no process ever loads a half-written library; whoever waited for the lock re-checks and usually
    finds the work done.
    """
    if not force and not needs_build():
        return LIB
    import fcntl
    with open(LIB + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not needs_build():
                return LIB
            tmp = f"{LIB}.tmp{os.getpid()}"
            cmd = [_nvcc(), "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-lineinfo",
                   "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
                   "-o", tmp] + [os.path.join(CSRC, s) for s in SOURCES] + ["-ldl"]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            if os.environ.get("OEQ_DEV_PROFILE"):
                cmd.insert(1, "-DOEQ_DEV_PROFILE")      # development build: cycle accounting inside the kernels
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError("building liboeq_b200.so failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
            os.replace(tmp, LIB)
            if verbose:
                print(res.stdout + res.stderr)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
