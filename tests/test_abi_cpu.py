"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT, problem_by_name


def header_functions():
    text = open(os.path.join(ROOT, "include", "oeq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(oeq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from openequivariance_b200 import _native
    lib = _native.lib()
    names = header_functions()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/oeq_b200.h but not exported"
        assert name in _native.SYMBOLS, f"{name} has no ctypes signature"
    assert b"sm_100a" in lib.oeq_version()


def test_descriptor_errors_are_reported_not_fatal():
    from openequivariance_b200 import _native
    lib = _native.lib()
    out = ctypes.c_void_p()
    assert lib.oeq_tp_create(None, ctypes.byref(out)) == 1
    assert b"null" in lib.oeq_last_error()
    p = problem_by_name("uvw_small")
    d = _native.Descriptor(p)
    d.struct.dtype = 7
    assert lib.oeq_tp_create(d.ref(), ctypes.byref(out)) == 1
    # a fused convolution over a 'uvw' problem is outside the supported set
    d2 = _native.Descriptor(p)
    assert lib.oeq_conv_create(d2.ref(), 1, ctypes.byref(out)) == 2
    assert b"uvu" in lib.oeq_last_error()


def test_front_end_rejects_what_the_reference_rejects():
    import openequivariance_b200 as oeq
    with pytest.raises(AssertionError):      # mixed connection modes
        oeq.TensorProduct(oeq.TPProblem("2x0e", "2x0e", "2x0e", [(0, 0, 0, "uvu", True), (0, 0, 0, "uvw", True)],
                                        shared_weights=False, internal_weights=False), torch_op=True)
    with pytest.raises(AssertionError):      # conv needs multiplicity 1 in the second input
        oeq.TensorProductConv(problem_by_name("uvu_v2"), torch_op=True)
    with pytest.raises(AssertionError):      # dtypes must agree
        oeq.TensorProduct(problem_by_name("readme", irrep_dtype=np.float64), torch_op=True)


def test_kernels_specialise_without_a_gpu(tmp_path):
    """Run-time specialisation (NVRTC for sm_100a) needs no device; the cache is keyed by content."""
    from openequivariance_b200 import _native
    lib = _native.lib()
    lib.oeq_set_cache_dir(str(tmp_path).encode())
    try:
        _native.precompile(problem_by_name("readme"), _native.KIND_BATCH | _native.KIND_CONV_DET)
        files = sorted(os.listdir(tmp_path))
        # batch forward / backward / one-pass second derivatives, convolution forward, sender-order and
        # receiver-order backward
        assert len(files) == 6 and all(f.endswith(".cubin") for f in files)
        _native.precompile(problem_by_name("readme"), _native.KIND_BATCH)
        assert sorted(os.listdir(tmp_path)) == files
    finally:
        lib.oeq_set_cache_dir(os.path.join(os.path.dirname(_native.library_path()), "_kcache").encode())
