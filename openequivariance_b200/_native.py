"""ctypes binding of ``liboeq_b200.so`` (C ABI declared in ``include/oeq_b200.h``).

This is the counterpart of the reference's pybind11 module import
(reference: openequivariance/extlib/__init__.py:22-65): the library is built
in-tree with nvcc on first use if it is missing, and every failure surfaces as
a Python exception carrying ``oeq_last_error()``.  There is no fallback path:
if the library cannot be built or loaded the operators do not work.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

import numpy as np

from .wigner import cg_nonzeros

OEQ_OK = 0
OEQ_ERR_UNSUPPORTED = 2
ERR_NAMES = {1: "invalid argument", 2: "unsupported problem", 3: "kernel specialisation failed",
             4: "CUDA error", 5: "device-side wait abandoned"}

KIND_BATCH, KIND_CONV_DET, KIND_CONV_ATOMIC = 1, 2, 4
KIND_CONV_SECOND = 8    # with a convolution kind: also the second-derivative kernels of that convolution


class OeqError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"oeq_b200: {ERR_NAMES.get(code, code)}: {message}")
        self.code = code


class _Irrep(C.Structure):
    _fields_ = [("mul", C.c_int32), ("l", C.c_int32), ("parity", C.c_int32)]


class _Instruction(C.Structure):
    _fields_ = [("i_in1", C.c_int32), ("i_in2", C.c_int32), ("i_out", C.c_int32), ("mode", C.c_int32),
                ("path_weight", C.c_double), ("cg_nnz", C.c_int32),
                ("cg_i", C.POINTER(C.c_int32)), ("cg_j", C.POINTER(C.c_int32)), ("cg_k", C.POINTER(C.c_int32)),
                ("cg_value", C.POINTER(C.c_double))]


class _ProblemDesc(C.Structure):
    _fields_ = [("n_in1", C.c_int32), ("n_in2", C.c_int32), ("n_out", C.c_int32), ("n_instr", C.c_int32),
                ("in1", C.POINTER(_Irrep)), ("in2", C.POINTER(_Irrep)), ("out", C.POINTER(_Irrep)),
                ("instr", C.POINTER(_Instruction)), ("dtype", C.c_int32), ("shared_weights", C.c_int32)]


# every symbol include/oeq_b200.h declares: name -> (restype, argtypes)
_P, _I64, _SZ, _INT = C.c_void_p, C.c_int64, C.c_size_t, C.c_int
_PI = C.POINTER(C.c_int)
SYMBOLS = {
    "oeq_version": (C.c_char_p, []),
    "oeq_last_error": (C.c_char_p, []),
    "oeq_set_kernel_dir": (_INT, [C.c_char_p]),
    "oeq_set_cache_dir": (_INT, [C.c_char_p]),
    "oeq_precompile": (_INT, [C.POINTER(_ProblemDesc), _INT]),
    "oeq_tp_create": (_INT, [C.POINTER(_ProblemDesc), C.POINTER(_P)]),
    "oeq_tp_destroy": (_INT, [_P]),
    "oeq_tp_weight_numel": (_I64, [_P]),
    "oeq_tp_forward": (_INT, [_P, _I64, _P, _P, _P, _P, _P]),
    "oeq_tp_workspace_bytes": (_SZ, [_P, _I64]),
    "oeq_tp_backward": (_INT, [_P, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _SZ, _P]),
    "oeq_tp_backward_noalloc": (_INT, [_P, _I64, _P, _P, _P, _P, _P, _P, _P, _P]),
    "oeq_tp_has_double_backward": (_INT, [_P]),
    "oeq_tp_double_backward": (_INT, [_P, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "oeq_tp_check": (_INT, [_P]),
    "oeq_conv_create": (_INT, [C.POINTER(_ProblemDesc), _INT, C.POINTER(_P)]),
    "oeq_conv_destroy": (_INT, [_P]),
    "oeq_conv_workspace_bytes": (_SZ, [_P, _I64, _I64]),
    "oeq_conv_forward": (_INT, [_P, _I64, _I64, _P, _P, _P, _P, _P, _P, _P, _SZ, _P]),
    "oeq_conv_backward": (_INT, [_P, _I64, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _SZ, _P]),
    "oeq_conv_check": (_INT, [_P]),
    "oeq_conv_last_backward_launches": (_INT, [_P]),
    "oeq_conv_has_double_backward": (_INT, [_P]),
    "oeq_conv_double_backward": (_INT, [_P, _I64, _I64] + [_P] * 14 + [_P, _SZ, _P]),
    "oeq_selftest_bounded_wait": (_INT, [_INT, _P]),
    "oeq_tp_launch_info": (_INT, [_P, _INT, _PI, _PI, _PI, _PI, _PI, _PI]),
    "oeq_conv_launch_info": (_INT, [_P, _INT, _PI, _PI, _PI, _PI, _PI, _PI]),
}

_lib = None
_lock = threading.Lock()


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "liboeq_b200.so")


def lib():
    """Load (building first if needed) the shared library; raises if impossible."""
    global _lib
    with _lock:
        if _lib is None:
            from .build import build_library
            path = build_library()
            handle = C.CDLL(path)
            for name, (restype, argtypes) in SYMBOLS.items():
                fn = getattr(handle, name)
                fn.restype, fn.argtypes = restype, argtypes
            _lib = handle
    return _lib


def check(code: int):
    if code != OEQ_OK:
        raise OeqError(code, lib().oeq_last_error().decode(errors="replace"))


class Descriptor:
    """Owns the ctypes arrays behind one ``oeq_problem_desc``."""

    def __init__(self, problem, unit_weights=False):
        modes = {ins.connection_mode for ins in problem.instructions}
        if len(problem.instructions) == 0:
            raise ValueError("Tensor product problem has no valid intructions!")
        assert len(modes) == 1, "all instructions must use the same connection mode"
        mode = modes.pop()
        assert mode in ("uvu", "uvw"), f"connection mode {mode!r} is not supported (uvu and uvw are)"
        assert problem.irrep_dtype == problem.weight_dtype, "irrep_dtype and weight_dtype must match"
        assert problem.irrep_dtype in (np.float32, np.float64)
        for ins in problem.instructions:
            assert ins.has_weight, "every instruction must carry weights"
        self._keep = []

        def irreps(src):
            arr = (_Irrep * max(1, len(src)))()
            for n, (mul, ir) in enumerate(src):
                arr[n] = _Irrep(mul, ir.l, ir.p)
            self._keep.append(arr)
            return arr

        in1, in2, out = irreps(problem.irreps_in1), irreps(problem.irreps_in2), irreps(problem.irreps_out)
        instr = (_Instruction * len(problem.instructions))()
        for n, ins in enumerate(problem.instructions):
            l1 = problem.irreps_in1[ins.i_in1].ir.l
            l2 = problem.irreps_in2[ins.i_in2].ir.l
            l3 = problem.irreps_out[ins.i_out].ir.l
            nz = cg_nonzeros(l1, l2, l3)
            ci = (C.c_int32 * len(nz))(*[t[0] for t in nz])
            cj = (C.c_int32 * len(nz))(*[t[1] for t in nz])
            ck = (C.c_int32 * len(nz))(*[t[2] for t in nz])
            cv = (C.c_double * len(nz))(*[t[3] for t in nz])
            self._keep += [ci, cj, ck, cv]
            instr[n] = _Instruction(ins.i_in1, ins.i_in2, ins.i_out, 0 if mode == "uvu" else 1,
                                    float(ins.path_weight), len(nz), ci, cj, ck, cv)
        self._keep.append(instr)
        self.struct = _ProblemDesc(len(problem.irreps_in1), len(problem.irreps_in2), len(problem.irreps_out),
                                   len(problem.instructions), in1, in2, out, instr,
                                   1 if problem.irrep_dtype == np.float64 else 0,
                                   2 if unit_weights else (1 if problem.shared_weights else 0))

    def ref(self):
        return C.byref(self.struct)


def precompile(problem, kinds: int, unit_weights: bool = False):
    """Specialise the kernels of ``problem`` into the on-disk cache (no GPU needed)."""
    d = Descriptor(problem, unit_weights=unit_weights)
    check(lib().oeq_precompile(d.ref(), kinds))


class _Handle:
    _destroy = None

    def __init__(self):
        self.ptr = _P()

    def __del__(self):
        try:
            if self.ptr and _lib is not None:
                getattr(_lib, self._destroy)(self.ptr)
        except Exception:
            pass

    def _info(self, fn, which):
        vals = [C.c_int() for _ in range(6)]
        check(fn(self.ptr, which, *[C.byref(v) for v in vals]))
        keys = ("threads", "groups_per_cta", "partitions", "stages", "smem_bytes", "registers")
        return dict(zip(keys, (v.value for v in vals)))


class TPHandle(_Handle):
    _destroy = "oeq_tp_destroy"

    def __init__(self, problem):
        super().__init__()
        self.desc = Descriptor(problem)
        check(lib().oeq_tp_create(self.desc.ref(), C.byref(self.ptr)))

    def forward(self, batch, x, y, w, z, stream):
        check(lib().oeq_tp_forward(self.ptr, batch, x, y, w, z, stream))

    def workspace_bytes(self, batch):
        return lib().oeq_tp_workspace_bytes(self.ptr, batch)

    def backward(self, batch, x, y, w, dz, dx, dy, dw, ws, ws_bytes, stream):
        check(lib().oeq_tp_backward(self.ptr, batch, x, y, w, dz, dx, dy, dw, ws, ws_bytes, stream))

    def has_double_backward(self):
        return bool(lib().oeq_tp_has_double_backward(self.ptr))

    def double_backward(self, batch, x, y, w, dz, ex, ey, ew, gx, gy, gw, gdz, stream):
        check(lib().oeq_tp_double_backward(self.ptr, batch, x, y, w, dz, ex, ey, ew, gx, gy, gw, gdz, stream))

    def check(self):
        check(lib().oeq_tp_check(self.ptr))

    def launch_info(self, which):
        return self._info(lib().oeq_tp_launch_info, which)


class ConvHandle(_Handle):
    _destroy = "oeq_conv_destroy"

    def __init__(self, problem, deterministic, unit_weights=False):
        super().__init__()
        self.desc = Descriptor(problem, unit_weights=unit_weights)
        check(lib().oeq_conv_create(self.desc.ref(), 1 if deterministic else 0, C.byref(self.ptr)))

    def workspace_bytes(self, nodes, edges):
        return lib().oeq_conv_workspace_bytes(self.ptr, nodes, edges)

    def forward(self, nodes, edges, x, y, w, rows, cols, z, ws, ws_bytes, stream):
        check(lib().oeq_conv_forward(self.ptr, nodes, edges, x, y, w, rows, cols, z, ws, ws_bytes, stream))

    def backward(self, nodes, edges, x, y, w, dz, rows, cols, perm, dx, dy, dw, ws, ws_bytes, stream):
        check(lib().oeq_conv_backward(self.ptr, nodes, edges, x, y, w, dz, rows, cols, perm, dx, dy, dw,
                                      ws, ws_bytes, stream))

    def check(self):
        check(lib().oeq_conv_check(self.ptr))

    def last_backward_launches(self):
        return int(lib().oeq_conv_last_backward_launches(self.ptr))

    def has_double_backward(self):
        return bool(lib().oeq_conv_has_double_backward(self.ptr))

    def double_backward(self, nodes, edges, x, y, w, dz, ex, ey, ew, rows, cols, perm, gx, gy, gw, gdz,
                        ws, ws_bytes, stream):
        check(lib().oeq_conv_double_backward(self.ptr, nodes, edges, x, y, w, dz, ex, ey, ew, rows, cols, perm,
                                             gx, gy, gw, gdz, ws, ws_bytes, stream))

    def launch_info(self, which):
        return self._info(lib().oeq_conv_launch_info, which)
