"""Float64 CPU restatement of the tensor product and the graph convolution.

TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline; never a product path).

What is restated, and from where in the reference project:

* the tensor-product contraction of ``e3nn.o3.TensorProduct`` as the reference
  states it in numpy for "uvu"
  (openequivariance/implementations/NumpyTensorProduct.py:18-46, einsum
  ``bui,bvj,buv,ijk->buvk`` with ``C = wigner_3j * path_weight``), extended to
  "uvw" and to shared weights with the same index convention: weights are in
  e3nn order, instruction-major, block shape ``path_shape``
  (openequivariance/implementations/e3nn_lite.py:519,566-571);
* the unfused convolution ``scatter_sum(tp(X[cols], Y, W), rows)``
  (openequivariance/implementations/convolution/E3NNConv.py:38-40,
  openequivariance/implementations/convolution/scatter.py:22-43);
* the canonical edge order and transpose permutation of ``CoordGraph``
  (openequivariance/implementations/convolution/ConvolutionBase.py:45-70);
* the e3nn<->kernel weight permutation
  (openequivariance/implementations/ComputationSchedule.py:146-230,427-471),
  written here as explicit loops, independently of the package's vectorised
  version.

Pinning: the Clebsch-Gordan tensors are read from ``tests/golden/wigner_3j.npz``,
which was produced by the reference's own generator
(openequivariance/implementations/e3nn_lite.py:593-649); the contraction is
checked in ``tests/test_oracle_golden.py`` against outputs of the reference's
``NumpyTensorProduct.forward_cpu``, ``reorder_weights``, ``CoordGraph`` and
``scatter_sum`` run in the build container (``tests/golden/make_golden.py``).
The reference's ground truth proper (e3nn) is a third-party package that is
not installed, so "uvw", shared weights and all backward passes are pinned only
through the shared index convention and autograd of the pinned forward.

Problems are duck-typed: any object with ``irreps_in1/2/out`` (iterables of
``(mul, (l, p))``), ``instructions`` (``i_in1, i_in2, i_out, connection_mode,
has_weight, path_weight, path_shape``) and ``shared_weights`` works.
"""

from __future__ import annotations

import os
from math import prod

import numpy as np
import torch

_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "tests", "golden",
                       "wigner_3j.npz")
_cg_cache = {}


def cg(l1: int, l2: int, l3: int) -> np.ndarray:
    """Reference-generated real Wigner 3j tensor (float64)."""
    if not _cg_cache:
        with np.load(_GOLDEN) as data:
            for key in data.files:
                _cg_cache[key] = data[key]
    key = f"{l1}_{l2}_{l3}"
    if key not in _cg_cache:
        raise KeyError(f"no reference Clebsch-Gordan tensor stored for l=({l1},{l2},{l3})")
    return _cg_cache[key]


def _layout(irreps):
    """[(mul, l, offset)] for each entry of an irreps-like iterable."""
    out, off = [], 0
    for mul, ir in irreps:
        l = ir[0]
        out.append((int(mul), int(l), off))
        off += int(mul) * (2 * int(l) + 1)
    return out, off


def tp_torch(problem, x, y, w, e3nn_style_pairs: bool = False, fold_second_input: bool = False):
    """Differentiable tensor product on torch tensors; ``w`` in e3nn order.

    ``w`` is ``[numel]`` when ``problem.shared_weights`` else ``[B, numel]``.
    The two flags select other, algebraically identical contraction orders:
    ``e3nn_style_pairs`` forms the outer product of the inputs first (the order in which
    e3nn's generated code is written); ``fold_second_input`` contracts the second input
    with the Clebsch-Gordan tensor first and then does one batched matmul per instruction
    (the cheapest order on a CPU when the second input has multiplicity 1, which is what
    an einsum path optimiser picks; used for the timed CPU baseline).
    """
    in1, _ = _layout(problem.irreps_in1)
    in2, _ = _layout(problem.irreps_in2)
    out, zdim = _layout(problem.irreps_out)
    batch = x.shape[0]
    blocks = [None] * len(out)          # per output irrep: sum of its instructions' results
    shared = w.dim() == 1
    woff = 0
    pair_cache = {}
    for ins in problem.instructions:
        m1, l1, o1 = in1[ins.i_in1]
        m2, l2, o2 = in2[ins.i_in2]
        m3, l3, o3 = out[ins.i_out]
        d1, d2, d3 = 2 * l1 + 1, 2 * l2 + 1, 2 * l3 + 1
        c = torch.as_tensor(cg(l1, l2, l3) * ins.path_weight, dtype=x.dtype)
        xs = x[:, o1:o1 + m1 * d1].reshape(batch, m1, d1)
        ys = y[:, o2:o2 + m2 * d2].reshape(batch, m2, d2)
        n = prod(ins.path_shape)
        wb = w[..., woff:woff + n]
        woff += n
        mode = ins.connection_mode
        if fold_second_input and m2 == 1 and mode == "uvu":
            folded = torch.einsum("bj,ijk->bik", ys[:, 0, :], c)          # [B, d1, d3]
            r = torch.bmm(xs, folded)                                      # [B, m1, d3]
            wv = wb.reshape(m1) if shared else wb.reshape(batch, m1)
            r = r * (wv.unsqueeze(-1) if not shared else wv.reshape(1, m1, 1))
        elif e3nn_style_pairs:
            # e3nn forms the outer product of the two inputs once per (in1, in2) pair
            key = (ins.i_in1, ins.i_in2)
            if key not in pair_cache:
                pair_cache[key] = torch.einsum("bui,bvj->buvij", xs, ys)
            xy = pair_cache[key]
            if mode == "uvu":
                wv = wb.reshape(m1, m2) if shared else wb.reshape(batch, m1, m2)
                r = torch.einsum("uv,ijk,buvij->buk" if shared else "buv,ijk,buvij->buk", wv, c, xy)
            else:
                wv = wb.reshape(m1, m2, m3) if shared else wb.reshape(batch, m1, m2, m3)
                r = torch.einsum("uvw,ijk,buvij->bwk" if shared else "buvw,ijk,buvij->bwk", wv, c, xy)
        else:
            t = torch.einsum("bui,bvj,ijk->buvk", xs, ys, c)
            if mode == "uvu":
                wv = wb.reshape(m1, m2) if shared else wb.reshape(batch, m1, m2)
                r = torch.einsum("buvk,uv->buk" if shared else "buvk,buv->buk", t, wv)
            elif mode == "uvw":
                wv = wb.reshape(m1, m2, m3) if shared else wb.reshape(batch, m1, m2, m3)
                r = torch.einsum("buvk,uvw->bwk" if shared else "buvk,buvw->bwk", t, wv)
            else:
                raise ValueError(f"oracle covers 'uvu' and 'uvw', got {mode!r}")
        r = r.reshape(batch, m3 * d3)
        blocks[ins.i_out] = r if blocks[ins.i_out] is None else blocks[ins.i_out] + r
    for n, (m3, l3, _) in enumerate(out):
        if blocks[n] is None:           # an output irrep that no instruction writes is zero
            blocks[n] = x.new_zeros(batch, m3 * (2 * l3 + 1))
    return torch.cat(blocks, dim=1) if blocks else x.new_zeros(batch, zdim)


def _t(a, dtype=torch.float64, grad=False):
    t = torch.as_tensor(np.asarray(a), dtype=dtype).clone()
    return t.requires_grad_(grad)


def tp_forward(problem, x, y, w, dtype=torch.float64) -> np.ndarray:
    with torch.no_grad():
        return tp_torch(problem, _t(x, dtype), _t(y, dtype), _t(w, dtype)).numpy()


def tp_backward(problem, x, y, w, dz, dtype=torch.float64):
    xt, yt, wt = _t(x, dtype, True), _t(y, dtype, True), _t(w, dtype, True)
    z = tp_torch(problem, xt, yt, wt)
    z.backward(_t(dz, dtype))
    return xt.grad.numpy(), yt.grad.numpy(), wt.grad.numpy()


def scatter_sum_rows(src, index, dim_size):
    """``zeros(dim_size, F).scatter_add_(0, index broadcast, src)``."""
    out = src.new_zeros(dim_size, src.shape[1])
    return out.index_add(0, index, src) if src.requires_grad else out.scatter_add_(
        0, index.unsqueeze(-1).expand_as(src), src)


def conv_torch(problem, x, y, w, rows, cols, e3nn_style_pairs: bool = False, fold_second_input: bool = False):
    """Gather sender rows, tensor product per edge, sum into receiver rows."""
    messages = tp_torch(problem, x[cols], y, w, e3nn_style_pairs, fold_second_input)
    out = x.new_zeros(x.shape[0], messages.shape[1])
    return out.index_add(0, rows, messages)


def conv_forward(problem, x, y, w, rows, cols, dtype=torch.float64) -> np.ndarray:
    r = torch.as_tensor(np.asarray(rows), dtype=torch.int64)
    c = torch.as_tensor(np.asarray(cols), dtype=torch.int64)
    with torch.no_grad():
        return conv_torch(problem, _t(x, dtype), _t(y, dtype), _t(w, dtype), r, c).numpy()


def conv_backward(problem, x, y, w, dz, rows, cols, dtype=torch.float64):
    r = torch.as_tensor(np.asarray(rows), dtype=torch.int64)
    c = torch.as_tensor(np.asarray(cols), dtype=torch.int64)
    xt, yt, wt = _t(x, dtype, True), _t(y, dtype, True), _t(w, dtype, True)
    z = conv_torch(problem, xt, yt, wt, r, c)
    z.backward(_t(dz, dtype))
    return xt.grad.numpy(), yt.grad.numpy(), wt.grad.numpy()


def tp_double_backward(problem, x, y, w, dz, gx, gy, gw, dtype=torch.float64):
    """Gradients of ``<gx,dX> + <gy,dY> + <gw,dW>`` w.r.t. (x, y, w, dz)."""
    xt, yt, wt, dzt = (_t(a, dtype, True) for a in (x, y, w, dz))
    z = tp_torch(problem, xt, yt, wt)
    dx, dy, dw = torch.autograd.grad(z, (xt, yt, wt), dzt, create_graph=True)
    scalar = (dx * _t(gx, dtype)).sum() + (dy * _t(gy, dtype)).sum() + (dw * _t(gw, dtype)).sum()
    grads = torch.autograd.grad(scalar, (xt, yt, wt, dzt), allow_unused=True)
    return tuple(None if g is None else g.numpy() for g in grads)


# --------------------------------------------------------------------------
# weight layout

def oeq_from_e3nn_index(problem, chunk: int = 32) -> np.ndarray:
    """Index ``g`` with ``w_oeq[t] = w_e3nn[g[t]]``, by explicit loops."""
    g = []
    base = 0
    for ins in problem.instructions:
        shape = tuple(ins.path_shape)
        if ins.connection_mode == "uvu":
            nu, nv = shape
            for u0 in range(0, nu, chunk):
                for v0 in range(0, nv, chunk):
                    for v in range(v0, min(v0 + chunk, nv)):
                        for u in range(u0, min(u0 + chunk, nu)):
                            g.append(base + u * nv + v)
        elif ins.connection_mode == "uvw":
            nu, nv, nw = shape
            for u0 in range(0, nu, chunk):
                for v0 in range(0, nv, chunk):
                    for w0 in range(0, nw, chunk):
                        for v in range(v0, min(v0 + chunk, nv)):
                            for u in range(u0, min(u0 + chunk, nu)):
                                for w in range(w0, min(w0 + chunk, nw)):
                                    g.append(base + (u * nv + v) * nw + w)
        else:
            raise ValueError(ins.connection_mode)
        base += prod(shape)
    return np.asarray(g, dtype=np.int64)


def e3nn_to_oeq(problem, w):
    return np.ascontiguousarray(np.asarray(w)[..., oeq_from_e3nn_index(problem)])


def oeq_to_e3nn(problem, w):
    g = oeq_from_e3nn_index(problem)
    out = np.empty_like(np.asarray(w))
    out[..., g] = np.asarray(w)
    return out


# --------------------------------------------------------------------------
# graph order

def coord_graph(rows, cols):
    """Receiver-major edge order and the transpose permutation.

    Returns ``(rows_sorted, cols_sorted, order, transpose_perm)`` where
    ``order`` is the permutation applied to the incoming edge list and
    ``transpose_perm[k]`` is the position, in the sorted list, of the k-th edge
    when edges are ordered by (sender, receiver).
    """
    rows = np.asarray(rows)
    cols = np.asarray(cols)
    order = np.lexsort((cols, rows))
    rs, cs = rows[order], cols[order]
    transpose_perm = np.lexsort((rs, cs)).astype(rows.dtype)
    return rs, cs, order, transpose_perm
