"""``TensorProductConv``: fused gather - tensor product - scatter graph convolution.

``Z[n] = sum over edges e with rows[e] == n of TP(X[cols[e]], Y[e], W[e])``.

Mirrors the reference's ``oeq.TensorProductConv`` / ``LoopUnrollConv``
(reference: openequivariance/implementations/convolution/TensorProductConv.py:3-10,
LoopUnrollConv.py:7-87, ConvolutionBase.py:45-109, 560-709):

* ``conv = TensorProductConv(problem, torch_op=True, deterministic=False)``;
  ``Z = conv.forward(X, Y, W, rows, cols)`` for edges in any order (atomic
  accumulation), or, with ``deterministic=True``,
  ``conv.forward(X, Y, W, rows, cols, sender_perm)`` for edges sorted by
  receiver, where ``sender_perm[k]`` is the position in that sorted list of the
  k-th edge in (sender, receiver) order.  The deterministic variant is
  bit-reproducible run to run.
* "uvu" problems whose second input has multiplicity 1 everywhere, per-edge
  weights, int64 indices.
* first and second derivatives as ``torch.library`` custom ops.

Unlike the reference, the deterministic backward pass reads the sender and the
receiver of the k-th edge through ``sender_perm[k]``, so it is also correct
for edge lists that are not structurally symmetric.
"""

import itertools
import typing

import numpy as np
import torch

from . import _native
from .problem import TPProblem
from .tensor_product import TensorProductBase, _require_cuda, _torch, _torch_dtype

_conv_ids = itertools.count()


class CoordGraph:
    """Canonical edge order of a graph: edges sorted by (row, col), plus the
    permutation that visits them in (col, row) order (reference:
    ConvolutionBase.py:45-70)."""

    def __init__(self, coords, rows, cols, name):
        assert len(rows) == len(cols)
        rows, cols = np.asarray(rows), np.asarray(cols)
        self.nnz = len(rows)
        self.node_count = coords.shape[0]
        self.coords = coords
        self.name = name
        order = np.lexsort((cols, rows))
        self.rows = rows[order]
        self.cols = cols[order]
        self.transpose_perm = np.lexsort((self.rows, self.cols)).astype(self.rows.dtype)


class TensorProductConv(TensorProductBase):
    def __init__(self, config: TPProblem, torch_op: bool = False, deterministic: bool = False,
                 idx_dtype=np.int64):
        super().__init__(config, torch_op=torch_op)
        assert idx_dtype == np.int64, "indices are int64"
        if len(config.instructions) == 0:
            raise ValueError("Tensor product problem has no valid intructions!")
        for mul, _ in self.L2:
            assert mul == 1, "the fused convolution needs multiplicity 1 for every irrep of the second input"
        for inst in config.instructions:
            assert inst.connection_mode == "uvu", "the fused convolution supports 'uvu' only"
        assert not config.shared_weights, "the fused convolution needs per-edge weights"
        self.idx_dtype = idx_dtype
        self.deterministic = deterministic
        self.conv_id = next(_conv_ids)
        self.internal = _native.ConvHandle(config, deterministic)
        # The forward pass needs no scratch (node-aligned segmented reduction).  The deterministic backward
        # pass takes optional scratch (one dX row per edge, capped); it is allocated on first use, per
        # device, and kept (the reference keeps its workspace on the object too: ConvolutionBase.py:93-99).
        self.workspace_size = 0
        self.workspace_ptr = 0
        self._scratch = {}
        self.setup_torch_module()

    @staticmethod
    def name():
        return "LoopUnrollConv"

    # ------------------------------------------------------------------ launches

    def _check(self, x, y, w, rows, cols, perm):
        _require_cuda(x, y, w, rows, cols)
        edges = rows.shape[0]
        if x.dim() != 2 or x.shape[1] != self.L1.dim:
            raise ValueError(f"node features must be [nodes, {self.L1.dim}], got {tuple(x.shape)}")
        if tuple(y.shape) != (edges, self.L2.dim):
            raise ValueError(f"edge features must be [{edges}, {self.L2.dim}], got {tuple(y.shape)}")
        if tuple(w.shape) != (edges, self.config.weight_numel):
            raise ValueError(f"weights must be [{edges}, {self.config.weight_numel}], got {tuple(w.shape)}")
        if cols.shape != rows.shape or rows.dim() != 1:
            raise ValueError("rows and cols must be 1-D and of equal length")
        if rows.dtype != torch.int64 or cols.dtype != torch.int64:
            raise ValueError("rows and cols must be int64")
        dt = _torch_dtype(self.irrep_dtype)
        if x.dtype != dt or y.dtype != dt or w.dtype != dt:
            raise ValueError(f"tensors must be {dt}")
        if perm is not None:
            _require_cuda(perm)
            if perm.shape != rows.shape or perm.dtype != torch.int64:
                raise ValueError("sender_perm must be int64 and as long as rows")

    def _forward_impl(self, x, y, w, rows, cols, perm=None, n_out=None):
        """``n_out``: number of output rows when receivers index a different node set than
        senders (a receiver shard of a partitioned graph); defaults to ``x.shape[0]``."""
        self._check(x, y, w, rows, cols, perm)
        x, y, w = x.contiguous(), y.contiguous(), w.contiguous()
        rows, cols = rows.contiguous(), cols.contiguous()
        n_out = x.shape[0] if n_out is None else int(n_out)
        z = torch.empty((n_out, self.L3.dim), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            self.internal.forward(n_out, rows.shape[0], x.data_ptr(), y.data_ptr(), w.data_ptr(),
                                  rows.data_ptr(), cols.data_ptr(), z.data_ptr(), 0, 0,
                                  torch.cuda.current_stream().cuda_stream)
        return z

    def _backward_scratch(self, device, nodes, edges):
        """(pointer, bytes) of the backward scratch for this call, growing the cached buffer if needed.
        When the device cannot spare the preferred size a quarter of it is tried, then none (the library
        then runs its scratch-free kernel)."""
        want = self.internal.workspace_bytes(nodes, edges) if self.deterministic else 0
        if want == 0:
            return 0, 0
        buf = self._scratch.get(device)
        if buf is None or buf.numel() < want:
            self._scratch.pop(device, None)
            buf = None
            for size in (want, want // 4):
                try:
                    buf = torch.empty(size, dtype=torch.uint8, device=device)
                    break
                except torch.OutOfMemoryError:
                    continue
            if buf is None:
                return 0, 0
            self._scratch[device] = buf
        self.workspace_size, self.workspace_ptr = buf.numel(), buf.data_ptr()
        return buf.data_ptr(), buf.numel()

    def _backward_impl(self, x, y, w, dz, rows, cols, perm=None):
        self._check(x, y, w, rows, cols, perm)
        if self.deterministic and perm is None:
            raise ValueError("the deterministic convolution needs sender_perm")
        x, y, w, dz = x.contiguous(), y.contiguous(), w.contiguous(), dz.contiguous()
        rows, cols = rows.contiguous(), cols.contiguous()
        perm_ptr = perm.contiguous().data_ptr() if (perm is not None and self.deterministic) else 0
        dx, dy, dw = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w)
        with torch.cuda.device(x.device):
            ws_ptr, ws_bytes = self._backward_scratch(x.device, x.shape[0], rows.shape[0])
            self.internal.backward(x.shape[0], rows.shape[0], x.data_ptr(), y.data_ptr(), w.data_ptr(),
                                   dz.data_ptr(), rows.data_ptr(), cols.data_ptr(), perm_ptr,
                                   dx.data_ptr(), dy.data_ptr(), dw.data_ptr(), ws_ptr, ws_bytes,
                                   torch.cuda.current_stream().cuda_stream)
        return dx, dy, dw

    def exec_conv_rawptrs(self, L1_in, L2_in, weights, L3_out, rows, cols, nnz, node_count, workspace=0,
                          stream=0):
        """Launch on raw device pointers; argument order of the reference's
        ``JITConvImpl.exec_conv_rawptrs`` (extension/convolution.hpp:27-50)."""
        self.internal.forward(int(node_count), int(nnz), int(L1_in), int(L2_in), int(weights), int(rows),
                              int(cols), int(L3_out), workspace, 0, stream)

    def backward_rawptrs(self, L1_in, L1_grad, L2_in, L2_grad, weights, weights_grad, L3_grad, rows, cols, nnz,
                         node_count, workspace=0, transpose_perm=0, stream=0):
        self.internal.backward(int(node_count), int(nnz), int(L1_in), int(L2_in), int(weights), int(L3_grad),
                               int(rows), int(cols), int(transpose_perm), int(L1_grad), int(L2_grad),
                               int(weights_grad), workspace, 0, stream)

    # ------------------------------------------------------------------ torch ops

    def setup_torch_module(self):
        conv = self
        T = torch.Tensor

        if not self.deterministic:
            @torch.library.custom_op(f"openequivariance_b200::conv_forward{self.conv_id}", mutates_args=(),
                                     device_types="cuda")
            def forward(L1_in: T, L2_in: T, weights: T, rows: T, cols: T) -> T:
                return conv._forward_impl(L1_in, L2_in, weights, rows, cols)

            @forward.register_fake
            def _(L1_in, L2_in, weights, rows, cols):
                return L1_in.new_empty(L1_in.shape[0], conv.L3.dim)

            @torch.library.custom_op(f"openequivariance_b200::conv_backward{self.conv_id}", mutates_args=(),
                                     device_types="cuda")
            def backward_helper(L1_in: T, L2_in: T, weights: T, L3_grad: T, rows: T,
                                cols: T) -> typing.List[T]:
                return list(conv._backward_impl(L1_in, L2_in, weights, L3_grad, rows, cols))

            @backward_helper.register_fake
            def _(L1_in, L2_in, weights, L3_grad, rows, cols):
                return [L1_in.new_empty(*L1_in.shape), L2_in.new_empty(*L2_in.shape),
                        weights.new_empty(*weights.shape)]
            n_index = 2
        else:
            @torch.library.custom_op(f"openequivariance_b200::conv_forward{self.conv_id}", mutates_args=(),
                                     device_types="cuda")
            def forward(L1_in: T, L2_in: T, weights: T, rows: T, cols: T, transpose_perm: T) -> T:
                return conv._forward_impl(L1_in, L2_in, weights, rows, cols, transpose_perm)

            @forward.register_fake
            def _(L1_in, L2_in, weights, rows, cols, transpose_perm):
                return L1_in.new_empty(L1_in.shape[0], conv.L3.dim)

            @torch.library.custom_op(f"openequivariance_b200::conv_backward{self.conv_id}", mutates_args=(),
                                     device_types="cuda")
            def backward_helper(L1_in: T, L2_in: T, weights: T, L3_grad: T, rows: T, cols: T,
                                transpose_perm: T) -> typing.List[T]:
                return list(conv._backward_impl(L1_in, L2_in, weights, L3_grad, rows, cols, transpose_perm))

            @backward_helper.register_fake
            def _(L1_in, L2_in, weights, L3_grad, rows, cols, transpose_perm):
                return [L1_in.new_empty(*L1_in.shape), L2_in.new_empty(*L2_in.shape),
                        weights.new_empty(*weights.shape)]
            n_index = 3

        nones = (None,) * n_index

        def setup_context(ctx, inputs, output):
            ctx.L1_in, ctx.L2_in, ctx.weights = inputs[:3]
            ctx.index = inputs[3:]

        def backward(ctx, grad_output):
            gx, gy, gw = backward_helper(ctx.L1_in, ctx.L2_in, ctx.weights, grad_output, *ctx.index)
            return (gx, gy, gw) + nones

        forward.register_autograd(backward, setup_context=setup_context)

        def setup_context_double_backward(ctx, inputs, output):
            ctx.L1_in, ctx.L2_in, ctx.weights, ctx.L3_grad = inputs[:4]
            ctx.index = inputs[4:]

        def double_backward(ctx, grad_output):
            # same trilinear identity as the batch product, with the graph held fixed
            x, y, w, dz, idx = ctx.L1_in, ctx.L2_in, ctx.weights, ctx.L3_grad, ctx.index
            ex, ey, ew = grad_output[0], grad_output[1], grad_output[2]
            a = backward_helper(ex, ey, w, dz, *idx)
            b = backward_helper(x, y, ew, dz, *idx)
            c = backward_helper(ex, y, w, dz, *idx)
            d = backward_helper(x, ey, w, dz, *idx)
            gz = forward(ex, y, w, *idx) + forward(x, ey, w, *idx) + forward(x, y, ew, *idx)
            return (a[0] + b[0], a[1] + b[1], c[2] + d[2], gz) + nones

        backward_helper.register_autograd(double_backward, setup_context=setup_context_double_backward)
        self.forward = forward
        self.backward_helper = backward_helper

    # ------------------------------------------------------------------ host-array entry points

    def forward_cpu(self, L1_in, L2_in, weights, L3_out, graph):
        """Host arrays and a ``CoordGraph`` in, ``L3_out`` filled in place
        (reference: LoopUnrollConv / ConvolutionBase.forward_cpu, ConvolutionBase.py:104-134)."""
        assert graph.rows.dtype == self.idx_dtype
        dev = [torch.from_numpy(np.ascontiguousarray(a)).cuda()
               for a in (L1_in, L2_in, weights, graph.rows, graph.cols)]
        perm = torch.from_numpy(np.ascontiguousarray(graph.transpose_perm)).cuda() if self.deterministic else None
        L3_out[:] = self._forward_impl(*dev, perm).cpu().numpy()

    def backward_cpu(self, L1_in, L1_grad, L2_in, L2_grad, L3_grad, weights, weights_grad, graph):
        assert graph.rows.dtype == self.idx_dtype
        x, y, w, dz, rows, cols = [torch.from_numpy(np.ascontiguousarray(a)).cuda()
                                   for a in (L1_in, L2_in, weights, L3_grad, graph.rows, graph.cols)]
        perm = torch.from_numpy(np.ascontiguousarray(graph.transpose_perm)).cuda() if self.deterministic else None
        dx, dy, dw = self._backward_impl(x, y, w, dz, rows, cols, perm)
        L1_grad[:] = dx.cpu().numpy()
        L2_grad[:] = dy.cpu().numpy()
        weights_grad[:] = dw.cpu().numpy()

    def check_device_status(self):
        self.internal.check()


LoopUnrollConv = TensorProductConv
