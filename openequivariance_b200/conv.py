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
* "uvw" problems with *shared* weights (second input of multiplicity 1), which the reference does not
  offer ("coming soon", reference: README.md:82-85): the dense weight contraction is linear, so the
  per-edge products are summed per receiver first (the fused gather - product - scatter kernel with every
  weight 1) and the weights are applied once per node, on the tensor cores, instead of once per edge
  (``UVWConvPlan``).
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


class UVWConvPlan:
    """How a shared-weight "uvw" convolution is split in two fused stages.

    ``Z[n, w, k] = sum_e pw_p sum_u W_p[u, w] sum_ij C_ijk x[s_e, u, i] y[e, j]`` is linear in the per-edge
    product, so the edge sum moves inside: stage 1 is the channel-wise ("uvu") convolution with every
    weight 1 and one output block ``mul_u x ir_out`` per instruction, ``S_p[n, u, k] = sum_e sum_ij C_ijk
    x[s_e, u, i] y[e, j]`` (the fused gather - product - scatter kernels, no weight array); stage 2 is the
    batch "uvw" product ``Z[n] = sum_p pw_p W_p . S_p[n]`` over *nodes*, written as ``S_p x 1x0e -> out``
    so that the tensor-core kernels take it (the l x 0 -> l Wigner tensor is the identity / sqrt(2l+1);
    its value is divided out of the path weight).  The weights keep their layout: instruction p has the
    same ``(u, 1, w)`` block in both problems.
    """

    def __init__(self, config: TPProblem):
        from .irreps import Irreps
        from .wigner import wigner_3j
        assert config.shared_weights, "the fused 'uvw' convolution needs shared weights"
        for mul, _ in config.irreps_in2:
            assert mul == 1, "the fused convolution needs multiplicity 1 for every irrep of the second input"
        blocks, edge_instr, dense_instr, dense_pw = [], [], [], []
        for p, ins in enumerate(config.instructions):
            assert ins.connection_mode == "uvw" and ins.has_weight
            mul_u = config.irreps_in1[ins.i_in1].mul
            ir_out = config.irreps_out[ins.i_out].ir
            blocks.append((mul_u, ir_out))
            edge_instr.append((ins.i_in1, ins.i_in2, p, "uvu", True))
            dense_instr.append((p, 0, ins.i_out, "uvw", True))
            identity = float(np.asarray(wigner_3j(ir_out.l, 0, ir_out.l))[0, 0, 0])
            dense_pw.append(ins.path_weight / identity)
        kw = dict(irrep_dtype=config.irrep_dtype, weight_dtype=config.weight_dtype, internal_weights=False)
        self.edge_sum = TPProblem(config.irreps_in1, config.irreps_in2, Irreps(blocks), edge_instr,
                                  shared_weights=False, **kw)
        self.edge_sum.instructions = [i._replace(path_weight=1.0) for i in self.edge_sum.instructions]
        self.dense = TPProblem(Irreps(blocks), "1x0e", config.irreps_out, dense_instr, shared_weights=True, **kw)
        self.dense.instructions = [i._replace(path_weight=w) for i, w in zip(self.dense.instructions, dense_pw)]
        assert self.dense.weight_numel == config.weight_numel


class TensorProductConv(TensorProductBase):
    def __init__(self, config: TPProblem, torch_op: bool = False, deterministic: bool = False,
                 idx_dtype=np.int64):
        super().__init__(config, torch_op=torch_op)
        assert idx_dtype == np.int64, "indices are int64"
        if len(config.instructions) == 0:
            raise ValueError("Tensor product problem has no valid intructions!")
        for mul, _ in self.L2:
            assert mul == 1, "the fused convolution needs multiplicity 1 for every irrep of the second input"
        self.idx_dtype = idx_dtype
        self.deterministic = deterministic
        self.conv_id = next(_conv_ids)
        self._scratch = {}
        self.workspace_size = 0
        self.workspace_ptr = 0
        self.unit_weights = False
        if all(inst.connection_mode == "uvw" for inst in config.instructions):
            self._setup_uvw(config)
            return
        for inst in config.instructions:
            assert inst.connection_mode == "uvu", "the fused convolution supports 'uvu', or 'uvw' with shared weights"
        assert not config.shared_weights, "the fused convolution needs per-edge weights"
        self.internal = _native.ConvHandle(config, deterministic)
        # The forward pass needs no scratch (node-aligned segmented reduction).  The deterministic backward
        # pass takes optional scratch (one dX row per edge, capped); it is allocated on first use, per
        # device, and kept (the reference keeps its workspace on the object too: ConvolutionBase.py:93-99).
        self.setup_torch_module()

    @staticmethod
    def name():
        return "LoopUnrollConv"

    # ------------------------------------------------------------------ shared-weight 'uvw' convolution

    def _setup_uvw(self, config):
        from .tensor_product import TensorProduct
        self.plan = UVWConvPlan(config)
        self.edge_sum = _UnitWeightConv(self.plan.edge_sum, self.deterministic)
        self.dense = TensorProduct(self.plan.dense, torch_op=True)
        self.internal = self.edge_sum.internal
        self._ones = {}
        edge_sum, dense, conv = self.edge_sum, self.dense, self

        def ones(ref, rows_n):
            key = (ref.device, ref.dtype, rows_n)
            if key not in conv._ones:
                conv._ones = {key: torch.ones((rows_n, 1), dtype=ref.dtype, device=ref.device)}
            return conv._ones[key]

        def forward(L1_in, L2_in, weights, rows, cols, transpose_perm=None):
            index = (rows, cols) if transpose_perm is None or not conv.deterministic else (rows, cols, transpose_perm)
            s = edge_sum.forward(L1_in, L2_in, *index)
            return dense.forward(s, ones(s, s.shape[0]), weights)

        def backward_helper(L1_in, L2_in, weights, L3_grad, rows, cols, transpose_perm=None):
            index = (rows, cols) if transpose_perm is None or not conv.deterministic else (rows, cols, transpose_perm)
            s = edge_sum.forward(L1_in, L2_in, *index)
            ds, _, dw = dense.backward_helper(s, ones(s, s.shape[0]), weights, L3_grad)
            dx, dy = edge_sum.backward_helper(L1_in, L2_in, ds, *index)
            return [dx, dy, dw]

        self.forward = forward
        self.backward_helper = backward_helper

    def check_device_status(self):
        self.internal.check()
        if hasattr(self, "dense"):
            self.dense.check_device_status()

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

    def _backward_impl(self, x, y, w, dz, rows, cols, perm=None, scratch=True):
        """``scratch=False`` runs the deterministic pass without scratch memory (the sender-order kernel)."""
        self._check(x, y, w, rows, cols, perm)
        if self.deterministic and perm is None:
            raise ValueError("the deterministic convolution needs sender_perm")
        x, y, w, dz = x.contiguous(), y.contiguous(), w.contiguous(), dz.contiguous()
        rows, cols = rows.contiguous(), cols.contiguous()
        perm_ptr = perm.contiguous().data_ptr() if (perm is not None and self.deterministic) else 0
        dx, dy, dw = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w)
        with torch.cuda.device(x.device):
            ws_ptr, ws_bytes = self._backward_scratch(x.device, x.shape[0], rows.shape[0]) if scratch else (0, 0)
            self.internal.backward(x.shape[0], rows.shape[0], x.data_ptr(), y.data_ptr(), w.data_ptr(),
                                   dz.data_ptr(), rows.data_ptr(), cols.data_ptr(), perm_ptr,
                                   dx.data_ptr(), dy.data_ptr(), dw.data_ptr(), ws_ptr, ws_bytes,
                                   torch.cuda.current_stream().cuda_stream)
        return dx, dy, dw

    def _has_fused_double_backward(self):
        return self.internal.has_double_backward()

    def _double_backward_impl(self, x, y, w, dz, ex, ey, ew, rows, cols, perm=None):
        """Gradients of ``<ex, dX> + <ey, dY> + <ew, dW>`` with respect to (x, y, w, dz) in two fused launches, or
        ``None`` when the library cannot run them here (no scratch memory for the deterministic variant)."""
        self._check(x, y, w, rows, cols, perm)
        if self.deterministic and perm is None:
            raise ValueError("the deterministic convolution needs sender_perm")
        x, y, w, dz, ex, ey, ew = (t.contiguous() for t in (x, y, w, dz, ex, ey, ew))
        rows, cols = rows.contiguous(), cols.contiguous()
        perm_ptr = perm.contiguous().data_ptr() if (perm is not None and self.deterministic) else 0
        gx, gy, gw, gdz = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w), torch.empty_like(dz)
        with torch.cuda.device(x.device):
            ws_ptr, ws_bytes = self._backward_scratch(x.device, x.shape[0], rows.shape[0])
            try:
                self.internal.double_backward(x.shape[0], rows.shape[0], x.data_ptr(), y.data_ptr(), w.data_ptr(),
                                              dz.data_ptr(), ex.data_ptr(), ey.data_ptr(), ew.data_ptr(),
                                              rows.data_ptr(), cols.data_ptr(), perm_ptr, gx.data_ptr(),
                                              gy.data_ptr(), gw.data_ptr(), gdz.data_ptr(), ws_ptr, ws_bytes,
                                              torch.cuda.current_stream().cuda_stream)
            except _native.OeqError as err:
                if err.code == _native.OEQ_ERR_UNSUPPORTED:
                    return None
                raise
        return gx, gy, gw, gdz

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
            if not torch.is_grad_enabled() and conv._has_fused_double_backward():
                # nothing differentiates through this result: two launches that stage an edge's rows once each
                fused = conv._double_backward_impl(x, y, w, dz, ex, ey, ew, *idx)
                if fused is not None:
                    return tuple(fused) + nones
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


class _UnitWeightConv:
    """The fused gather - product - scatter kernels with every weight 1 and no weight array (first stage of the
    shared-weight "uvw" convolution): ``S = forward(X, Y, rows, cols[, sender_perm])``, first and second
    derivatives with respect to X and Y as custom ops."""

    def __init__(self, problem: TPProblem, deterministic: bool):
        self.config, self.deterministic = problem, deterministic
        self.L1, self.L2, self.L3 = problem.irreps_in1, problem.irreps_in2, problem.irreps_out
        self.conv_id = next(_conv_ids)
        self.internal = _native.ConvHandle(problem, deterministic, unit_weights=True)
        self._scratch = None
        self._setup_ops()

    def _forward_impl(self, x, y, rows, cols, perm=None):
        _require_cuda(x, y, rows, cols)
        x, y, rows, cols = x.contiguous(), y.contiguous(), rows.contiguous(), cols.contiguous()
        z = torch.empty((x.shape[0], self.L3.dim), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            self.internal.forward(x.shape[0], rows.shape[0], x.data_ptr(), y.data_ptr(), 0, rows.data_ptr(),
                                  cols.data_ptr(), z.data_ptr(), 0, 0, torch.cuda.current_stream().cuda_stream)
        return z

    def _backward_impl(self, x, y, dz, rows, cols, perm=None):
        _require_cuda(x, y, dz, rows, cols)
        if self.deterministic and perm is None:
            raise ValueError("the deterministic convolution needs sender_perm")
        x, y, dz, rows, cols = x.contiguous(), y.contiguous(), dz.contiguous(), rows.contiguous(), cols.contiguous()
        perm_ptr = perm.contiguous().data_ptr() if (perm is not None and self.deterministic) else 0
        dx, dy = torch.empty_like(x), torch.empty_like(y)
        with torch.cuda.device(x.device):
            ws_ptr = ws_bytes = 0
            want = self.internal.workspace_bytes(x.shape[0], rows.shape[0]) if self.deterministic else 0
            if want:
                if self._scratch is None or self._scratch.numel() < want or self._scratch.device != x.device:
                    self._scratch = torch.empty(want, dtype=torch.uint8, device=x.device)
                ws_ptr, ws_bytes = self._scratch.data_ptr(), self._scratch.numel()
            self.internal.backward(x.shape[0], rows.shape[0], x.data_ptr(), y.data_ptr(), 0, dz.data_ptr(),
                                   rows.data_ptr(), cols.data_ptr(), perm_ptr, dx.data_ptr(), dy.data_ptr(), 0,
                                   ws_ptr, ws_bytes, torch.cuda.current_stream().cuda_stream)
        return dx, dy

    def _setup_ops(self):
        conv = self
        T = torch.Tensor
        if self.deterministic:
            @torch.library.custom_op(f"openequivariance_b200::conv_edge_sum{self.conv_id}", mutates_args=(),
                                     device_types="cuda")
            def forward(L1_in: T, L2_in: T, rows: T, cols: T, transpose_perm: T) -> T:
                return conv._forward_impl(L1_in, L2_in, rows, cols, transpose_perm)

            @torch.library.custom_op(f"openequivariance_b200::conv_edge_sum_backward{self.conv_id}", mutates_args=(),
                                     device_types="cuda")
            def backward_helper(L1_in: T, L2_in: T, L3_grad: T, rows: T, cols: T,
                                transpose_perm: T) -> typing.List[T]:
                return list(conv._backward_impl(L1_in, L2_in, L3_grad, rows, cols, transpose_perm))
            n_index = 3
        else:
            @torch.library.custom_op(f"openequivariance_b200::conv_edge_sum{self.conv_id}", mutates_args=(),
                                     device_types="cuda")
            def forward(L1_in: T, L2_in: T, rows: T, cols: T) -> T:
                return conv._forward_impl(L1_in, L2_in, rows, cols)

            @torch.library.custom_op(f"openequivariance_b200::conv_edge_sum_backward{self.conv_id}", mutates_args=(),
                                     device_types="cuda")
            def backward_helper(L1_in: T, L2_in: T, L3_grad: T, rows: T, cols: T) -> typing.List[T]:
                return list(conv._backward_impl(L1_in, L2_in, L3_grad, rows, cols))
            n_index = 2

        @forward.register_fake
        def _(L1_in, L2_in, *index):
            return L1_in.new_empty(L1_in.shape[0], conv.L3.dim)

        @backward_helper.register_fake
        def _(L1_in, L2_in, L3_grad, *index):
            return [L1_in.new_empty(*L1_in.shape), L2_in.new_empty(*L2_in.shape)]

        nones = (None,) * n_index

        def setup_context(ctx, inputs, output):
            ctx.L1_in, ctx.L2_in = inputs[:2]
            ctx.index = inputs[2:]

        def backward(ctx, grad_output):
            gx, gy = backward_helper(ctx.L1_in, ctx.L2_in, grad_output, *ctx.index)
            return (gx, gy) + nones

        forward.register_autograd(backward, setup_context=setup_context)

        def setup_context_double_backward(ctx, inputs, output):
            ctx.L1_in, ctx.L2_in, ctx.L3_grad = inputs[:3]
            ctx.index = inputs[3:]

        def double_backward(ctx, grad_output):
            # S is bilinear in (X, Y): d<ex,dX>+<ey,dY> / dX = dX(ey, dS), / dY = dY(ex, dS), / dS = S(ex, y) + S(x, ey)
            x, y, ds, idx = ctx.L1_in, ctx.L2_in, ctx.L3_grad, ctx.index
            ex, ey = grad_output[0], grad_output[1]
            a = backward_helper(ex, ey, ds, *idx)
            gs = forward(ex, y, *idx) + forward(x, ey, *idx)
            return (a[0], a[1], gs) + nones

        backward_helper.register_autograd(double_backward, setup_context=setup_context_double_backward)
        self.forward = forward
        self.backward_helper = backward_helper


LoopUnrollConv = TensorProductConv
