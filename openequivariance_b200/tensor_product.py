"""``TensorProduct``: the batch Clebsch-Gordan tensor product as a PyTorch op.

Mirrors the public behaviour of the reference's ``oeq.TensorProduct`` /
``LoopUnrollTP`` (reference: openequivariance/implementations/TensorProduct.py:3-9,
LoopUnrollTP.py:12-71, TensorProductBase.py:11-298):

* ``tp = TensorProduct(problem, torch_op=True)``; ``Z = tp(X, Y, W)`` with
  ``X [B, in1.dim]``, ``Y [B, in2.dim]``, ``W [B, weight_numel]`` (or
  ``[weight_numel]`` when ``problem.shared_weights``) on a CUDA device; weights
  are in the kernel ("oeq") order, ``tp.reorder_weights_e3nn_to_oeq`` converts;
* first and second derivatives through ``torch.library`` custom ops with the
  reference's op structure (forward op, gradient-helper op, double backward
  composed from those two);
* ``forward_cpu`` / ``backward_cpu`` take numpy host arrays, copy them to the
  device, run the kernels and copy the result back, applying the e3nn -> oeq
  weight permutation first, exactly as the reference's test entry points do.

Differences that fix reference defects: launches go to torch's current stream
on the tensors' device (the reference uses the NULL stream of device 0);
shared-weight gradients are summed over the batch in a fixed order (the
reference's kernel overwrites / atomically adds into an uninitialised buffer);
output irreps that no instruction writes are zero (uninitialised in the
reference).
"""

import itertools
import typing

import numpy as np
import torch

from . import _native, weights as _weights
from .problem import TPProblem

_op_ids = itertools.count()


def _torch():
    return torch


def _torch_dtype(np_dtype):
    return {np.float32: torch.float32, np.float64: torch.float64}[np_dtype]


def _require_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("openequivariance_b200 runs on CUDA tensors only (there is no CPU fallback)")


class TensorProductBase:
    """State shared by the batch and the convolution front ends."""

    def __init__(self, config: TPProblem, torch_op: bool = False):
        assert isinstance(config, TPProblem)
        assert isinstance(torch_op, bool)
        self.config, self.torch_op = config, torch_op
        self.L1, self.L2, self.L3 = config.irreps_in1, config.irreps_in2, config.irreps_out
        self.irrep_dtype, self.weight_dtype = config.irrep_dtype, config.weight_dtype
        self.reorder_weights_e3nn_to_oeq = (
            lambda input, output, has_batch_dim: _weights.reorder_weights(config, input, output, "forward",
                                                                          has_batch_dim))
        self.reorder_weights_oeq_to_e3nn = (
            lambda input, output, has_batch_dim: _weights.reorder_weights(config, input, output, "backward",
                                                                          has_batch_dim))

    @staticmethod
    def load_cg_tensor(l1, l2, l3):
        from .wigner import wigner_3j
        return wigner_3j(l1, l2, l3)


class TensorProduct(TensorProductBase):
    """``torch_op`` is kept for signature compatibility (the reference's ``TensorProduct`` requires it, its
    ``LoopUnrollTP`` defaults it to True; this class serves under both names): the torch custom ops are
    registered whatever its value, because device memory and streams come from torch in either case."""

    def __init__(self, problem: TPProblem, torch_op: bool = True):
        super().__init__(problem, torch_op=torch_op)
        if len(problem.instructions) == 0:
            raise ValueError("Tensor product problem has no valid intructions!")
        for inst in problem.instructions:
            assert inst.connection_mode == problem.instructions[0].connection_mode
        assert problem.instructions[0].connection_mode in ["uvu", "uvw"]
        assert problem.irrep_dtype == problem.weight_dtype
        self.is_uvw = problem.instructions[0].connection_mode == "uvw"
        self.tp_id = next(_op_ids)
        self.internal = _native.TPHandle(problem)
        self._has_fused_double_backward = self.internal.has_double_backward()
        self._workspace = None
        # both modes need torch to drive device memory and streams
        self.setup_torch_custom_op()

    @staticmethod
    def name():
        return "LoopUnrollTP"

    def __call__(self, L1_in, L2_in, weights):
        return self.forward(L1_in, L2_in, weights)

    # ------------------------------------------------------------------ raw launches

    def _check_shapes(self, x, y, w):
        cfg = self.config
        if x.dim() != 2 or x.shape[1] != self.L1.dim:
            raise ValueError(f"first input must be [batch, {self.L1.dim}], got {tuple(x.shape)}")
        if y.dim() != 2 or y.shape != (x.shape[0], self.L2.dim):
            raise ValueError(f"second input must be [{x.shape[0]}, {self.L2.dim}], got {tuple(y.shape)}")
        want = (cfg.weight_numel,) if cfg.shared_weights else (x.shape[0], cfg.weight_numel)
        if tuple(w.shape) != want:
            raise ValueError(f"weights must be {want}, got {tuple(w.shape)}")
        dt = _torch_dtype(self.irrep_dtype)
        if x.dtype != dt or y.dtype != dt or w.dtype != dt:
            raise ValueError(f"tensors must be {dt}")

    def _forward_impl(self, x, y, w):
        _require_cuda(x, y, w)
        self._check_shapes(x, y, w)
        x, y, w = x.contiguous(), y.contiguous(), w.contiguous()
        z = torch.empty((x.shape[0], self.L3.dim), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            self.internal.forward(x.shape[0], x.data_ptr(), y.data_ptr(), w.data_ptr(), z.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
        return z

    def _backward_impl(self, x, y, w, dz):
        _require_cuda(x, y, w, dz)
        self._check_shapes(x, y, w)
        x, y, w, dz = x.contiguous(), y.contiguous(), w.contiguous(), dz.contiguous()
        dx, dy, dw = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w)
        ws_bytes = self.internal.workspace_bytes(x.shape[0])
        ws_ptr = 0
        if ws_bytes:
            ws = self._workspace
            if ws is None or ws.numel() < ws_bytes or ws.device != x.device:
                ws = self._workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
            ws_ptr = ws.data_ptr()
        with torch.cuda.device(x.device):
            self.internal.backward(x.shape[0], x.data_ptr(), y.data_ptr(), w.data_ptr(), dz.data_ptr(),
                                   dx.data_ptr(), dy.data_ptr(), dw.data_ptr(), ws_ptr, ws_bytes,
                                   torch.cuda.current_stream().cuda_stream)
        return dx, dy, dw

    def _double_backward_impl(self, x, y, w, dz, ex, ey, ew):
        """Gradients of ``<ex, dX> + <ey, dY> + <ew, dW>`` with respect to (x, y, w, dz) in one launch (problems
        for which the library has the one-pass kernel: ``self._has_fused_double_backward``)."""
        _require_cuda(x, y, w, dz, ex, ey, ew)
        self._check_shapes(x, y, w)
        x, y, w, dz, ex, ey, ew = (t.contiguous() for t in (x, y, w, dz, ex, ey, ew))
        gx, gy, gw, gdz = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w), torch.empty_like(dz)
        with torch.cuda.device(x.device):
            self.internal.double_backward(x.shape[0], x.data_ptr(), y.data_ptr(), w.data_ptr(), dz.data_ptr(),
                                          ex.data_ptr(), ey.data_ptr(), ew.data_ptr(), gx.data_ptr(), gy.data_ptr(),
                                          gw.data_ptr(), gdz.data_ptr(), torch.cuda.current_stream().cuda_stream)
        return gx, gy, gw, gdz

    def forward_raw(self, batch, L1_in, L2_in, L3_out, weights, stream=0):
        """Launch on raw device pointers (argument order of the reference's
        ``forward_raw``, TensorProductBase.py:41-49)."""
        self.internal.forward(int(batch), int(L1_in), int(L2_in), int(weights), int(L3_out), stream)

    def backward_raw(self, batch_size, L1_in, L1_grad, L2_in, L2_grad, weights, weights_grad, L3_grad,
                     workspace=0, workspace_bytes=0, stream=0):
        self.internal.backward(int(batch_size), int(L1_in), int(L2_in), int(weights), int(L3_grad),
                               int(L1_grad), int(L2_grad), int(weights_grad), workspace, workspace_bytes, stream)

    # ------------------------------------------------------------------ torch ops

    def setup_torch_custom_op(self):
        tp = self

        @torch.library.custom_op(f"openequivariance_b200::tp_forward{self.tp_id}", mutates_args=(),
                                 device_types="cuda")
        def forward(L1_in: torch.Tensor, L2_in: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
            return tp._forward_impl(L1_in, L2_in, weights)

        @forward.register_fake
        def _(L1_in, L2_in, weights):
            return L1_in.new_empty(L1_in.shape[0], tp.L3.dim)

        @torch.library.custom_op(f"openequivariance_b200::tp_grad_helper{self.tp_id}", mutates_args=(),
                                 device_types="cuda")
        def backward_helper(L1_in: torch.Tensor, L2_in: torch.Tensor, weights: torch.Tensor,
                            L3_grad: torch.Tensor) -> typing.List[torch.Tensor]:
            return list(tp._backward_impl(L1_in, L2_in, weights, L3_grad))

        @backward_helper.register_fake
        def _(L1_in, L2_in, weights, L3_grad):
            return [L1_in.new_empty(*L1_in.shape), L2_in.new_empty(*L2_in.shape),
                    weights.new_empty(*weights.shape)]

        def setup_context(ctx, inputs, output):
            ctx.L1_in, ctx.L2_in, ctx.weights = inputs

        def backward(ctx, grad_output):
            gx, gy, gw = backward_helper(ctx.L1_in, ctx.L2_in, ctx.weights, grad_output)
            return gx, gy, gw

        forward.register_autograd(backward, setup_context=setup_context)

        def setup_context_double_backward(ctx, inputs, output):
            ctx.L1_in, ctx.L2_in, ctx.weights, ctx.L3_grad = inputs

        def double_backward(ctx, grad_output):
            # The product is trilinear in (x, y, w).  With cotangents (ex, ey, ew) of (dX, dY, dW):
            #   d/d(dz) = f(ex, y, w) + f(x, ey, w) + f(x, y, ew)
            #   d/dx    = dX(ey, w, dz) + dX(y, ew, dz)     and likewise for y and w.
            x, y, w, dz = ctx.L1_in, ctx.L2_in, ctx.weights, ctx.L3_grad
            ex, ey, ew = grad_output[0], grad_output[1], grad_output[2]
            if tp._has_fused_double_backward and not torch.is_grad_enabled():
                # nothing differentiates through this result: one launch that reads the row's arrays once
                return tp._double_backward_impl(x, y, w, dz, ex, ey, ew)
            a = backward_helper(ex, ey, w, dz)   # dX(ey, w), dY(ex, w)
            b = backward_helper(x, y, ew, dz)    # dX(y, ew), dY(x, ew)
            c = backward_helper(ex, y, w, dz)    # dW(ex, y)
            d = backward_helper(x, ey, w, dz)    # dW(x, ey)
            gz = forward(ex, y, w) + forward(x, ey, w) + forward(x, y, ew)
            return a[0] + b[0], a[1] + b[1], c[2] + d[2], gz

        backward_helper.register_autograd(double_backward, setup_context=setup_context_double_backward)
        self.forward = forward
        self.backward_helper = backward_helper

    # ------------------------------------------------------------------ host-array entry points

    def _weights_to_device(self, weights):
        w = np.ascontiguousarray(weights)
        reordered = np.zeros_like(w)
        self.reorder_weights_e3nn_to_oeq(w, reordered, not self.config.shared_weights)
        return torch.from_numpy(reordered).cuda()

    def forward_cpu(self, L1_in, L2_in, L3_out, weights) -> None:
        """Host arrays in, ``L3_out`` filled in place; ``weights`` in e3nn order
        (reference: TensorProductBase.py:63-84)."""
        x = torch.from_numpy(np.ascontiguousarray(L1_in)).cuda()
        y = torch.from_numpy(np.ascontiguousarray(L2_in)).cuda()
        w = self._weights_to_device(weights)
        L3_out[:] = self._forward_impl(x, y, w).cpu().numpy()

    def backward_cpu(self, L1_in, L1_grad, L2_in, L2_grad, L3_grad, weights, weights_grad) -> None:
        """Host arrays in, the three gradients filled in place, ``weights_grad``
        returned in e3nn order (reference: TensorProductBase.py:86-112)."""
        x = torch.from_numpy(np.ascontiguousarray(L1_in)).cuda()
        y = torch.from_numpy(np.ascontiguousarray(L2_in)).cuda()
        dz = torch.from_numpy(np.ascontiguousarray(L3_grad)).cuda()
        w = self._weights_to_device(weights)
        dx, dy, dw = self._backward_impl(x, y, w, dz)
        L1_grad[:] = dx.cpu().numpy()
        L2_grad[:] = dy.cpu().numpy()
        dw_oeq = dw.cpu().numpy()
        self.reorder_weights_oeq_to_e3nn(dw_oeq, weights_grad, not self.config.shared_weights)

    def check_device_status(self):
        """Raises if a kernel of this object abandoned a bounded wait."""
        self.internal.check()


LoopUnrollTP = TensorProduct
