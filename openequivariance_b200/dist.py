"""Receiver-sharded graph convolution over several GPUs (one process per GPU).

The reference is single-GPU (device 0 is hard-coded, reference:
openequivariance/extension/util/backend_cuda.hpp:204,258); this layer is new.

Partition: rank ``g`` of ``G`` owns the receiver nodes ``[g*C, min((g+1)*C, N))``
with ``C = ceil(N / G)`` and, because edges are sorted by receiver, a contiguous
slice of the edge list.  Edge features, weights and their gradients never leave
their rank.  The only exchange is on node features:

* forward: all-gather of the owners' ``X`` rows into a local ``[G*C, X.dim]``
  buffer, then the local deterministic convolution writes ``Z`` for owned rows;
* backward: the local kernel produces this rank's contribution to ``dX`` of
  *every* sender, and a reduce-scatter (sum) leaves each rank with ``dX`` of the
  nodes it owns.

Collectives go through ``torch.distributed`` (NCCL on GPUs; gloo works for the
host-side logic on CPU tensors when a ``local_conv`` stand-in is supplied).
"""

from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


class ShardPlan:
    """Which nodes and edges a rank owns, and its local index arrays."""

    def __init__(self, rows: np.ndarray, cols: np.ndarray, nodes: int, rank: int, world: int):
        rows = np.asarray(rows, dtype=np.int64)
        cols = np.asarray(cols, dtype=np.int64)
        if rows.size and np.any(np.diff(rows) < 0):
            raise ValueError("edges must be sorted by receiver")
        if not (0 <= rank < world):
            raise ValueError("rank out of range")
        self.nodes, self.rank, self.world = int(nodes), rank, world
        self.chunk = -(-self.nodes // world) if nodes else 0
        self.node_lo = min(rank * self.chunk, self.nodes)
        self.node_hi = min((rank + 1) * self.chunk, self.nodes)
        self.edge_lo = int(np.searchsorted(rows, self.node_lo, side="left"))
        self.edge_hi = int(np.searchsorted(rows, self.node_hi, side="left"))
        self.local_rows = rows[self.edge_lo:self.edge_hi] - self.node_lo     # receivers, local numbering
        self.local_cols = cols[self.edge_lo:self.edge_hi].copy()             # senders, global numbering
        # k-th local edge in (sender, receiver) order
        self.local_perm = np.lexsort((self.local_rows, self.local_cols)).astype(np.int64)

    @property
    def owned(self) -> int:
        return self.node_hi - self.node_lo

    @property
    def padded_nodes(self) -> int:
        return self.chunk * self.world


class _ShardedConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, module, x_owned, y, w):
        x_full = module.gather_senders(x_owned)
        ctx.module = module
        ctx.save_for_backward(x_full, y, w)
        return module.local_forward(x_full, y, w)

    @staticmethod
    def backward(ctx, dz):
        module = ctx.module
        x_full, y, w = ctx.saved_tensors
        dx_all, dy, dw = module.local_backward(x_full, y, w, dz.contiguous())
        return None, module.scatter_sender_grads(dx_all), dy, dw


class ShardedTensorProductConv:
    """Deterministic fused convolution on one receiver shard of a graph.

    ``rows`` / ``cols`` are the *global*, receiver-sorted edge list (every rank
    passes the same arrays); ``forward`` takes this rank's owned rows of ``X``
    and its slice of ``Y`` and ``W`` (``plan.edge_lo:plan.edge_hi``).
    """

    def __init__(self, problem, rows, cols, nodes, group=None, device=None, local_conv=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.plan = ShardPlan(rows, cols, nodes, self.rank, self.world)
        self.problem = problem
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if local_conv is None:
            from .conv import TensorProductConv
            local_conv = TensorProductConv(problem, torch_op=True, deterministic=True)
        self.conv = local_conv
        as_dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.device)
        self.rows = as_dev(self.plan.local_rows)
        self.cols = as_dev(self.plan.local_cols)
        self.perm = as_dev(self.plan.local_perm)
        self._x_full = None

    # ---- exchange steps -------------------------------------------------------------

    def gather_senders(self, x_owned: torch.Tensor) -> torch.Tensor:
        """All-gather of the owned rows of X into ``[world*chunk, X.dim]`` (tail ranks zero-padded)."""
        plan = self.plan
        if x_owned.shape[0] != plan.owned:
            raise ValueError(f"rank {self.rank} owns {plan.owned} nodes, got {x_owned.shape[0]} rows")
        if self.world == 1:
            return x_owned.contiguous()
        buf = self._x_full
        if buf is None or buf.dtype != x_owned.dtype or buf.shape[1] != x_owned.shape[1]:
            buf = self._x_full = torch.zeros((plan.padded_nodes, x_owned.shape[1]), dtype=x_owned.dtype,
                                             device=x_owned.device)
        send = buf[self.rank * plan.chunk:(self.rank + 1) * plan.chunk]
        send[:plan.owned].copy_(x_owned)
        dist.all_gather_into_tensor(buf, send, group=self.group)
        return buf

    def scatter_sender_grads(self, dx_all: torch.Tensor) -> torch.Tensor:
        """Reduce-scatter (sum) of the per-rank dX contributions; returns the owned rows."""
        plan = self.plan
        if self.world == 1:
            return dx_all[:plan.owned]
        out = torch.empty((plan.chunk, dx_all.shape[1]), dtype=dx_all.dtype, device=dx_all.device)
        dist.reduce_scatter_tensor(out, dx_all, op=dist.ReduceOp.SUM, group=self.group)
        return out[:plan.owned]

    # ---- local kernels -----------------------------------------------------------------

    def local_forward(self, x_full, y, w):
        return self.conv._forward_impl(x_full, y, w, self.rows, self.cols, self.perm, n_out=self.plan.owned)

    def local_backward(self, x_full, y, w, dz):
        return self.conv._backward_impl(x_full, y, w, dz, self.rows, self.cols, self.perm)

    # ---- public ------------------------------------------------------------------------

    def forward(self, x_owned, y, w):
        return _ShardedConvFn.apply(self, x_owned, y, w)

    __call__ = forward

    def forward_backward(self, x_owned, y, w, dz):
        """One fused step without autograd bookkeeping: returns (Z, dX_owned, dY, dW)."""
        x_full = self.gather_senders(x_owned)
        z = self.local_forward(x_full, y, w)
        dx_all, dy, dw = self.local_backward(x_full, y, w, dz)
        return z, self.scatter_sender_grads(dx_all), dy, dw
