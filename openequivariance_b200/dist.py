"""Receiver-sharded graph convolution over several GPUs (one process per GPU).

The reference is single-GPU (device 0 is hard-coded, reference:
openequivariance/extension/util/backend_cuda.hpp:204,258); this layer is new.

Partition: rank ``g`` of ``G`` owns the receiver nodes ``[g*C, min((g+1)*C, N))``
with ``C = ceil(N / G)`` and, because edges are sorted by receiver, a contiguous
slice of the edge list.  Edge features, weights and their gradients never leave
their rank.  The only exchange is on node features, and only on the *halo*: the
sender nodes of a rank's edges that another rank owns.

* forward: every rank sends the rows of ``X`` that its peers' edges read
  (all-to-all with per-peer row lists fixed at set-up); the local deterministic
  kernel then runs on ``[owned rows | halo rows]`` with sender ids renumbered
  into that compact space;
* backward: the local kernel produces ``dX`` for owned and halo rows; halo rows
  travel back to their owners (the mirrored all-to-all) and are added to the
  owners' rows peer by peer in rank order, so the result is reproducible.

The batch tensor product shards by rows with no exchange at all; only a shared weight
tensor's gradient is summed over the ranks (``ShardedTensorProduct``).

With spatially ordered node ids the halo is a thin shell, so the exchanged
volume is a small fraction of an all-gather of ``X``.  Collectives go through
``torch.distributed`` (NCCL on GPUs; gloo works for the host-side logic on CPU
tensors when a ``local_conv`` stand-in is supplied).  Every rank builds the
plan of every rank from the global edge list, so set-up needs no communication.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


def _owned_range(nodes: int, rank: int, world: int):
    chunk = -(-nodes // world) if nodes else 0
    return min(rank * chunk, nodes), min((rank + 1) * chunk, nodes)


class ShardPlan:
    """Which nodes and edges a rank owns, its halo, and its local index arrays."""

    def __init__(self, rows: np.ndarray, cols: np.ndarray, nodes: int, rank: int, world: int):
        rows = np.asarray(rows, dtype=np.int64)
        cols = np.asarray(cols, dtype=np.int64)
        if rows.size and np.any(np.diff(rows) < 0):
            raise ValueError("edges must be sorted by receiver")
        if not (0 <= rank < world):
            raise ValueError("rank out of range")
        self.nodes, self.rank, self.world = int(nodes), rank, world
        self.node_lo, self.node_hi = _owned_range(self.nodes, rank, world)
        self.edge_lo = int(np.searchsorted(rows, self.node_lo, side="left"))
        self.edge_hi = int(np.searchsorted(rows, self.node_hi, side="left"))
        local_cols = cols[self.edge_lo:self.edge_hi]
        senders = np.unique(local_cols)
        outside = (senders < self.node_lo) | (senders >= self.node_hi)
        self.halo = senders[outside]                               # global ids, ascending
        # compact sender numbering: owned nodes first, then the halo in ascending global order
        halo_pos = np.searchsorted(self.halo, local_cols)
        is_owned = (local_cols >= self.node_lo) & (local_cols < self.node_hi)
        self.local_cols = np.where(is_owned, local_cols - self.node_lo, self.owned + halo_pos).astype(np.int64)
        self.local_rows = rows[self.edge_lo:self.edge_hi] - self.node_lo
        # k-th local edge in (sender, receiver) order of the compact numbering
        self.local_perm = np.lexsort((self.local_rows, self.local_cols)).astype(np.int64)
        # halo rows grouped by owner (owners hold contiguous id ranges, so this is a split of self.halo)
        bounds = [_owned_range(self.nodes, q, world)[0] for q in range(world)] + [self.nodes]
        self.recv_counts = [int(np.searchsorted(self.halo, bounds[q + 1]) - np.searchsorted(self.halo, bounds[q]))
                            for q in range(world)]
        self.send_rows = None     # filled by build_exchange

    @property
    def owned(self) -> int:
        return self.node_hi - self.node_lo

    @property
    def local_nodes(self) -> int:
        return self.owned + int(self.halo.size)

    @staticmethod
    def build_all(rows, cols, nodes, world):
        """Plans of all ranks with their send lists (rows each rank ships to each peer)."""
        plans = [ShardPlan(rows, cols, nodes, r, world) for r in range(world)]
        for me in plans:
            me.send_rows = []
            for peer in plans:
                if peer.rank == me.rank:
                    me.send_rows.append(np.zeros(0, dtype=np.int64))
                    continue
                wanted = peer.halo[(peer.halo >= me.node_lo) & (peer.halo < me.node_hi)]
                me.send_rows.append((wanted - me.node_lo).astype(np.int64))
        return plans

    @staticmethod
    def build_one(rows, cols, nodes, rank, world):
        """The plan of one rank with its send lists, without building the peers' plans: the rows this rank
        ships to peer q are the distinct senders it owns among the edges of q's slice (ascending, which is
        the order of q's halo)."""
        rows = np.asarray(rows, dtype=np.int64)
        cols = np.asarray(cols, dtype=np.int64)
        me = ShardPlan(rows, cols, nodes, rank, world)
        mine = np.nonzero((cols >= me.node_lo) & (cols < me.node_hi))[0]         # edges whose sender this rank owns
        edge_lo = [int(np.searchsorted(rows, _owned_range(me.nodes, q, world)[0], side="left")) for q in range(world)]
        owner = np.searchsorted(np.asarray(edge_lo[1:], dtype=np.int64), mine, side="right")   # rank holding each edge
        me.send_rows = []
        for q in range(world):
            if q == rank:
                me.send_rows.append(np.zeros(0, dtype=np.int64))
            else:
                me.send_rows.append((np.unique(cols[mine[owner == q]]) - me.node_lo).astype(np.int64))
        return me


class _ShardedConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, module, x_owned, y, w):
        # a fresh tensor: it is saved for the backward pass, and a second forward before that backward must
        # not overwrite it (the module's re-used buffer serves the calls that keep nothing)
        x_local = module.gather_senders(x_owned, fresh=True)
        ctx.module = module
        ctx.save_for_backward(x_local, y, w)
        return module.local_forward(x_local, y, w)

    @staticmethod
    def backward(ctx, dz):
        module = ctx.module
        x_local, y, w = ctx.saved_tensors
        dx_local, dy, dw = module.local_backward(x_local, y, w, dz.contiguous())
        return None, module.scatter_sender_grads(dx_local), dy, dw


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
        self.plan = ShardPlan.build_one(rows, cols, nodes, self.rank, self.world)
        self.problem = problem
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if local_conv is None:
            from .conv import TensorProductConv
            local_conv = TensorProductConv(problem, torch_op=True, deterministic=True)
        self.conv = local_conv
        as_dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.device)
        plan = self.plan
        self.rows = as_dev(plan.local_rows)
        self.cols = as_dev(plan.local_cols)
        self.perm = as_dev(plan.local_perm)
        self.send_counts = [int(s.size) for s in plan.send_rows]
        self.recv_counts = list(plan.recv_counts)
        self.send_index = as_dev(np.concatenate(plan.send_rows)) if self.world > 1 else None
        self.send_index_per_peer = [as_dev(s) for s in plan.send_rows] if self.world > 1 else []
        self._x_local = None
        self._x_owned = None
        self._streamed = None
        self._streamed_slab_edges = None

    # ---- exchange steps -------------------------------------------------------------

    def gather_senders(self, x_owned: torch.Tensor, fresh: bool = False) -> torch.Tensor:
        """``[owned rows | halo rows]`` of X: one all-to-all of the rows the peers' edges read.  The result
        lives in a buffer that the next call overwrites unless ``fresh`` asks for a new tensor."""
        plan = self.plan
        if x_owned.shape[0] != plan.owned:
            raise ValueError(f"rank {self.rank} owns {plan.owned} nodes, got {x_owned.shape[0]} rows")
        if self.world == 1:
            return x_owned.contiguous()
        buf = None if fresh else self._x_local
        if buf is None or buf.dtype != x_owned.dtype or buf.shape[1] != x_owned.shape[1]:
            buf = torch.empty((plan.local_nodes, x_owned.shape[1]), dtype=x_owned.dtype, device=x_owned.device)
            if not fresh:
                self._x_local = buf
        if x_owned.data_ptr() != buf.data_ptr():        # a caller that filled ``owned_buffer`` has no copy to pay
            buf[:plan.owned].copy_(x_owned)
        send = x_owned.index_select(0, self.send_index)
        dist.all_to_all_single(buf[plan.owned:], send, output_split_sizes=self.recv_counts,
                               input_split_sizes=self.send_counts, group=self.group)
        return buf

    def owned_buffer(self, width: int, dtype=torch.float32) -> torch.Tensor:
        """The first ``owned`` rows of the gather buffer: a caller that keeps its node features there saves
        ``gather_senders`` the copy of the owned rows (the halo rows behind them are overwritten by every call)."""
        buf = self._x_local
        if buf is None or buf.dtype != dtype or buf.shape[1] != width:
            buf = self._x_local = torch.empty((self.plan.local_nodes, width), dtype=dtype, device=self.device)
        return buf[:self.plan.owned]

    def scatter_sender_grads(self, dx_local: torch.Tensor) -> torch.Tensor:
        """Halo rows of dX go back to their owners and are added peer by peer in rank order.  The owned rows of
        ``dx_local`` are updated in place and returned as a view."""
        plan = self.plan
        dx_owned = dx_local[:plan.owned]
        if self.world == 1:
            return dx_owned
        recv = torch.empty((sum(self.send_counts), dx_local.shape[1]), dtype=dx_local.dtype, device=dx_local.device)
        dist.all_to_all_single(recv, dx_local[plan.owned:].contiguous(), output_split_sizes=self.send_counts,
                               input_split_sizes=self.recv_counts, group=self.group)
        out = dx_owned          # dx_local is this step's own result: the peers' rows are added in place
        start = 0
        for peer, count in enumerate(self.send_counts):      # fixed order; indices are unique within a peer
            if count:
                out.index_add_(0, self.send_index_per_peer[peer], recv[start:start + count])
                start += count
        return out

    # ---- local kernels -----------------------------------------------------------------

    def local_forward(self, x_local, y, w):
        return self.conv._forward_impl(x_local, y, w, self.rows, self.cols, self.perm, n_out=self.plan.owned)

    def local_backward(self, x_local, y, w, dz):
        return self.conv._backward_impl(x_local, y, w, dz, self.rows, self.cols, self.perm)

    # ---- public ------------------------------------------------------------------------

    def forward(self, x_owned, y, w):
        return _ShardedConvFn.apply(self, x_owned, y, w)

    __call__ = forward

    def forward_backward(self, x_owned, y, w, dz):
        """One fused step without autograd bookkeeping: returns (Z, dX_owned, dY, dW)."""
        x_local = self.gather_senders(x_owned)
        z = self.local_forward(x_local, y, w)
        dx_local, dy, dw = self.local_backward(x_local, y, w, dz)
        return z, self.scatter_sender_grads(dx_local), dy, dw


    def slab_plan(self, slab_edges: int = 1 << 18):
        """The slab pipeline over this rank's edges (``StreamedTensorProductConv``; ``.slabs``, ``.max_edges``
        and ``.max_receivers`` size the caller's pinned tiles), built once per slab size."""
        if self._streamed is None or self._streamed_slab_edges != slab_edges:
            from .stream import StreamedTensorProductConv
            plan = self.plan
            self._streamed = StreamedTensorProductConv(self.problem, plan.local_rows, plan.local_cols, plan.owned,
                                                       slab_edges=slab_edges, device=self.device, local_conv=self.conv)
            self._streamed_slab_edges = slab_edges
        return self._streamed

    def forward_backward_host(self, x_h, y_h, w_h, dz_h, z_h, dx_h, dy_h, dw_h, slab_edges: int = 1 << 18):
        """The same step on host tensors of this rank's shard (owned rows of ``X`` and ``dZ``, the rank's
        edge slice of ``Y`` and ``W``; outputs into ``z_h``, ``dx_h``, ``dy_h``, ``dw_h``).

        The owned rows of ``X`` go to the device and the halo is exchanged once; the per-edge arrays then
        stream through the GPU in edge slabs whose copies overlap the kernels
        (``StreamedTensorProductConv.stream_slabs``); ``dX`` stays on the device until its halo rows have
        gone back to their owners.  Edge arrays may be callables ``f(slab_index, e0, e1)`` as in the
        single-GPU entry point (edge positions relative to the rank's slice).  Results are complete once
        the current stream is."""
        plan = self.plan
        streamed = self.slab_plan(slab_edges)
        if x_h.shape[0] != plan.owned:
            raise ValueError(f"rank {self.rank} owns {plan.owned} nodes, got {x_h.shape[0]} rows")
        if self.device.type == "cuda":
            buf = self._x_owned
            if buf is None or buf.dtype != x_h.dtype:
                buf = self._x_owned = torch.empty((plan.owned, x_h.shape[1]), dtype=x_h.dtype, device=self.device)
            buf.copy_(x_h, non_blocking=True)
            x_owned = buf
        else:
            x_owned = x_h
        x_local = self.gather_senders(x_owned)
        dx_local = streamed.stream_slabs(x_local, y_h, w_h, dz_h, z_h, dy_h, dw_h)
        dx_h.copy_(self.scatter_sender_grads(dx_local), non_blocking=True)

    def host_bytes(self, elem: int):
        """(host-to-device, device-to-host) bytes of one ``forward_backward_host`` step on this rank."""
        p, plan = self.problem, self.plan
        edges = plan.edge_hi - plan.edge_lo
        node = plan.owned * (p.irreps_in1.dim + p.irreps_out.dim) * elem
        edge = edges * (p.irreps_in2.dim + p.weight_numel) * elem
        return node + edge + edges * 24, node + edge


# ---------------------------------------------------------------------------------------------------
# batch tensor product: rows are independent


def row_range(batch: int, rank: int, world: int):
    """Rows ``[lo, hi)`` of a batch of ``batch`` rows that rank ``rank`` of ``world`` owns."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    chunk = -(-batch // world) if batch else 0
    return min(rank * chunk, batch), min((rank + 1) * chunk, batch)


class _ShardedTPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, module, x, y, w):
        ctx.module = module
        ctx.save_for_backward(x, y, w)
        return module.tp._forward_impl(x, y, w)

    @staticmethod
    def backward(ctx, dz):
        x, y, w = ctx.saved_tensors
        dx, dy, dw = ctx.module.local_backward(x, y, w, dz.contiguous())
        return None, dx, dy, dw


class ShardedTensorProduct:
    """Batch tensor product on this rank's rows of a batch that is split by rows over the ranks.

    Forward and the input gradients need no communication.  With ``shared_weights`` every rank holds the
    whole weight tensor and the weight gradient is the sum over all rows, so the local gradients are added
    with one all-reduce (``weight_numel`` values).  ``local_tp`` may replace the CUDA tensor product by an
    object with the same ``_forward_impl`` / ``_backward_impl`` (tests of the host logic).
    """

    def __init__(self, problem, group=None, local_tp=None):
        self.problem = problem
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if local_tp is None:
            from .tensor_product import TensorProduct
            local_tp = TensorProduct(problem, torch_op=True)
        self.tp = local_tp

    def local_backward(self, x, y, w, dz):
        dx, dy, dw = self.tp._backward_impl(x, y, w, dz)
        if self.problem.shared_weights and self.world > 1:
            dist.all_reduce(dw, op=dist.ReduceOp.SUM, group=self.group)
        return dx, dy, dw

    def forward(self, x, y, w):
        return _ShardedTPFn.apply(self, x, y, w)

    __call__ = forward

