"""Dim-0 sharding of the tensor operators over the ranks of a ``torch.distributed`` job (one
process per GPU).

Every operator on this path is independent along the outermost (batch) dim, so a rank only ever
holds and processes its slab ``[start:stop]`` of dim 0; operands whose dim 0 is 1 (a broadcast
``B[1,C,1,W]``, per-channel gamma/beta) are replicated.  Elementwise / broadcast / Scale / Softmax
(axis != 0) and reductions that keep dim 0 need no communication at all.  A reduction whose axes
include dim 0 reduces the slab to one DOUBLE partial per output (``sb200_reduce_partial``),
combines the ranks' partials with ONE collective - an all-reduce (``reduce``) or, where several
reductions share it and the bits must not depend on the collective's order, an all-gather of the
ranks' records folded in rank order (``ReduceMany``; through the C entry points of
``libsb200_nccl.so`` when given a ``comm.Communicator``) - and finishes on every rank (cast, or divide
by the global count for Avg, or sqrt for L2).  The reference has no multi-device code; this layer is new.

The partial/finalize steps are injectable so the host logic (slab bounds, collective choice,
global counts) can be exercised with CPU tensors over the ``gloo`` backend.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

RED_PROD, RED_SUM, RED_MAX, RED_MIN, RED_AVG, RED_L1, RED_L2 = range(7)


def world() -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def shard_bounds(extent: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous slab of a dim of size ``extent`` for ``rank``: sizes differ by at most one, the
    first ``extent % world_size`` ranks get the larger slabs; a rank may get an empty slab."""
    if not 0 <= rank < world_size:
        raise ValueError("rank %d outside world of %d" % (rank, world_size))
    base, extra = divmod(extent, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def collective_op(operation: int):
    """Which all-reduce combines the partials of a reduction."""
    if operation == RED_PROD:
        return dist.ReduceOp.PRODUCT
    if operation == RED_MAX:
        return dist.ReduceOp.MAX
    if operation == RED_MIN:
        return dist.ReduceOp.MIN
    if operation in (RED_SUM, RED_AVG, RED_L1, RED_L2):
        return dist.ReduceOp.SUM
    raise ValueError("unknown reduce operation %d" % operation)


FLT_MAX = 3.4028234663852886e38


def identity(operation: int) -> float:
    """Neutral partial of an empty slab (the reference's accumulator start values)."""
    return {RED_PROD: 1.0, RED_MAX: -FLT_MAX, RED_MIN: FLT_MAX}.get(operation, 0.0)


def _cuda_partial(x, operation, axes):
    from . import functional as F
    return F.reduce_partial(x, operation, axes)


def _cuda_finalize(part, operation, total):
    from . import functional as F
    return F.reduce_finalize(part, operation, total)


def _cuda_reduce(x, operation, axes):
    from . import functional as F
    return F.reduce(x, operation, axes, keep_dims=True)


def reduce(x_local: torch.Tensor, operation: int, axes: Sequence[int], global_dim0: Optional[int] = None,
           keep_dims: bool = True, group=None, partial_fn: Callable = _cuda_partial,
           finalize_fn: Callable = _cuda_finalize, local_fn: Callable = _cuda_reduce) -> torch.Tensor:
    """Reduce a tensor that is sharded on dim 0.  ``x_local`` is this rank's slab; ``global_dim0``
    the unsharded extent of dim 0 (default: sum over ranks of the local extents, computed here with
    one small all-reduce only if it is not given)."""
    rank, size = world()
    axes = list(axes) if len(axes) else list(range(x_local.dim()))
    crosses = 0 in axes and size > 1
    if not crosses:
        # no cross-rank step: the plain single-device reduction (also the 1-GPU path)
        y = local_fn(x_local, operation, axes)
    else:
        if global_dim0 is None:
            n = torch.tensor([x_local.shape[0]], dtype=torch.int64, device=x_local.device)
            dist.all_reduce(n, op=dist.ReduceOp.SUM, group=group)
            global_dim0 = int(n.item())
        if x_local.shape[0] == 0:   # more ranks than batch entries: contribute the neutral element
            shape = [1 if n in axes else d for n, d in enumerate(x_local.shape)]
            part = torch.full(shape, identity(operation), dtype=torch.float64, device=x_local.device)
        else:
            part = partial_fn(x_local, operation, axes)
        dist.all_reduce(part, op=collective_op(operation), group=group)
        total = global_dim0
        for ax in axes:
            if ax != 0:
                total *= x_local.shape[ax]
        y = finalize_fn(part, operation, total)
    if not keep_dims:
        y = y.reshape([d for n, d in enumerate(y.shape) if n not in axes])
    return y


class ReduceMany:
    """Several reductions (different operations, same axes) of one dim-0-sharded tensor with ONE
    exchange per call: every rank writes its double partials into one record, the records are
    all-gathered, and each rank folds them locally in rank order (deterministic) and finishes.

    Buffers are allocated once, so calls can be captured in a CUDA graph and replayed.  There are
    ``slots`` independent sets of (record, gathered, results): with ``side_stream`` given to a call,
    the exchange and the fold of that call go to the side stream (which first waits for the
    partials), so the caller's stream is free to start the next step's kernels at once; the results
    of slot k are valid after ``join()``.  A graph that holds ``slots`` consecutive steps, each in
    its own slot, followed by one ``join()``, overlaps every exchange but the last with compute.

    ``comm`` is a ``shadow_b200.comm.Communicator`` (the C entry points over NCCL).  Without one the
    exchange is ``torch.distributed.all_gather_into_tensor`` on ``group``, which together with the
    injectable ``partial_fn`` / ``combine_fn`` lets the host logic run on CPU tensors over gloo.

    A rank whose slab is empty (more ranks than entries of dim 0) contributes the neutral record."""

    def __init__(self, operations: Sequence[int], local_shape: Sequence[int], axes: Sequence[int], global_dim0: int,
                 device, group=None, comm=None, slots: int = 1, partial_fn: Optional[Callable] = None,
                 combine_fn: Optional[Callable] = None, local_fn: Optional[Callable] = None):
        self.ops = list(operations)
        self.axes = list(axes) if len(axes) else list(range(len(local_shape)))
        self.group, self.comm = group, comm
        self.rank, self.size = (comm.rank, comm.n_ranks) if comm is not None else world()
        self.count = 1
        self.total = 1
        for n, d in enumerate(local_shape):
            if n in self.axes:
                self.total *= global_dim0 if n == 0 else d
            else:
                self.count *= d
        self.empty = len(local_shape) > 0 and local_shape[0] == 0
        self.crosses = 0 in self.axes and self.size > 1
        self.slots = max(1, int(slots))
        width = len(self.ops) * self.count
        self.records = torch.empty(self.slots, width, dtype=torch.float64, device=device)
        self.gathers = torch.empty(self.slots, self.size * width, dtype=torch.float64, device=device)
        self.results = [[torch.empty(self.count, dtype=torch.float32, device=device) for _ in self.ops]
                        for _ in range(self.slots)]
        # the record of an empty slab: each reduction's neutral element
        self.neutral = torch.cat([torch.full((self.count,), identity(op), dtype=torch.float64) for op in self.ops]).to(device)
        self.partial_fn = partial_fn or self._cuda_partial
        self.combine_fn = combine_fn or self._cuda_combine
        self.local_fn = local_fn or self._cuda_local
        self._side = None

    # -- the CUDA steps (C ABI through `functional`)
    @staticmethod
    def _cuda_partial(x, operation, axes, out):
        from . import functional as F
        F.reduce_partial(x, operation, axes, out=out)

    @staticmethod
    def _cuda_combine(gathered, n_parts, stride, count, operation, total, out):
        from . import functional as F
        F.reduce_combine(gathered, n_parts, stride, count, operation, total, out=out)

    @staticmethod
    def _cuda_local(x, operation, axes, out):
        from . import functional as F
        F.reduce(x, operation, axes, keep_dims=True, out=out)

    def _exchange(self, slot: int) -> None:
        record, gathered, results = self.records[slot], self.gathers[slot], self.results[slot]
        if self.comm is not None:
            stream = torch.cuda.current_stream().cuda_stream
            self.comm.sharded_reduce_finish(record, gathered, self.ops, self.count, self.total, results, stream)
            return
        dist.all_gather_into_tensor(gathered, record, group=self.group)
        for i, op in enumerate(self.ops):
            self.combine_fn(gathered[i * self.count:], self.size, record.numel(), self.count, op, self.total, results[i])

    def __call__(self, x_local: torch.Tensor, slot: int = 0, side_stream=None):
        if not 0 <= slot < self.slots:
            raise ValueError("slot %d outside 0..%d" % (slot, self.slots - 1))
        results = self.results[slot]
        if not self.crosses:
            for i, op in enumerate(self.ops):
                self.local_fn(x_local, op, self.axes, results[i])
            return results
        record = self.records[slot]
        if self.empty:
            record.copy_(self.neutral)
        else:
            for i, op in enumerate(self.ops):
                self.partial_fn(x_local, op, self.axes, record[i * self.count:(i + 1) * self.count])
        if side_stream is None:
            self._exchange(slot)
        else:
            side_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side_stream):
                self._exchange(slot)
            self._side = side_stream
        return results

    def join(self) -> None:
        """Make the current stream wait for every exchange issued on a side stream so far."""
        if self._side is not None:
            torch.cuda.current_stream().wait_stream(self._side)
