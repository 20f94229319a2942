"""Dim-0 sharding of the tensor operators over the ranks of a ``torch.distributed`` job (one
process per GPU).

Every operator on this path is independent along the outermost (batch) dim, so a rank only ever
holds and processes its slab ``[start:stop]`` of dim 0; operands whose dim 0 is 1 (a broadcast
``B[1,C,1,W]``, per-channel gamma/beta) are replicated.  Elementwise / broadcast / Scale / Softmax
(axis != 0) and reductions that keep dim 0 need no communication at all.  A reduction whose axes
include dim 0 reduces the slab to one DOUBLE partial per output (``sb200_reduce_partial``),
combines the ranks' partials with ONE all-reduce (sum, product, max or min - 8 bytes per output),
and finishes on every rank (``sb200_reduce_finalize``: cast, or divide by the global count for
Avg, or sqrt for L2).  The reference has no multi-device code; this layer is new.

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
    collective: every rank writes its double partials into one record, the records are
    all-gathered, and each rank merges them locally in rank order (deterministic) and finishes.
    Buffers are allocated once, so a step can be captured in a CUDA graph and replayed."""

    def __init__(self, operations: Sequence[int], local_shape: Sequence[int], axes: Sequence[int], global_dim0: int,
                 device, group=None):
        from . import functional as F
        self.F = F
        self.ops = list(operations)
        self.axes = list(axes) if len(axes) else list(range(len(local_shape)))
        self.group = group
        self.rank, self.size = world()
        self.count = 1
        self.total = 1
        for n, d in enumerate(local_shape):
            if n in self.axes:
                self.total *= global_dim0 if n == 0 else d
            else:
                self.count *= d
        self.crosses = 0 in self.axes and self.size > 1
        self.record = torch.empty(len(self.ops) * self.count, dtype=torch.float64, device=device)
        self.gathered = torch.empty(self.size * self.record.numel(), dtype=torch.float64, device=device)
        self.results = [torch.empty(self.count, dtype=torch.float32, device=device) for _ in self.ops]

    def __call__(self, x_local: torch.Tensor):
        F = self.F
        if not self.crosses:
            for i, op in enumerate(self.ops):
                F.reduce(x_local, op, self.axes, keep_dims=True, out=self.results[i])
            return self.results
        for i, op in enumerate(self.ops):
            F.reduce_partial(x_local, op, self.axes, out=self.record[i * self.count:(i + 1) * self.count])
        dist.all_gather_into_tensor(self.gathered, self.record, group=self.group)
        stride = self.record.numel()
        for i, op in enumerate(self.ops):
            F.reduce_combine(self.gathered[i * self.count:], self.size, stride, self.count, op, self.total,
                             out=self.results[i])
        return self.results
