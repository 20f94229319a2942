"""Host logic of the multi-GPU path on CPU: world_size-2 (and 3) gloo ranks shard a tensor on
dim 0, compute per-rank partials with the C oracle, combine them with the all-reduce that
shadow_b200.sharded chooses, and must reproduce the single-process oracle result."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

import cases
from oracle import oracle as orc
from shadow_b200 import sharded

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds_cover_exactly():
    for extent in (0, 1, 7, 8, 9, 64):
        for world in (1, 2, 3, 4, 8):
            spans = [sharded.shard_bounds(extent, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == extent
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharded.shard_bounds(8, 2, 2)


def _cpu_partial(x, operation, axes):
    """What sb200_reduce_partial produces, computed on CPU: one double per kept position."""
    a = x.numpy().astype(np.float64)
    ax = tuple(axes)
    if operation == 0:
        p = np.prod(a, axis=ax, keepdims=True)
    elif operation in (1, 4):
        p = np.sum(a, axis=ax, keepdims=True)
    elif operation == 2:
        p = np.max(a, axis=ax, keepdims=True)
    elif operation == 3:
        p = np.min(a, axis=ax, keepdims=True)
    elif operation == 5:
        p = np.sum(np.abs(a), axis=ax, keepdims=True)
    else:
        sq = (np.abs(x.numpy()) * np.abs(x.numpy())).astype(np.float64)   # float square, as the reference
        p = np.sum(sq, axis=ax, keepdims=True)
    return torch.from_numpy(np.ascontiguousarray(p))


def _cpu_finalize(part, operation, total):
    p = part.numpy()
    if operation == 4:
        y = (p / float(total)).astype(np.float32)
    elif operation == 6:
        y = np.sqrt(p.astype(np.float32))
    else:
        y = p.astype(np.float32)
    return torch.from_numpy(y)


def _cpu_local(x, operation, axes):
    return torch.from_numpy(orc.reduce(x.numpy(), operation, axes, keep_dims=True))


def _worker(rank, world, port, shape, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = cases.normal(4242, shape)
        full_pos = cases.uniform(4243, shape, 0.9, 1.1)
        lo, hi = sharded.shard_bounds(shape[0], rank, world)
        failures = []
        for op in range(7):
            src = full_pos if op == 0 else full
            local = torch.from_numpy(np.ascontiguousarray(src[lo:hi]))
            for axes, keep in (([], False), ([0, 2], True), ([1], True), ([0], False)):
                got = sharded.reduce(local, op, axes, global_dim0=shape[0], keep_dims=keep,
                                     partial_fn=_cpu_partial, finalize_fn=_cpu_finalize, local_fn=_cpu_local).numpy()
                want = orc.reduce(src, op, axes, keep_dims=keep)
                if 0 not in (axes or list(range(len(shape)))):
                    want = want[lo:hi]       # dim 0 is kept: each rank owns its slab of the result
                n = max(2, int(np.prod([shape[a] for a in (axes or range(len(shape)))])))
                if got.shape != want.shape or not np.allclose(got, want, rtol=1e-5 * np.log2(n), atol=0):
                    failures.append((op, axes, keep, got.shape, want.shape))
        # unknown global extent: discovered with one extra all-reduce
        local = torch.from_numpy(np.ascontiguousarray(full[lo:hi]))
        got = sharded.reduce(local, 4, [], keep_dims=False, partial_fn=_cpu_partial, finalize_fn=_cpu_finalize,
                             local_fn=_cpu_local).numpy()
        if not np.allclose(got, orc.reduce(full, 4, [], keep_dims=False), rtol=1e-4):
            failures.append(("avg-unknown-extent",))
        with open(os.path.join(out_dir, "rank%d.txt" % rank), "w") as f:
            f.write(repr(failures))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,shape", [(2, (6, 5, 7)), (3, (2, 4, 3)), (2, (1, 3, 4))])
def test_sharded_reduce_over_gloo(tmp_path, world, shape):
    """world 3 over a batch of 2 and world 2 over a batch of 1 leave a rank with an empty slab."""
    port = 29500 + (os.getpid() % 2000) + world
    mp.spawn(_worker, args=(world, port, shape, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(os.path.join(str(tmp_path), "rank%d.txt" % r)).read() == "[]"


def test_collective_choice():
    import torch.distributed as dist
    assert sharded.collective_op(0) == dist.ReduceOp.PRODUCT
    assert sharded.collective_op(2) == dist.ReduceOp.MAX
    assert sharded.collective_op(3) == dist.ReduceOp.MIN
    for op in (1, 4, 5, 6):
        assert sharded.collective_op(op) == dist.ReduceOp.SUM
    with pytest.raises(ValueError):
        sharded.collective_op(7)
    assert sharded.identity(0) == 1.0 and sharded.identity(2) < -3e38 and sharded.identity(1) == 0.0


def _cpu_partial_into(x, operation, axes, out):
    out.copy_(_cpu_partial(x, operation, axes).reshape(-1))


def _cpu_combine_into(gathered, n_parts, stride, count, operation, total, out):
    """What sb200_reduce_combine does: part p of output o at gathered[p*stride + o], folded in order."""
    g = gathered.numpy()
    acc = g[0:count].copy()
    for p in range(1, n_parts):
        nxt = g[p * stride:p * stride + count]
        if operation == 0:
            acc = acc * nxt
        elif operation == 2:
            acc = np.maximum(acc, nxt)
        elif operation == 3:
            acc = np.minimum(acc, nxt)
        else:
            acc = acc + nxt
    out.copy_(_cpu_finalize(torch.from_numpy(acc), operation, total))


def _cpu_local_into(x, operation, axes, out):
    out.copy_(_cpu_local(x, operation, axes).reshape(-1))


def _many_worker(rank, world, port, shape, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = cases.normal(5151, shape)
        lo, hi = sharded.shard_bounds(shape[0], rank, world)
        local = torch.from_numpy(np.ascontiguousarray(full[lo:hi]))
        failures = []
        ops = [1, 2, 3, 4, 6]
        for axes in ([], [0, 2], [1]):
            many = sharded.ReduceMany(ops, local.shape, axes, shape[0], "cpu", slots=2, partial_fn=_cpu_partial_into,
                                      combine_fn=_cpu_combine_into, local_fn=_cpu_local_into)
            for slot in (0, 1):
                scaled = local * float(slot + 1)       # different data per slot: slots must not alias
                res = many(scaled, slot=slot)
                many.join()                            # no side stream was used: a no-op
                for op, r in zip(ops, res):
                    want = orc.reduce(full * np.float32(slot + 1), op, axes, keep_dims=True)
                    if 0 not in (axes or list(range(len(shape)))):
                        want = want[lo:hi]
                    n = max(2, int(np.prod([shape[a] for a in (axes or range(len(shape)))])))
                    if r.numel() != want.size or not np.allclose(r.numpy().ravel(), want.ravel(), rtol=1e-5 * np.log2(n), atol=0):
                        failures.append((op, axes, slot))
            try:
                many(local, slot=2)
                failures.append("slot range not checked")
            except ValueError:
                pass
        with open(os.path.join(out_dir, "many%d.txt" % rank), "w") as f:
            f.write(repr(failures))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,shape", [(2, (6, 5, 7)), (3, (2, 4, 3))])
def test_reduce_many_over_gloo(tmp_path, world, shape):
    """Several reductions behind one all-gather, two record slots; world 3 over a batch of 2 leaves a
    rank with an empty slab, which must contribute the neutral record instead of failing before the
    collective (the other ranks would wait in it for ever)."""
    port = 31500 + (os.getpid() % 2000) + world
    mp.spawn(_many_worker, args=(world, port, shape, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(os.path.join(str(tmp_path), "many%d.txt" % r)).read() == "[]"
