"""The cross-GPU combine on ONE GPU.

* The C entry points of libsb200_nccl.so through a one-rank communicator: ncclCommInitRank, the
  all-reduce, the all-gather and the gather-and-fold call really run (on NCCL) and give the
  single-device reduction.
* sharded.ReduceMany's record slots, side-stream exchange and join, driven with a stand-in
  communicator that plays the other ranks from precomputed partials of their slabs (several ranks as
  separate processes on one GPU are not an option: kernels that wait on each other must not share a GPU).
"""
import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def one_rank():
    from shadow_b200 import build as sbuild
    from shadow_b200 import comm
    if sbuild.build_comm() is None:
        pytest.skip("no NCCL on this machine")
    import torch
    torch.cuda.set_device(0)
    c = comm.Communicator(comm.new_id(), 1, 0)
    yield c
    c.close()


def test_one_rank_communicator(one_rank):
    import torch
    from oracle import oracle as orc
    from shadow_b200 import functional as F
    assert one_rank.query() == (1, 0)
    stream = torch.cuda.current_stream().cuda_stream
    full = cases.normal(901, (6, 40, 5))
    x = torch.from_numpy(full).cuda()
    ops = [1, 2, 3, 4, 6]
    axes = [0, 1]
    count = 5
    record = torch.empty(len(ops) * count + 3, dtype=torch.float64, device="cuda")   # records may carry spare room
    for i, op in enumerate(ops):
        F.reduce_partial(x, op, axes, out=record[i * count:(i + 1) * count])
    before = record.clone()
    one_rank.allreduce_partials(record[:count], 1, stream)        # one rank: values unchanged
    torch.cuda.synchronize()
    assert torch.equal(record[:count], before[:count])
    gathered = torch.empty_like(record)
    one_rank.allgather_records(record, gathered, stream)
    torch.cuda.synchronize()
    assert torch.equal(gathered[:len(ops) * count], record[:len(ops) * count])
    results = [torch.empty(count, device="cuda") for _ in ops]
    gathered.zero_()
    one_rank.sharded_reduce_finish(record, gathered, ops, count, 6 * 40, results, stream)
    torch.cuda.synchronize()
    for op, r in zip(ops, results):
        want = orc.reduce(full, op, axes, keep_dims=False)
        case = {"name": "one_rank", "op": "Reduce", "args": {"operation": op, "axes": axes}, "inputs": [full]}
        cases.assert_parity(case, r.cpu().numpy().reshape(want.shape), want)
    # argument checks that need a live communicator
    from shadow_b200 import capi
    with pytest.raises(capi.Sb200Error):
        one_rank.sharded_reduce_finish(record[:4], gathered, ops, count, 240, results, stream)   # record too short
    with pytest.raises(ValueError):
        one_rank.allgather_records(record, gathered[:-1], stream)


class _OtherRanks:
    """Stand-in for comm.Communicator inside one process: this process is rank `rank` of `n_ranks`;
    the records of the other ranks are given.  sharded_reduce_finish lays the records out as an
    all-gather would and folds them with the library's combine kernel on the current stream."""

    def __init__(self, n_ranks, rank, other_records):
        self.n_ranks, self.rank, self.others = n_ranks, rank, other_records
        self.calls = []

    def sharded_reduce_finish(self, record, gathered, operations, count, total, results, stream):
        import torch
        from shadow_b200 import functional as F
        assert stream == torch.cuda.current_stream().cuda_stream
        self.calls.append(stream)
        width = record.numel()
        for r in range(self.n_ranks):
            src = record if r == self.rank else self.others[r]
            gathered[r * width:(r + 1) * width].copy_(src)
        for i, op in enumerate(operations):
            F.reduce_combine(gathered[i * count:], self.n_ranks, width, count, op, total, out=results[i])


@pytest.mark.parametrize("rank", [0, 2])
def test_reduce_many_slots_and_side_stream(rank):
    import torch
    from oracle import oracle as orc
    from shadow_b200 import functional as F
    from shadow_b200 import sharded
    shape, world = (7, 24, 10), 3
    ops, axes, count = [1, 2, 4], [0, 1], 10
    fulls = [cases.normal(950 + s, shape) for s in range(3)]         # one tensor per slot
    bounds = [sharded.shard_bounds(shape[0], r, world) for r in range(world)]
    lo, hi = bounds[rank]
    side = torch.cuda.Stream()
    many = None
    for s, full in enumerate(fulls):
        others = {}
        for r, (a, b) in enumerate(bounds):
            if r == rank:
                continue
            rec = torch.empty(len(ops) * count, dtype=torch.float64, device="cuda")
            slab = torch.from_numpy(np.ascontiguousarray(full[a:b])).cuda()
            for i, op in enumerate(ops):
                F.reduce_partial(slab, op, axes, out=rec[i * count:(i + 1) * count])
            others[r] = rec
        fake = _OtherRanks(world, rank, others)
        if many is None:
            many = sharded.ReduceMany(ops, (hi - lo,) + shape[1:], axes, shape[0], torch.device("cuda", 0), comm=fake, slots=3)
        many.comm = fake
        local = torch.from_numpy(np.ascontiguousarray(full[lo:hi])).cuda()
        torch.cuda.synchronize()
        many(local, slot=s, side_stream=side)
        assert fake.calls == [side.cuda_stream]      # the exchange went to the side stream
    many.join()
    torch.cuda.current_stream().synchronize()        # joined: the side stream's work is ordered before this
    for s, full in enumerate(fulls):                 # every slot kept its own results
        for op, r in zip(ops, many.results[s]):
            want = orc.reduce(full, op, axes, keep_dims=False)
            case = {"name": "many", "op": "Reduce", "args": {"operation": op, "axes": axes}, "inputs": [full]}
            cases.assert_parity(case, r.cpu().numpy().reshape(want.shape), want)


def test_reduce_many_empty_slab_contributes_the_neutral_record():
    import torch
    from oracle import oracle as orc
    from shadow_b200 import functional as F
    from shadow_b200 import sharded
    full = cases.normal(990, (1, 6, 4))
    ops, axes, count = [1, 2, 3], [0, 2], 6
    rec0 = torch.empty(len(ops) * count, dtype=torch.float64, device="cuda")
    x0 = torch.from_numpy(full).cuda()
    for i, op in enumerate(ops):
        F.reduce_partial(x0, op, axes, out=rec0[i * count:(i + 1) * count])
    fake = _OtherRanks(2, 1, {0: rec0})                       # this process is rank 1 of 2 over a batch of 1
    many = sharded.ReduceMany(ops, (0, 6, 4), axes, 1, torch.device("cuda", 0), comm=fake)
    res = many(torch.empty(0, 6, 4, device="cuda"))
    torch.cuda.synchronize()
    for op, r in zip(ops, res):
        want = orc.reduce(full, op, axes, keep_dims=False)
        case = {"name": "empty", "op": "Reduce", "args": {"operation": op, "axes": axes}, "inputs": [full]}
        cases.assert_parity(case, r.cpu().numpy().reshape(want.shape), want)
