"""ctypes binding of the cross-GPU combine library (``include/sb200_nccl.h`` ->
``shadow_b200/lib/libsb200_nccl.so``) and a small ``Communicator`` object over it.

A C or C++ host calls the same entry points directly; this module exists so that the Python
harnesses (``sharded``, ``bench.py``, the tests) go through the C ABI instead of
``torch.distributed`` for the one exchange the sharded path has.  ``torch.distributed`` is used
here for nothing but shipping the 128-byte identifier from rank 0 to the others.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

from . import capi

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libsb200_nccl.so")
ID_BYTES = 128
ERR_COMM = 5

EXPORTED = ["sb200_comm_last_error", "sb200_comm_new_id", "sb200_comm_create", "sb200_comm_destroy", "sb200_comm_query",
            "sb200_allreduce_partials", "sb200_allreduce_scalar", "sb200_allgather_records", "sb200_sharded_reduce_finish"]

_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built (python -m shadow_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: run `python -m shadow_b200.build` (needs NCCL's header and library)" % LIB_PATH)
        capi.lib()   # libsb200.so first: the combine kernel lives there
        L = C.CDLL(LIB_PATH)
        vp, i64, i32 = C.c_void_p, C.c_int64, C.c_int
        sig = {
            "sb200_comm_last_error": (C.c_char_p, []),
            "sb200_comm_new_id": (i32, [vp]),
            "sb200_comm_create": (i32, [vp, i32, i32, C.POINTER(vp)]),
            "sb200_comm_destroy": (i32, [vp]),
            "sb200_comm_query": (i32, [vp, C.POINTER(i32), C.POINTER(i32)]),
            "sb200_allreduce_partials": (i32, [vp, vp, i64, i32, vp]),
            "sb200_allreduce_scalar": (i32, [vp, vp, i32, vp]),
            "sb200_allgather_records": (i32, [vp, vp, vp, i64, vp]),
            "sb200_sharded_reduce_finish": (i32, [vp, vp, vp, i64, i32, C.POINTER(i32), i64, i64, C.POINTER(vp), vp]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(status: int, what: str) -> None:
    if status == ERR_COMM:
        raise capi.Sb200Error(status, what, lib().sb200_comm_last_error().decode())
    capi.check(status, what)


def new_id() -> bytes:
    buf = C.create_string_buffer(ID_BYTES)
    check(lib().sb200_comm_new_id(buf), "sb200_comm_new_id")
    return buf.raw


class Communicator:
    """One NCCL communicator on the current CUDA device, created through the C ABI."""

    def __init__(self, unique_id: bytes, n_ranks: int, rank: int):
        if len(unique_id) != ID_BYTES:
            raise ValueError("identifier must be %d bytes" % ID_BYTES)
        handle = C.c_void_p()
        check(lib().sb200_comm_create(unique_id, n_ranks, rank, C.byref(handle)), "sb200_comm_create")
        self.handle, self.n_ranks, self.rank = handle, n_ranks, rank

    @classmethod
    def from_process_group(cls, group=None) -> "Communicator":
        """Ranks of an initialised torch.distributed job: rank 0 makes the identifier, the job's
        own broadcast carries it, every rank then calls ncclCommInitRank through the C ABI.  The
        caller has already selected its CUDA device."""
        import torch.distributed as dist
        rank, size = dist.get_rank(group), dist.get_world_size(group)
        box = [new_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls(box[0], size, rank)

    def close(self) -> None:
        if self.handle is not None:
            check(lib().sb200_comm_destroy(self.handle), "sb200_comm_destroy")
            self.handle = None

    def query(self):
        n, r = C.c_int(0), C.c_int(0)
        check(lib().sb200_comm_query(self.handle, C.byref(n), C.byref(r)), "sb200_comm_query")
        return n.value, r.value

    def allreduce_partials(self, partial, operation: int, stream: int) -> None:
        check(lib().sb200_allreduce_partials(self.handle, partial.data_ptr(), partial.numel(), operation, stream),
              "sb200_allreduce_partials")

    def allgather_records(self, record, gathered, stream: int) -> None:
        if gathered.numel() != record.numel() * self.n_ranks:
            raise ValueError("gathered must hold one record per rank")
        check(lib().sb200_allgather_records(self.handle, record.data_ptr(), gathered.data_ptr(), record.numel(), stream),
              "sb200_allgather_records")

    def sharded_reduce_finish(self, record, gathered, operations: Sequence[int], count: int, total_reduced_count: int,
                              results: Sequence, stream: int) -> None:
        ops = (C.c_int * len(operations))(*[int(o) for o in operations])
        outs = (C.c_void_p * len(results))(*[r.data_ptr() for r in results])
        check(lib().sb200_sharded_reduce_finish(self.handle, record.data_ptr(), gathered.data_ptr(), record.numel(),
                                                len(operations), ops, count, total_reduced_count, outs, stream),
              "sb200_sharded_reduce_finish")
