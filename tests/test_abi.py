"""The C-ABI library loads and exports every symbol include/sb200.h declares; argument checks
that happen before any launch.  Needs no GPU (no compute call is made)."""
import os
import re

import pytest

from shadow_b200 import build as sbuild
from shadow_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    sbuild.build_kernels()
    return capi.lib()


def declared_functions(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sb200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions("sb200.h")
    assert len(names) >= 17
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(capi.EXPORTED) == names


def test_status_strings(lib):
    assert capi.status_string(0) == "ok"
    assert "argument" in capi.status_string(1)
    assert "unknown" in capi.status_string(99)


def test_bad_arguments_are_rejected_before_launch(lib):
    before = capi.launch_count()
    assert lib.sb200_unary(None, None, 16, 0, None) == 1
    assert lib.sb200_unary(None, None, -1, 0, None) == 1
    assert lib.sb200_unary(256, 512, 16, 99, None) == 1            # unknown operation code
    assert lib.sb200_activate(256, 512, 16, 0, 0.1, None) == 1      # PReLU goes through sb200_prelu
    assert lib.sb200_binary(256, None, 512, 16, 0, None) == 1
    assert lib.sb200_binary_scalar(256, 1.0, 512, 16, 7, None) == 1
    assert lib.sb200_scale_bias(256, 512, 16, None, None, 4, 4, None) == 1
    assert lib.sb200_scale_bias(256, 512, 16, 1024, None, 0, 4, None) == 1
    assert lib.sb200_softmax(256, 512, 4, 0, 1, None) == 1
    assert lib.sb200_prelu(256, 512, 2, 3, 4, None, 0, None) == 1
    shp, bad = capi.ints([2, 3]), capi.ints([2, 4])
    assert lib.sb200_binary_broadcast(256, shp, 512, bad, shp, 2, 1024, 0, None) == 1   # 4 vs 3
    assert lib.sb200_reduce(256, shp, 2, capi.ints([2]), 1, 1, 512, None, 0, None) == 1  # axis out of range
    assert lib.sb200_reduce(256, shp, 2, capi.ints([1, 1]), 2, 1, 512, None, 0, None) == 1  # duplicate axis
    assert lib.sb200_reduce(256, shp, 2, capi.ints([1]), 1, 9, 512, None, 0, None) == 1  # unknown op
    assert lib.sb200_unary(258, 512, 16, 0, None) == 1              # not 4-byte aligned
    assert capi.launch_count() == before
    # the operators added after the first six
    import ctypes
    ptrs = (ctypes.c_void_p * 2)(256, 512)
    widths = (ctypes.c_int64 * 2)(4, 0)
    assert lib.sb200_eltwise(ptrs, 1, None, 1024, 16, 1, None) == 1                     # needs two inputs
    assert lib.sb200_axpy(256, 512, 768, 1024, 2, 0, None) == 1                        # inner < 1
    assert lib.sb200_batch_norm(256, 512, 16, None, 1024, 4, 4, 1.0, 1e-5, None) == 1   # no mean
    assert lib.sb200_normalize(256, 512, 2, 0, 4, 2.0, 1e-12, None) == 1                # dim < 1
    assert lib.sb200_ssd_normalize(256, 512, 2, 0, 4, 1, 1e-5, None, 1, None) == 1
    assert lib.sb200_row_norm(256, 512, 2, 8, 1e-5, None, None, 1, 1, 1, 1, None) == 1  # affine without scale
    assert lib.sb200_row_norm(256, 512, 2, 8, 1e-5, 1024, 2048, 2, 2, 3, 2, None) == 1  # 3*2 != inner
    assert lib.sb200_concat(ptrs, widths, 2, 1024, 3, None) == 1                        # a zero width
    assert lib.sb200_slice(256, ptrs, widths, 2, 3, None) == 1
    assert lib.sb200_permute(256, 512, shp, capi.ints([0, 0]), 2, None) == 1            # not a permutation
    assert lib.sb200_permute(256, 256, shp, capi.ints([1, 0]), 2, None) == 1            # in place
    assert lib.sb200_gather(256, None, 2, 1, 4, 3, 512, None) == 1                      # no indexes
    assert lib.sb200_pad(256, 512, 2, 4, 4, capi.ints([-3, -3, 0, 0]), 0.0, None) == 1  # nothing left
    three = capi.ints([1, 4, 4])
    assert lib.sb200_pooling(256, 512, 2, three, three, capi.ints([1, 0, 2]), three, capi.ints([0, 0, 0]), 0, None) == 1
    assert lib.sb200_pooling(256, 512, 2, three, three, three, three, capi.ints([0, 0, 0]), 2, None) == 1  # pool type
    assert capi.launch_count() == before
    # zero-size calls succeed without launching
    assert lib.sb200_concat(ptrs, widths, 2, None, 0, None) == 0
    assert lib.sb200_unary(None, None, 0, 0, None) == 0
    assert lib.sb200_fill(None, 0, 1.0, None) == 0
    assert capi.launch_count() == before


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", "/nonexistent/libsb200.so")
    with pytest.raises(ImportError):
        capi.lib()


def test_comm_library_exports_and_argument_checks():
    """libsb200_nccl.so (include/sb200_nccl.h): every declared symbol is exported; arguments are
    checked before NCCL is touched, so this needs neither a GPU nor peers."""
    import ctypes
    from shadow_b200 import comm
    if sbuild.build_comm() is None:
        pytest.skip("no NCCL header/library on this machine")
    L = comm.lib()
    names = declared_functions("sb200_nccl.h")
    assert sorted(comm.EXPORTED) == names
    for name in names:
        assert hasattr(L, name), name
    assert L.sb200_comm_new_id(None) == 1
    handle = ctypes.c_void_p()
    ident = b"\0" * comm.ID_BYTES
    assert L.sb200_comm_create(ident, 2, 2, ctypes.byref(handle)) == 1      # rank outside the world
    assert L.sb200_comm_create(ident, 0, 0, ctypes.byref(handle)) == 1
    assert L.sb200_comm_create(None, 1, 0, ctypes.byref(handle)) == 1
    assert L.sb200_comm_destroy(None) == 1
    assert L.sb200_comm_query(None, None, None) == 1
    assert L.sb200_allreduce_partials(None, 256, 4, 1, None) == 1           # no communicator
    assert L.sb200_allgather_records(None, 256, 512, 4, None) == 1
    ops = (ctypes.c_int * 1)(1)
    outs = (ctypes.c_void_p * 1)(1024)
    assert L.sb200_sharded_reduce_finish(None, 256, 512, 4, 1, ops, 4, 8, outs, None) == 1
    assert L.sb200_comm_last_error() == b""
    with pytest.raises(ValueError):
        comm.Communicator(b"short", 1, 0)
