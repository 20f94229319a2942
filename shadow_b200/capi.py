"""ctypes binding of the kernel C ABI (``include/sb200.h`` -> ``shadow_b200/lib/libsb200.so``).

There is no fallback: if the compiled library is missing, or a call returns a non-zero status,
an exception is raised.  Pointers are raw device addresses (ints); ``stream`` is a cudaStream_t
value (int, 0 = default stream).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Sequence

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libsb200.so")

STATUS_OK = 0


class Sb200Error(RuntimeError):
    def __init__(self, status: int, what: str, detail: str = ""):
        self.status = status
        super().__init__("%s failed: status %d (%s)%s" % (what, status, status_string(status),
                                                          (": " + detail) if detail else ""))


_lib = None


def lib() -> C.CDLL:
    """The loaded kernel library.  Raises if it has not been built (python -m shadow_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("CUDA kernel library %s is missing: run `python -m shadow_b200.build` "
                              "(needs nvcc); there is no CPU fallback" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float
        ip = C.POINTER(C.c_int)
        sig = {
            "sb200_status_string": (C.c_char_p, [i32]),
            "sb200_last_cuda_error": (C.c_char_p, []),
            "sb200_device_sm_count": (i32, []),
            "sb200_launch_count": (C.c_longlong, []),
            "sb200_fill": (i32, [vp, i64, f32, vp]),
            "sb200_unary": (i32, [vp, vp, i64, i32, vp]),
            "sb200_activate": (i32, [vp, vp, i64, i32, f32, vp]),
            "sb200_prelu": (i32, [vp, vp, i64, i64, i64, vp, i32, vp]),
            "sb200_binary_scalar": (i32, [vp, f32, vp, i64, i32, vp]),
            "sb200_binary": (i32, [vp, vp, vp, i64, i32, vp]),
            "sb200_binary_broadcast": (i32, [vp, ip, vp, ip, ip, i32, vp, i32, vp]),
            "sb200_scale_bias": (i32, [vp, vp, i64, vp, vp, i64, i64, vp]),
            "sb200_reduce_scratch_bytes": (i64, [ip, i32, ip, i32, i32]),
            "sb200_reduce": (i32, [vp, ip, i32, ip, i32, i32, vp, vp, i64, vp]),
            "sb200_reduce_static": (i32, [vp, ip, i32, ip, i32, i32, vp, vp]),
            "sb200_reduce_partial": (i32, [vp, ip, i32, ip, i32, i32, vp, vp, i64, vp]),
            "sb200_reduce_finalize": (i32, [vp, vp, i64, i32, i64, vp]),
            "sb200_reduce_combine": (i32, [vp, i64, i64, vp, i64, i32, i64, vp]),
            "sb200_softmax": (i32, [vp, vp, i64, i64, i64, vp]),
            "sb200_softmax_ring_timeouts": (C.c_longlong, []),
            "sb200_eltwise": (i32, [C.POINTER(vp), i32, C.POINTER(f32), vp, i64, i32, vp]),
            "sb200_axpy": (i32, [vp, vp, vp, vp, i64, i64, vp]),
            "sb200_batch_norm": (i32, [vp, vp, i64, vp, vp, i64, i64, f32, f32, vp]),
            "sb200_normalize": (i32, [vp, vp, i64, i64, i64, f32, f32, vp]),
            "sb200_concat": (i32, [vp, vp, i32, vp, i64, vp]),
            "sb200_slice": (i32, [vp, vp, vp, i32, i64, vp]),
            "sb200_permute": (i32, [vp, vp, vp, vp, i32, vp]),
            "sb200_gather": (i32, [vp, vp, i64, i64, i64, i64, vp, vp]),
            "sb200_pad": (i32, [vp, vp, i64, i32, i32, vp, f32, vp]),
            "sb200_pooling": (i32, [vp, vp, i64, vp, vp, vp, vp, vp, i32, vp]),
            "sb200_ssd_normalize": (i32, [vp, vp, i64, i64, i64, i32, f32, vp, i32, vp]),
            "sb200_row_norm": (i32, [vp, vp, i64, i64, f32, vp, vp, i32, i64, i64, i64, vp]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)   # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


EXPORTED = ["sb200_status_string", "sb200_last_cuda_error", "sb200_device_sm_count", "sb200_launch_count",
            "sb200_fill", "sb200_unary", "sb200_activate", "sb200_prelu", "sb200_binary_scalar",
            "sb200_binary", "sb200_binary_broadcast", "sb200_scale_bias", "sb200_reduce_scratch_bytes",
            "sb200_reduce", "sb200_reduce_static", "sb200_reduce_partial", "sb200_reduce_finalize", "sb200_reduce_combine", "sb200_softmax", "sb200_softmax_ring_timeouts", "sb200_eltwise", "sb200_axpy", "sb200_batch_norm", "sb200_normalize", "sb200_ssd_normalize", "sb200_row_norm",
            "sb200_concat", "sb200_slice", "sb200_permute", "sb200_gather", "sb200_pad", "sb200_pooling"]


def status_string(status: int) -> str:
    return lib().sb200_status_string(status).decode()


def check(status: int, what: str) -> None:
    if status != STATUS_OK:
        detail = lib().sb200_last_cuda_error().decode() if status in (3, 4) else ""
        raise Sb200Error(status, what, detail)


def ints(seq: Sequence[int]):
    return (C.c_int * max(len(seq), 1))(*[int(v) for v in seq])


def launch_count() -> int:
    return int(lib().sb200_launch_count())
