"""Every float bit pattern through the transcendental operators of the library as built.

Exp, Log and the six trigonometric codes (`sb200_unary`), Sigmoid, SoftPlus and Tanh (`sb200_activate`) are run on
the GPU over all 2^32 float inputs (64 launches of 2^26 elements each) and compared on the host with the reference's
own CPU arithmetic - glibc's expf / logf / tanhf / sinf ... atanf and the compositions 1/(1+expf(-x)) and
log1pf(expf(x)) of shadow/operators/kernels/activate.cpp:15-26 and shadow/core/blas.cpp:143-167 -
evaluated by the oracle's C helper on all host threads.  The bar is the one the operators are built
to: at most 2 ulp from the reference on EVERY input, NaN for NaN, no zero of the wrong sign.
Reciprocal and Sqrt are single IEEE operations and must be bit-exact everywhere.

A machine with fewer than 8 host threads scans every 61st bit pattern instead (70 million inputs per
function, all exponents and both signs), so the test stays within a few minutes.

The table of per-function histograms is written to the test's stdout (`pytest -s`) and, when
`SB200_ULP_TABLE` names a file, to that file.
"""
import ctypes as C
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

CHUNK = 1 << 26
# (name, scan code of the oracle helper, how to run it on the device, ulp bar)
FUNCTIONS = [
    ("Exp", 0, ("unary", 4), 2),
    ("Log", 1, ("unary", 3), 2),
    ("Sigmoid", 2, ("activate", 3), 2),
    ("SoftPlus", 3, ("activate", 4), 2),
    ("Tanh", 4, ("activate", 5), 2),
    ("Reciprocal", 5, ("unary", 14), 0),
    ("Sqrt", 6, ("unary", 2), 0),
    ("Sin", 7, ("unary", 5), 2),
    ("Cos", 8, ("unary", 6), 2),
    ("Tan", 9, ("unary", 7), 2),
    ("Asin", 10, ("unary", 8), 2),
    ("Acos", 11, ("unary", 9), 2),
    ("Atan", 12, ("unary", 10), 2),
]


def _scan_lib():
    lib = orc.port()
    lib.orc_ulp_scan.restype = C.c_int
    lib.orc_ulp_scan.argtypes = [C.c_int, C.c_uint32, C.c_uint32, C.c_int64, C.POINTER(C.c_float), C.POINTER(C.c_uint64),
                                 C.POINTER(C.c_int64), C.POINTER(C.c_uint32), C.c_int, C.POINTER(C.c_int)]
    return lib


def _scan_slice(lib, code, base, stride, got):
    """One host thread's share: got[i] belongs to the float with bits base + i*stride."""
    hist = (C.c_uint64 * 5)()
    stats = (C.c_int64 * 3)()
    over = (C.c_uint32 * 64)()
    n_over = C.c_int(0)
    rc = lib.orc_ulp_scan(code, C.c_uint32(base & 0xFFFFFFFF), C.c_uint32(stride), got.size,
                          got.ctypes.data_as(C.POINTER(C.c_float)), hist, stats, over, 64, C.byref(n_over))
    assert rc == 0
    return list(hist), list(stats), [over[i] for i in range(min(n_over.value, 64))], n_over.value


def _device_results(how, threads):
    """Runs one function over every float bit pattern (every 61st on a small host) and yields, launch
    by launch, (first bit pattern, stride, results on the host)."""
    import torch
    from shadow_b200 import functional as F
    full = threads >= 8
    dev = torch.device("cuda", 0)
    out_dev = torch.empty(CHUNK, dtype=torch.float32, device=dev)
    host = torch.empty(CHUNK, dtype=torch.float32).pin_memory()
    stride = 1 if full else 61
    per = CHUNK * stride            # bit patterns covered per launch
    for base in range(0, 1 << 32, per):
        count = min(CHUNK, ((1 << 32) - base + stride - 1) // stride)
        bits64 = torch.arange(base, base + count * stride, stride, dtype=torch.int64, device=dev)
        # the int64 pattern -> the float with those 32 bits
        x = torch.where(bits64 >= (1 << 31), bits64 - (1 << 32), bits64).to(torch.int32).view(torch.float32)
        y = out_dev[:count]
        if how[0] == "unary":
            F.unary(x, how[1], out=y)
        else:
            F.activate(x, how[1], 0.1, out=y)
        host[:count].copy_(y)
        torch.cuda.synchronize()
        yield base, stride, host[:count].numpy()


def _expected_total(threads):
    return (1 << 32) if threads >= 8 else len(range(0, 1 << 32, 61))


def _report(line):
    print(line)
    table = os.environ.get("SB200_ULP_TABLE")
    if table:
        with open(table, "a") as fh:
            fh.write(line + "\n")


@pytest.mark.parametrize("name,code,how,bar", FUNCTIONS, ids=[f[0] for f in FUNCTIONS])
def test_every_float_within_the_bar(name, code, how, bar):
    lib = _scan_lib()
    threads = os.cpu_count() or 1
    hist, worst, wrong_sign, over, n_over = [0] * 5, (0, 0), 0, [], 0
    pool = ThreadPoolExecutor(max_workers=threads)
    for base, stride, got in _device_results(how, threads):
        count = got.size
        share = (count + threads - 1) // threads
        jobs = [pool.submit(_scan_slice, lib, code, base + lo * stride, stride, got[lo:lo + share])
                for lo in range(0, count, share)]
        results = [j.result() for j in jobs]
        for h, st, o, n in results:
            hist = [a + c for a, c in zip(hist, h)]
            if st[0] > worst[0]:
                worst = (st[0], st[1])
            wrong_sign += st[2]
            over, n_over = (over + o)[:64], n_over + n
    pool.shutdown()
    total = sum(hist)
    _report("%-10s inputs %d  0ulp %d  1ulp %d  2ulp %d  3ulp %d  >=4ulp %d  max %d at 0x%08x  wrong-sign zeros %d" % (
        name, total, hist[0], hist[1], hist[2], hist[3], hist[4], worst[0], worst[1], wrong_sign))
    assert total == _expected_total(threads)
    assert worst[0] <= bar, "%s: %d inputs above %d ulp, first ones %s" % (
        name, n_over if bar == 2 else total - hist[0], bar, ["0x%08x" % b for b in over[:16]])
    assert wrong_sign == 0, "%s: %d zeros of the wrong sign" % (name, wrong_sign)


def _gelu_slice(lib, base, stride, got):
    hist = (C.c_uint64 * 5)()
    stats = (C.c_int64 * 3)()
    rc = lib.orc_gelu_scan(C.c_uint32(base & 0xFFFFFFFF), C.c_uint32(stride), got.size, got.ctypes.data_as(C.POINTER(C.c_float)),
                           hist, stats)
    assert rc == 0
    return list(hist), list(stats)


def test_gelu_on_every_float():
    """Gelu = 0.5f*x*(1 + erff(0.707107f*x)) (shadow/operators/kernels/activate.cpp:25-26).  For x << 0 the sum
    1 + erf cancels, so a one-ulp difference in erf is magnified in the result; the bar is therefore 2 ulp of
    the result plus one ulp of erf (2^-24) times |x/2|, and it has to hold on every input."""
    lib = _scan_lib()
    lib.orc_gelu_scan.restype = C.c_int
    lib.orc_gelu_scan.argtypes = [C.c_uint32, C.c_uint32, C.c_int64, C.POINTER(C.c_float), C.POINTER(C.c_uint64), C.POINTER(C.c_int64)]
    threads = os.cpu_count() or 1
    hist, outside, first, wrong_sign = [0] * 5, 0, None, 0
    pool = ThreadPoolExecutor(max_workers=threads)
    for base, stride, got in _device_results(("activate", 8), threads):
        share = (got.size + threads - 1) // threads
        jobs = [pool.submit(_gelu_slice, lib, base + lo * stride, stride, got[lo:lo + share]) for lo in range(0, got.size, share)]
        for h, st in [j.result() for j in jobs]:
            hist = [a + c for a, c in zip(hist, h)]
            if st[0] and first is None:
                first = st[1]
            outside += st[0]
            wrong_sign += st[2]
    pool.shutdown()
    total = sum(hist)
    _report("%-10s inputs %d  0ulp %d  1ulp %d  2ulp %d  3ulp %d  >=4ulp %d  outside 2 ulp + |x/2|*2^-24: %d  wrong-sign zeros %d" % (
        "Gelu", total, hist[0], hist[1], hist[2], hist[3], hist[4], outside, wrong_sign))
    assert total == _expected_total(threads)
    assert outside == 0, "Gelu: %d inputs outside the bar, the first one 0x%08x" % (outside, first or 0)
    assert wrong_sign == 0
