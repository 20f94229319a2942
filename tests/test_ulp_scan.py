"""The comparison helpers behind the exhaustive GPU tests, checked on the host: `orc_ulp_scan` and
`orc_gelu_scan` (oracle/oracle_port.c) must report no distance for the reference's own values and must
see a perturbation of a few units in the last place, a NaN on one side, and a zero of the wrong sign."""
import ctypes as C

import numpy as np

from oracle import oracle as orc

N = 1 << 16
BASES = [0x3F000000, 0xBF800000, 0x00000000, 0x7F7FFF00, 0x42000000]   # around 0.5, -1, 0, the largest floats, 32


def _lib():
    lib = orc.port()
    lib.orc_ulp_scan.restype = C.c_int
    lib.orc_ulp_scan.argtypes = [C.c_int, C.c_uint32, C.c_uint32, C.c_int64, C.POINTER(C.c_float), C.POINTER(C.c_uint64),
                                 C.POINTER(C.c_int64), C.POINTER(C.c_uint32), C.c_int, C.POINTER(C.c_int)]
    lib.orc_gelu_scan.restype = C.c_int
    lib.orc_gelu_scan.argtypes = [C.c_uint32, C.c_uint32, C.c_int64, C.POINTER(C.c_float), C.POINTER(C.c_uint64), C.POINTER(C.c_int64)]
    return lib


def _inputs(base, stride=1):
    bits = (np.uint64(base) + np.arange(N, dtype=np.uint64) * np.uint64(stride)) & np.uint64(0xFFFFFFFF)
    return bits.astype(np.uint32).view(np.float32)


def _scan(lib, fn, base, got, stride=1):
    hist, stats, over, n_over = (C.c_uint64 * 5)(), (C.c_int64 * 3)(), (C.c_uint32 * 8)(), C.c_int(0)
    got = np.ascontiguousarray(got, dtype=np.float32)
    assert lib.orc_ulp_scan(fn, C.c_uint32(base), C.c_uint32(stride), got.size, got.ctypes.data_as(C.POINTER(C.c_float)), hist, stats,
                            over, 8, C.byref(n_over)) == 0
    return list(hist), list(stats), n_over.value


# scan code -> how the oracle's operator entry points compute the same function
SAME_FUNCTION = [(0, lambda x: orc.unary(x, 4)), (1, lambda x: orc.unary(x, 3)), (2, lambda x: orc.activate(x, 3)),
                 (3, lambda x: orc.activate(x, 4)), (4, lambda x: orc.activate(x, 5)), (5, lambda x: orc.unary(x, 14)),
                 (6, lambda x: orc.unary(x, 2)), (7, lambda x: orc.unary(x, 5)), (8, lambda x: orc.unary(x, 6)),
                 (9, lambda x: orc.unary(x, 7)), (10, lambda x: orc.unary(x, 8)), (11, lambda x: orc.unary(x, 9)),
                 (12, lambda x: orc.unary(x, 10))]


def test_scan_reports_zero_distance_for_the_oracle_operators():
    lib = _lib()
    with np.errstate(all="ignore"):
        for fn, op in SAME_FUNCTION:
            for base in BASES:
                hist, stats, n_over = _scan(lib, fn, base, op(_inputs(base)))
                assert hist == [N, 0, 0, 0, 0] and stats[0] == 0 and stats[2] == 0 and n_over == 0, (fn, hex(base), hist, stats)


def test_scan_sees_perturbations_nan_and_signed_zero():
    lib = _lib()
    base = 0x3F000000
    want = orc.unary(_inputs(base), 4)               # expf
    got = want.copy()
    got_bits = got.view(np.uint32)
    got_bits[10] += 1                                # 1 ulp
    got_bits[20] += 3                                # 3 ulp: above the bar
    got[30] = np.nan                                 # NaN on one side only
    hist, stats, n_over = _scan(lib, 0, base, got)
    assert hist[1] == 1 and hist[3] == 1 and hist[4] == 1 and n_over == 2 and stats[0] == 1 << 31
    # sin(-0) = -0: a +0 there is a zero of the wrong sign
    x = _inputs(0x80000000)
    got = orc.unary(x, 5).copy()
    got[0] = 0.0
    _, stats, _ = _scan(lib, 7, 0x80000000, got)
    assert stats[2] == 1
    # a stride covers every 61st pattern
    hist, _, _ = _scan(lib, 6, 0x3F000000, orc.unary(_inputs(0x3F000000, 61), 2), stride=61)
    assert hist[0] == N


def test_gelu_scan_accepts_the_oracle_and_flags_what_is_outside_its_bar():
    lib = _lib()
    for base in (0x3F000000, 0xC0400000, 0x00000000):   # 0.5, -3 (where 1 + erf cancels), 0
        x = _inputs(base)
        want = orc.activate(x, 8)
        hist, stats = (C.c_uint64 * 5)(), (C.c_int64 * 3)()
        assert lib.orc_gelu_scan(C.c_uint32(base), 1, N, want.ctypes.data_as(C.POINTER(C.c_float)), hist, stats) == 0
        assert list(hist) == [N, 0, 0, 0, 0] and stats[0] == 0
        bad = want.copy()
        bad[5] = bad[5] * np.float32(1.001) + np.float32(1e-6)
        assert lib.orc_gelu_scan(C.c_uint32(base), 1, N, bad.ctypes.data_as(C.POINTER(C.c_float)), hist, stats) == 0
        assert stats[0] == 1 and stats[1] == base + 5
