"""Binary Pow against the reference's powf (glibc, through the oracle's C loop) on 24 million operand pairs.

Pow has no exhaustive test (2^64 pairs), so the pairs are drawn to cover what the kernel distinguishes:
bases over the whole positive range with exponents that keep the result normal (the double-precision
exp(y * ln x) path), bases next to 1 with huge exponents (where ln x must be RELATIVELY accurate),
results around the overflow and underflow thresholds and in the denormal range, integer and
half-integer exponents, and zero / negative / denormal / infinite / NaN operands (the library's
double pow rounded once).  The bar is the one of the transcendental codes: at most 2 ulp, NaN for NaN.
"""
import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

N = 4_000_000


def _regimes():
    rng = np.random.Generator(np.random.PCG64(20240777))
    f32 = np.float32
    # 1. positive bases over all exponents of the float format, exponents scaled so that |y * log2 x| < 120
    xb = rng.integers(0x00800000, 0x7f800000, N, dtype=np.int64).astype(np.int32).view(f32)
    lg = np.log2(xb.astype(np.float64))
    y = (rng.uniform(-120, 120, N) / np.where(np.abs(lg) < 1e-3, 1e-3, lg)).astype(f32)
    yield "all positive bases", xb, y
    # 2. bases next to 1, exponents up to 1e7
    x = (1.0 + rng.uniform(-1e-3, 1e-3, N)).astype(f32)
    y = (rng.uniform(-1, 1, N) * 10.0 ** rng.uniform(0, 7, N)).astype(f32)
    yield "bases next to 1", x, y
    # 3. everyday operands
    yield "everyday", rng.uniform(0.01, 20, N).astype(f32), rng.uniform(-8, 8, N).astype(f32)
    # 4. results around overflow, underflow and in the denormal range
    x = rng.uniform(1.5, 50, N).astype(f32)
    target = rng.choice([-151.0, -149.0, -127.0, -126.0, -125.0, 126.0, 127.5, 128.5], N) + rng.uniform(-1.5, 1.5, N)
    yield "range limits", x, (target / np.log2(x.astype(np.float64))).astype(f32)
    # 5. integer and half-integer exponents, bases of both signs
    x = rng.uniform(-30, 30, N).astype(f32)
    yield "integer exponents", x, (rng.integers(-12, 13, N) * 0.5).astype(f32)
    # 6. special operands against each other and against ordinary numbers
    pool = np.array([0.0, -0.0, 1.0, -1.0, 2.0, -2.0, 0.5, -0.5, 3.0, -3.0, np.inf, -np.inf, np.nan, 1e-45, -1e-45, 1e-40,
                     3.4e38, -3.4e38, 1.1754944e-38, 0.99999994, 1.0000001, 2.5, -2.5, 1e10, -1e10], dtype=f32)
    x = pool[rng.integers(0, pool.size, N)]
    y = pool[rng.integers(0, pool.size, N)]
    half = N // 2
    x[:half // 2] = rng.uniform(-5, 5, half // 2).astype(f32)
    y[half // 2:half] = rng.uniform(-5, 5, half - half // 2).astype(f32)
    yield "special operands", x, y


def test_pow_pairs_within_two_ulp():
    import torch
    from shadow_b200 import functional as F
    for name, x, y in _regimes():
        want = orc.binary(x, y, 4)
        got = F.binary(torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda(), 4).cpu().numpy()
        d = orc.ulp_distance(got, want)
        worst = int(d.argmax())
        assert d[worst] <= 2, "%s: %d ulp at pow(%r, %r): got %r, reference %r (%d pairs above 2 ulp)" % (
            name, d[worst], x[worst], y[worst], got[worst], want[worst], int((d > 2).sum()))
        zeros = (got == 0) & (want == 0)
        assert np.array_equal(np.signbit(got[zeros]), np.signbit(want[zeros])), "%s: a zero of the wrong sign" % name
        print("%-20s pairs %d  0ulp %d  1ulp %d  2ulp %d" % (name, d.size, int((d == 0).sum()), int((d == 1).sum()), int((d == 2).sum())))


def test_pow_with_a_scalar_exponent():
    import torch
    from shadow_b200 import functional as F
    rng = np.random.Generator(np.random.PCG64(20240778))
    x = rng.uniform(0.0, 40.0, 1_000_003).astype(np.float32)
    for scalar in (2.0, 0.5, -1.5, 3.0, 0.0, 1.0, 7.25):
        want = orc.binary_scalar(x, scalar, 4)
        got = F.binary_scalar(torch.from_numpy(x).cuda(), scalar, 4).cpu().numpy()
        assert orc.ulp_distance(got, want).max() <= 2, scalar
