// Per-element arithmetic of the operators, written so that results match the reference's CPU
// build: every + - * / is one IEEE round-to-nearest operation (explicit __f*_rn intrinsics, so
// the compiler can never contract a multiply and an add into an FMA), comparisons pick operands
// exactly like std::max / std::min, and transcendental functions stay within 2 ulp of glibc's
// float functions (which are within 1 ulp of the true value, mostly correctly rounded).
#pragma once

#include <cuda_runtime.h>
#include <math_constants.h>

#include "sb200.h"

namespace sb200 {

// ---- transcendental functions -------------------------------------------------------------------
// The parity bar is 2 ulp against glibc's float functions, checked over ALL 2^32 float inputs
// (tests/test_gpu_ulp_exhaustive.py).  CUDA's logf is within 1 ulp of glibc's everywhere (used as
// is); CUDA's expf reaches 2 ulp and tanhf 3 ulp, and the reference's Sigmoid composition
// 1/(1+expf(-x)) magnifies a 1-ulp difference in expf up to 4 ulp where 1+e^-x crosses 2^24.  So
// e^x follows glibc's own algorithm step by step (expf_like_glibc: the same bits as glibc 2.39 on
// every input), Sigmoid builds on it with IEEE operations and is therefore bit-exact too, and
// Tanh uses a double-precision e^x (exp_core) and rounds once at the end.

// 2^(i/32) as a double's bit pattern minus i << 47, i = 0..31: the table of the expf algorithm below
// (each entry the correctly rounded double of 2^(i/32)); two 128-byte lines.
__device__ __align__(128) const unsigned long long kExp2fTable[32] = {
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull};

// expf as glibc computes it (sysdeps/ieee754/flt-32/e_expf.c, the algorithm of Arm's optimized
// routines): in double, x*32/ln2 = k + r with k an integer (found by adding 1.5*2^52), e^x =
// 2^(k/32) * 2^(r/32) with 2^(k/32) from a 32-entry table and its exponent field, 2^(r/32) by a cubic;
// the double result is rounded once to float.  The fused steps (the rounding step k, the residual r and
// the polynomial) are the ones glibc's build for processors with FMA contracts; with them the result
// equals glibc 2.39's expf on all 2^32 inputs (checked on the host), and a build without FMA differs
// on two inputs by one ulp.
// The six double constants of expf_like_glibc held in (vector) REGISTERS for a whole thread.  Written
// as literals they are materialised again and again through uniform registers and moves (profile: 5-7
// integer move instructions per element); read once per thread through an index the compiler cannot
// fold (a zero loaded from memory) they stay in twelve registers.  Used by Sigmoid (34 instead of 40
// instructions per element, 0.74 instead of 0.70 of 8 TB/s).  The same treatment made Tanh slower (the
// compiler moved its nine constants back to uniform registers) and delays the start of the plain Exp,
// which streams at the DRAM limit anyway: both keep literals.
struct ExpfConsts {
  double inv_ln2n, shift, c0, c1, c2, one;
};
__device__ const double kExpfConstTable[6] = {0x1.71547652b82fep+0 * 32.0, 0x1.8p+52,
                                             0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0, 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0,
                                             0x1.62e42ff0c52d6p-1 / 32.0, 1.0};
__device__ int g_expf_zero = 0;
__device__ __forceinline__ ExpfConsts load_expf_consts() {
  int z;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(z) : "l"(&g_expf_zero));
  ExpfConsts k;
  k.inv_ln2n = kExpfConstTable[z + 0], k.shift = kExpfConstTable[z + 1], k.c0 = kExpfConstTable[z + 2];
  k.c1 = kExpfConstTable[z + 3], k.c2 = kExpfConstTable[z + 4], k.one = kExpfConstTable[z + 5];
  return k;
}
// expf_like_glibc with the constants passed in (same operations, same bits).
__device__ __forceinline__ float expf_like_glibc(float x, const ExpfConsts& c) {
  float xc;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(xc) : "f"(x), "f"(-104.5f));
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(xc) : "f"(xc), "f"(89.f));
  const double xd = static_cast<double>(xc);
  double kd = fma(c.inv_ln2n, xd, c.shift);
  const int ki = __double2loint(kd);
  kd = __dsub_rn(kd, c.shift);
  const double r = fma(c.inv_ln2n, xd, -kd);
  const double tab = __longlong_as_double(static_cast<long long>(__ldg(&kExp2fTable[ki & 31])));
  const double s = __hiloint2double(__double2hiint(tab) + static_cast<int>(static_cast<unsigned>(ki) << 15), __double2loint(tab));
  const double q = fma(c.c0, r, c.c1);
  const double r2 = __dmul_rn(r, r);
  double y = fma(c.c2, r, c.one);
  y = fma(q, r2, y);
  y = __dmul_rn(y, s);
  return static_cast<float>(y);
}

__device__ __forceinline__ float expf_like_glibc(float x) {
  constexpr double kInvLn2N = 0x1.71547652b82fep+0 * 32.0;
  constexpr double kShift = 0x1.8p+52;
  constexpr double kC0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0, kC1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0,
                   kC2 = 0x1.62e42ff0c52d6p-1 / 32.0;
  // Beyond these bounds the float result is inf / 0 (also for the infinities).  The clamps are the
  // NaN-propagating forms, so a NaN runs through the arithmetic and comes out as a NaN by itself.
  float xc;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(xc) : "f"(x), "f"(-104.5f));
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(xc) : "f"(xc), "f"(89.f));
  const double xd = static_cast<double>(xc);
  double kd = fma(kInvLn2N, xd, kShift);              // k = round(x*32/ln2) sits in the low word
  const int ki = __double2loint(kd);
  kd = __dsub_rn(kd, kShift);
  const double r = fma(kInvLn2N, xd, -kd);
  // 2^(k/32): the table entry with k>>5 added to its exponent field (k << 47 in the 64-bit pattern,
  // which touches the high word only)
  const double tab = __longlong_as_double(static_cast<long long>(__ldg(&kExp2fTable[ki & 31])));
  const double s = __hiloint2double(__double2hiint(tab) + static_cast<int>(static_cast<unsigned>(ki) << 15), __double2loint(tab));
  const double q = fma(kC0, r, kC1);
  const double r2 = __dmul_rn(r, r);
  double y = fma(kC2, r, 1.0);
  y = fma(q, r2, y);
  y = __dmul_rn(y, s);
  return static_cast<float>(y);
}

// 2^(j/16), j = 0..15: one 128-byte line, so a warp's 32 lookups are a single L1 transaction.
__device__ __align__(128) const double kExp2Sixteenths[16] = {
    1.0,                1.0442737824274138, 1.0905077326652577, 1.1387886347566916,
    1.189207115002721,  1.241857812073484,  1.2968395546510096, 1.3542555469368927,
    1.4142135623730951, 1.4768261459394993, 1.5422108254079407, 1.6104903319492543,
    1.681792830507429,  1.7562521603732995, 1.8340080864093424, 1.9152065613971474};

// e^x for x in [-105, 90], as a double with relative error < 1e-10 (table-driven reduction, the
// classic scheme): x = k*(ln2/16) + r with k = round(x*16/ln2), |r| <= ln2/32, then
// e^x = 2^(k>>4) * 2^((k&15)/16) * e^r with e^r by its degree-4 Taylor polynomial
// (r^5/120 < 4.1e-11).  k is found by adding the 1.5*2^52 rounding constant in double (no
// conversion instruction); the reduction is one fused multiply-add with ln2/16 in double.
// The two factors are returned separately so that a caller can fuse the last multiplication with what follows
// (1 - e^x, (e^x + 1)/2): e^x = p * scale * 2^-bias_down, with scale an exact power-of-two multiple of the table entry.
struct ExpParts {
  double p, scale;
};
__device__ __forceinline__ ExpParts exp_parts(double xd, int bias_down) {
  const double kRound = 6755399441055744.0;                 // 1.5 * 2^52: adding it rounds to an integer
  const double t = fma(xd, 23.083120654223414, kRound);     // x * 16/ln2, integer part in the low word
  const int ki = __double2loint(t);                         // k as a signed integer (|k| < 2^12)
  const double kd = t - kRound;
  // one-step reduction: the rounding of ln2/16 to double moves r by at most 2^9 * 5e-18, far below the
  // 4e-11 of the polynomial
  const double r = fma(kd, -0.043321698784996581, xd);
  ExpParts e;
  e.p = fma(r, 4.16666666666666666667e-02, 1.66666666666666666667e-01);
  e.p = fma(e.p, r, 0.5);
  e.p = fma(e.p, r, 1.0);
  e.p = fma(e.p, r, 1.0);
  // 2^(k>>4 - bias_down) * 2^((k&15)/16) through the table entry's exponent field; k>>4 stays within [-152, 130]
  const double tab = __ldg(&kExp2Sixteenths[ki & 15]);      // in [1, 2)
  e.scale = __hiloint2double(__double2hiint(tab) + (((ki >> 4) - bias_down) << 20), __double2loint(tab));
  return e;
}
__device__ __forceinline__ double exp_core(double xd) {
  const ExpParts e = exp_parts(xd, 0);
  return e.p * e.scale;
}
__device__ __forceinline__ double exp_core(float x) { return exp_core(static_cast<double>(x)); }

// 1/d for a positive double d whose float image and its reciprocal are normal floats (the callers'
// ranges: [1e-10, 1e9]), relative error ~1e-14: hardware float reciprocal as the seed,
// one Newton step in double (a full double division costs an order of magnitude more).  The seed
// goes double -> float -> double by bit manipulation (truncation is fine for a seed), because
// each cvt instruction costs a slot of the conversion unit, the busiest pipe of the tanh kernel.
__device__ __forceinline__ double rcp_newton(double d) {
  const float df = __double2float_rz(d);   // (the kernel is bound by instruction issue: one conversion beats four integer operations)
  float seed;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(seed) : "f"(df));
  const unsigned sb = __float_as_uint(seed);                                   // positive, normal
  const double r0 = __hiloint2double(static_cast<int>((sb >> 3) + 0x38000000u), static_cast<int>(sb << 29));
  return fma(r0, fma(-d, r0, 1.0), r0);
}

// 1/y for a float y >= 1 (or +inf, or NaN), correctly rounded wherever the result is a normal float:
// hardware seed (within 1 ulp) and one fma correction, r1 = r0 + r0*(1 - y*r0), computed on y * 2^-32 so
// that seed and result stay normal for every y (no denormal handling code around the flush-to-zero
// seed, no branch), then scaled back by 2^-32 - exact unless the result is denormal (y > 2^126), where
// this second rounding can differ from the IEEE quotient by one unit of the denormal grid (through
// Sigmoid: 34,015 of the 2^32 inputs, all with x < -87.3).  Infinity gives 0, a NaN runs through.
__device__ __forceinline__ float rcp_correct(float y) {
  const float ys = __fmul_rn(y, 0x1p-32f);
  float r0;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(ys));
  const float e = fmaf(-ys, r0, 1.0f);
  const float r1 = fmaf(r0, e, r0);
  return (y == CUDART_INF_F) ? 0.f : __fmul_rn(r1, 0x1p-32f);
}

// tanh(x) = 1 - 2/(e^{2|x|} + 1) in double, rounded once; for |x| < 2^-12 the float result is x
// itself (tanh x = x - x^3/3 and the correction is below half an ulp).  The exponential is exp_core's scheme
// written out so that its last multiplication, the addition of 1 and a halving are ONE fused multiply-add:
// wh = p * (table entry with the exponent k>>4 - 1) + 0.5 = (e^{2|x|} + 1) / 2, whose reciprocal is the
// 2/(e^{2|x|} + 1) that is wanted (11 double-precision instructions in all, two fewer than through exp_core;
// the results are the same bit for bit).
__device__ __forceinline__ float tanh_accurate(float x) {
  const float ax = fminf(fabsf(x), 10.f);         // beyond 10, 1 - 2e^{-2|x|} rounds to 1 (also for inf)
  const ExpParts e = exp_parts(static_cast<double>(ax + ax), 1);   // e^{2|x|} / 2 = e.p * e.scale
  const double wh = fma(e.p, e.scale, 0.5);        // (e^{2|x|} + 1) / 2 in [1, 2.5e8]
  const double q = rcp_newton(wh);                 // 2 / (e^{2|x|} + 1)
  const double t = 1.0 - q;
  const float y = copysignf(static_cast<float>(t), x);
  // tiny arguments (and +-0) return x itself, and so does a NaN: one test covers both
  return (fabsf(x) >= 2.44140625e-4f) ? y : x;
}

// tan(x) rounded to float.  |x| < 2^20: x = k*(pi/2) + r in double (k by the 1.5*2^52 rounding constant, pi/2 as
// two doubles: the fused steps leave r accurate to 1e-16 of ITSELF even where a float lies within 1e-9 of a
// multiple of pi/2), sin r and cos r by their Taylor polynomials up to r^11 and r^10 (|r| <= pi/4: truncation
// below 2e-10 relative), then sin/cos or -cos/sin by k's parity through a Newton reciprocal.  The result is the
// correctly rounded tangent on all but a fraction of a percent of inputs and within one ulp of it on those.
// Larger arguments, infinities and NaN take the library's double tan (its argument reduction works for any size).
__device__ __forceinline__ float tan_accurate(float x) {
  if (!(fabsf(x) < 1048576.f)) return static_cast<float>(tan(static_cast<double>(x)));
  const double xd = static_cast<double>(x);
  const double kRound = 6755399441055744.0;
  const double t = fma(xd, 0.63661977236758138, kRound);
  const int k = __double2loint(t);
  const double kd = t - kRound;
  double r = fma(kd, -1.5707963267948966, xd);
  r = fma(kd, -6.123233995736766e-17, r);
  const double r2 = r * r;
  double sp = -2.505210838544172e-08;
  sp = fma(sp, r2, 2.7557319223985893e-06);
  sp = fma(sp, r2, -0.00019841269841269841);
  sp = fma(sp, r2, 0.0083333333333333332);
  sp = fma(sp, r2, -0.16666666666666666);
  sp = fma(sp * r2, r, r);                    // sin r
  double cp = -2.7557319223985888e-07;
  cp = fma(cp, r2, 2.4801587301587302e-05);
  cp = fma(cp, r2, -0.0013888888888888889);
  cp = fma(cp, r2, 0.041666666666666664);
  cp = fma(cp, r2, -0.5);
  cp = fma(cp, r2, 1.0);                      // cos r
  const bool odd = (k & 1) != 0;
  double num = odd ? -cp : sp;
  const double den = odd ? sp : cp;           // |den| >= 1e-10 for a float argument: its reciprocal is a normal float
  num = den < 0.0 ? -num : num;
  const float y = static_cast<float>(num * rcp_newton(fabs(den)));
  return (x == 0.f) ? x : y;                 // tan(-0) = -0 (the polynomial's sum of zeros comes out positive)
}

// pow(x, y) rounded to float.  Fast path for a positive normal x, a finite y and a result well inside the
// normal range (|y * ln x| <= 87): exp(y * ln x) in double, with ln x = k*ln2 + ln m, m in [sqrt(1/2), sqrt(2)),
// ln m = 2*atanh(s), s = (m - 1)/(m + 1), by its odd series up to s^13 (|s| <= 0.1716: truncation below 1e-12
// relative, and relative also when x is close to 1, where y may be huge), the quotient through a Newton
// reciprocal; the product and the exponential keep a relative error near 1e-10, so the float result is the
// correctly rounded power on all but about one input in a thousand and within one ulp of it on those (glibc's
// powf, the reference, is within one ulp too).  Everything else - zero, negative, denormal, infinite or NaN
// operands, results that overflow, underflow or are denormal - takes the library's double pow rounded once,
// which carries powf's special cases.  The slow path costs a warp about ten times the fast one, so tensors of
// positive values run at the fast path's speed.
__device__ __forceinline__ float pow_accurate(float x, float y) {
  const int xb = __float_as_int(x);
  bool fast = (xb >= 0x00800000) && (xb < 0x7f800000) && (fabsf(y) < CUDART_INF_F);
  double l = 0.0;
  if (fast) {
    const int k = (xb - 0x3f3504f3) >> 23;                  // m = x * 2^-k in [0.7071068, 1.4142135)
    const double m = static_cast<double>(__int_as_float(xb - (k << 23)));
    const double f = m - 1.0;
    const double s = f * rcp_newton(2.0 + f);
    const double s2 = s * s;
    double p = 2.0 / 13.0;
    p = fma(p, s2, 2.0 / 11.0);
    p = fma(p, s2, 2.0 / 9.0);
    p = fma(p, s2, 2.0 / 7.0);
    p = fma(p, s2, 2.0 / 5.0);
    p = fma(p, s2, 2.0 / 3.0);
    p = fma(p, s2, 2.0);
    const double lnx = fma(static_cast<double>(k), 0.69314718055994531, s * p);
    l = static_cast<double>(y) * lnx;
    fast = fabs(l) <= 87.0;
  }
  if (fast) return static_cast<float>(exp_core(l));
  return static_cast<float>(pow(static_cast<double>(x), static_cast<double>(y)));
}

// erf(t) rounded to float from a double evaluation with absolute error < 1e-9 (so the result is the
// correctly rounded float on all but a few percent of inputs, and within one ulp of it on those):
// erf(|t|) = 1 - exp(-|t| * Q(|t|)) with Q = -log(erfc(t)) / t, a smooth function on (0, 4]
// fitted here by a degree-12 polynomial in u = t/2 - 1 (least squares on Chebyshev nodes against a
// double-precision erfc; fit error 8.1e-10 absolute, 3.2e-9 relative in erf; degree 14 gives 4.7e-11 and
// costs two more instructions).  Beyond 4 the float result is 1 (1 - erf(4) = 1.5e-8 is below half an ulp of 1); below 2^-13 erf(t) = 2t/sqrt(pi) to
// within t^2/3 < 2^-27 relative.  One code path for every lane: about 22 double-precision
// instructions against the several times more of the library's erf, which is exact to 1e-16.
__device__ __forceinline__ float erf_accurate(float t) {
  const float at = fminf(fabsf(t), 4.0f);
  const double a = static_cast<double>(at);
  const double u = fma(a, 0.5, -1.0);
  double q = 7.925364052454135e-06;
  q = fma(q, u, 1.9407545862610534e-05);
  q = fma(q, u, -0.00012562602419222807);
  q = fma(q, u, 0.00021772371069488542);
  q = fma(q, u, -0.00021807212067134331);
  q = fma(q, u, -3.2761795408242533e-05);
  q = fma(q, u, 0.0013293422255206775);
  q = fma(q, u, -0.0056599643885220955);
  q = fma(q, u, 0.017386238525634652);
  q = fma(q, u, -0.045951902259856459);
  q = fma(q, u, 0.11181143059940291);
  q = fma(q, u, 1.7356902054909418);
  q = fma(q, u, 2.6824706331264441);
  const ExpParts ex = exp_parts(-(a * q), 0);
  const double e = fma(-ex.p, ex.scale, 1.0);   // 1 - e^{-a q}: the product and the subtraction in one rounding
  const double r = (at < 1.220703125e-4f) ? a * 1.1283791670955126 : e;
  return copysignf(static_cast<float>(r), t);
}

// x / d, correctly rounded, without the division instruction.  `rcp` is the correctly rounded
// reciprocal of d.  q0 = x*rcp is within an ulp of the quotient, the residual r = x - d*q0 is
// exact in one fused multiply-add, and q0 + r*rcp rounds to the IEEE quotient (Markstein's
// division step).  That argument needs every intermediate to stay a normal float, which holds
// when |x| and d lie in [2^-60, 2^60] (`d_ok` covers d); anything else - zeros, denormals, huge
// values, infinities, NaN - takes the division instruction.
__device__ __forceinline__ float div_exact(float x, float d, float rcp, bool d_ok) {
  const uint32_t ax = __float_as_uint(x) & 0x7fffffffu;
  const uint32_t lo = (127u - 60u) << 23, hi = (127u + 60u) << 23;
  if (d_ok && (ax - lo) <= (hi - lo)) {
    const float q0 = __fmul_rn(x, rcp);
    const float r = __fmaf_rn(-d, q0, x);
    return __fmaf_rn(r, rcp, q0);
  }
  return __fdiv_rn(x, d);
}

// Four quotients at once with ONE decision for the group: when all four dividends are zero or lie in
// [2^-60, 2^60] and all divisors are fine, the three-instruction step runs for all of them; otherwise
// each goes through div_exact on its own.  (A zero dividend is safe in the fast step: q0 = +-0, the
// residual is 0, the result +-0 with the dividend's sign.)  One divergence region per float4 instead
// of one per element: about three instructions per element less in the normalisation kernels.
__device__ __forceinline__ bool div_fast_ok(float x) {
  const uint32_t ax = __float_as_uint(x) & 0x7fffffffu;
  const uint32_t lo = (127u - 60u) << 23, hi = (127u + 60u) << 23;
  return (ax - lo) <= (hi - lo) || ax == 0u;
}
__device__ __forceinline__ void div_exact4(float (&x)[4], const float (&d)[4], const float (&rcp)[4], const bool (&d_ok)[4]) {
  const bool fast = d_ok[0] && d_ok[1] && d_ok[2] && d_ok[3] && div_fast_ok(x[0]) && div_fast_ok(x[1]) && div_fast_ok(x[2]) &&
                    div_fast_ok(x[3]);
  if (fast) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float q0 = __fmul_rn(x[e], rcp[e]);
      const float r = __fmaf_rn(-d[e], q0, x[e]);
      x[e] = __fmaf_rn(r, rcp[e], q0);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = div_exact(x[e], d[e], rcp[e], d_ok[e]);
  }
}
// The same with one divisor for the four.
__device__ __forceinline__ void div_exact4(float (&x)[4], float d, float rcp, bool d_ok) {
  const float dd[4] = {d, d, d, d}, rr[4] = {rcp, rcp, rcp, rcp};
  const bool oo[4] = {d_ok, d_ok, d_ok, d_ok};
  div_exact4(x, dd, rr, oo);
}

// ---- functors -----------------------------------------------------------------------------------
// std::max(a, b) == (a < b) ? b : a and std::min(a, b) == (b < a) ? b : a.
__device__ __forceinline__ float std_max(float a, float b) { return (a < b) ? b : a; }
__device__ __forceinline__ float std_min(float a, float b) { return (b < a) ? b : a; }

template <int OP>
struct BinaryFn {
  __device__ __forceinline__ float operator()(float a, float b) const {
    if (OP == SB200_ADD) return __fadd_rn(a, b);
    if (OP == SB200_SUB) return __fsub_rn(a, b);
    if (OP == SB200_MUL) return __fmul_rn(a, b);
    if (OP == SB200_DIV) return __fdiv_rn(a, b);
    if (OP == SB200_POW) return pow_accurate(a, b);
    if (OP == SB200_MAX) return std_max(a, b);
    return std_min(a, b);
  }
};

template <int OP>
struct UnaryFn {
  // Which tile code path the elementwise kernel uses for this functor (see ew_vec_kernel): for the
  // double-precision exp the per-group guarded form schedules markedly better (6.6 vs 5.5 TB/s).
  static constexpr bool kGuardedTile = (OP == SB200_EXP);
  // (Exp alone streams at the DRAM limit with literal constants; loading them per thread only delays its start)
  static constexpr bool kUsesExpfConsts = false;
  __device__ __forceinline__ float eval(float x, const ExpfConsts& c) const { return expf_like_glibc(x, c); }
  __device__ __forceinline__ float operator()(float x) const {
    if (OP == SB200_ABS) return fabsf(x);
    if (OP == SB200_SQUARE) return __fmul_rn(x, x);
    if (OP == SB200_SQRT) return __fsqrt_rn(x);
    if (OP == SB200_LOG) return logf(x);   // within 1 ulp of glibc's logf on every input
    if (OP == SB200_EXP) return expf_like_glibc(x);
    if (OP == SB200_SIN) return sinf(x);
    if (OP == SB200_COS) return cosf(x);
    // (CUDA's tanf is 3 ulp from glibc's on 55,858 of the 2^32 inputs - above the bar - so Tan has its own
    // double-precision evaluation; the float sin / cos / asin / acos / atan are within 2 ulp of glibc's on every input)
    if (OP == SB200_TAN) return tan_accurate(x);
    if (OP == SB200_ASIN) return asinf(x);
    if (OP == SB200_ACOS) return acosf(x);
    if (OP == SB200_ATAN) return atanf(x);
    if (OP == SB200_FLOOR) return floorf(x);
    if (OP == SB200_CEIL) return ceilf(x);
    if (OP == SB200_NEG) return -x;
    return __fdiv_rn(1.f, x);
  }
};

// Activation types 1..8 (PReLU has its own channel-indexed kernel).
template <int TYPE>
struct ActivateFn {
  static constexpr bool kGuardedTile = (TYPE == SB200_SIGMOID || TYPE == SB200_TANH);
  static constexpr bool kUsesExpfConsts = (TYPE == SB200_SIGMOID);
  float slope;
  __device__ __forceinline__ float eval(float x, const ExpfConsts& c) const {
    return rcp_correct(__fadd_rn(1.f, expf_like_glibc(-x, c)));
  }
  __device__ __forceinline__ float operator()(float x) const {
    if (TYPE == SB200_RELU) return x > 0.f ? x : 0.f;
    if (TYPE == SB200_LEAKY) return x > 0.f ? x : __fmul_rn(slope, x);
    // 1 / (1 + exp(-x)): glibc's expf bit for bit, a float add, then the reciprocal (== IEEE 1.0f / y
    // for every normal result)
    if (TYPE == SB200_SIGMOID) return rcp_correct(__fadd_rn(1.f, expf_like_glibc(-x)));
    if (TYPE == SB200_SOFTPLUS) {
      // log1pf(expf(x)): expf as glibc computes it, then CUDA's float log1pf (documented to stay within 1 ulp of
      // the true value, as glibc's does: at most 2 ulp between the two, checked on every float input)
      return log1pf(expf_like_glibc(x));
    }
    if (TYPE == SB200_TANH) return tanh_accurate(x);
    if (TYPE == SB200_RELU6) return x < 0.f ? 0.f : (x > 6.f ? 6.f : x);
    if (TYPE == SB200_HARDSWISH)
      return x < -3.f ? 0.f : (x > 3.f ? x : __fdiv_rn(__fmul_rn(x, __fadd_rn(x, 3.f)), 6.f));
    // Gelu: 0.5f * x * (1 + erf(0.707107f * x)), left to right
    float t = __fmul_rn(0.707107f, x);
    float e = erf_accurate(t);
    return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.f, e));
  }
};

struct ScaleBiasFn {   // two roundings: (x * s) then (+ b)
  __device__ __forceinline__ float operator()(float x, float s, float b) const {
    return __fadd_rn(__fmul_rn(x, s), b);
  }
};
struct ScaleFn {
  __device__ __forceinline__ float operator()(float x, float s, float) const { return __fmul_rn(x, s); }
};
struct BiasFn {
  __device__ __forceinline__ float operator()(float x, float, float b) const { return __fadd_rn(x, b); }
};
struct BatchNormFn {   // (x - mean*sf) / sqrt(|var*sf| + eps), every step one IEEE float operation
  float sf, eps;
  __device__ __forceinline__ float operator()(float x, float mean, float var) const {
    const float m = __fmul_rn(mean, sf);
    const float d = __fsqrt_rn(__fadd_rn(fabsf(__fmul_rn(var, sf)), eps));
    return __fdiv_rn(__fsub_rn(x, m), d);
  }
};
struct PReluFn {       // x > 0 ? x : x * slope[c]
  __device__ __forceinline__ float operator()(float x, float s, float) const {
    return x > 0.f ? x : __fmul_rn(x, s);
  }
};

}  // namespace sb200
