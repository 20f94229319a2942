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
// The parity bar is 2 ulp against glibc's float functions.  Measured over ALL 2^32 float inputs
// on B200 against glibc 2.39: CUDA's logf is within 1 ulp of glibc's everywhere (used as is);
// CUDA's expf reaches 2 ulp and tanhf 3 ulp, and the reference's Sigmoid composition
// 1/(1+expf(-x)) magnifies a 1-ulp difference in expf up to 4 ulp.  So e^x is computed here in
// double precision and rounded ONCE to float (correctly rounded except for rare double-rounding
// ties; at most 1 ulp from glibc on every input), and Sigmoid / Tanh / SoftPlus build on it.

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
// conversion instruction: the conversion unit is the scarce pipe of these kernels); the reduction
// runs in double with ln2/16 split so that k*hi is exact.
__device__ __forceinline__ double exp_core(float x) {
  const double xd = static_cast<double>(x);
  const double kRound = 6755399441055744.0;                 // 1.5 * 2^52: adding it rounds to an integer
  const double t = fma(xd, 23.083120654223414, kRound);     // x * 16/ln2, integer part in the low word
  const int ki = __double2loint(t);                         // k as a signed integer (|k| < 2^12)
  const double kd = t - kRound;
  double r = fma(kd, -0.043321698773070239, xd);
  r = fma(kd, -1.1926343307941173e-11, r);
  double p = fma(r, 4.16666666666666666667e-02, 1.66666666666666666667e-01);
  p = fma(p, r, 0.5);
  p = fma(p, r, 1.0);
  p = fma(p, r, 1.0);
  const double v = p * __ldg(&kExp2Sixteenths[ki & 15]);  // in [1, 2.05)
  // scale by 2^(k>>4) through the exponent field; k>>4 stays within [-152, 130]
  return __hiloint2double(__double2hiint(v) + ((ki >> 4) << 20), __double2loint(v));
}

__device__ __forceinline__ float exp_accurate(float x) {
  // Branch-free: clamp into the range where exp_core is valid.  e^-105 converts to 0 and e^90 to
  // +inf, which are the float results for everything beyond the clamp; denormal results come out
  // right because the scaling is done in double and the single conversion to float rounds into
  // the denormal range.  fminf/fmaxf drop a NaN, so it is put back at the end.
  const float xc = fminf(fmaxf(x, -105.f), 90.f);
  const float y = static_cast<float>(exp_core(xc));
  return (x == x) ? y : x;
}

// 1/d for a double d in [2, 1e9], relative error ~1e-14: hardware float reciprocal as the seed,
// one Newton step in double (a full double division costs an order of magnitude more).  The seed
// goes double -> float -> double by bit manipulation (truncation is fine for a seed), because
// each cvt instruction costs a slot of the conversion unit, the busiest pipe of the tanh kernel.
__device__ __forceinline__ double rcp_newton(double d) {
  const unsigned hi = static_cast<unsigned>(__double2hiint(d)), lo = static_cast<unsigned>(__double2loint(d));
  const float df = __uint_as_float(((hi - 0x38000000u) << 3) | (lo >> 29));   // d truncated to float
  float seed;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(seed) : "f"(df));
  const unsigned sb = __float_as_uint(seed);                                   // positive, normal
  const double r0 = __hiloint2double(static_cast<int>((sb >> 3) + 0x38000000u), static_cast<int>(sb << 29));
  return fma(r0, fma(-d, r0, 1.0), r0);
}

// Correctly rounded 1/y for a float y >= 1 (or +inf): hardware seed (within 1 ulp) and one fma
// correction, r1 = r0 + r0*(1 - y*r0).  Bit-identical to __frcp_rn on this domain (checked through
// Sigmoid over all 2^32 inputs) at a fraction of its cost.  y = inf gives r0 = 0 and a NaN residual.
__device__ __forceinline__ float rcp_correct(float y) {
  float r0;
  asm("rcp.approx.f32 %0, %1;" : "=f"(r0) : "f"(y));
  const float e = fmaf(-y, r0, 1.0f);
  const float r1 = fmaf(r0, e, r0);
  return (e == e) ? r1 : r0;
}

// tanh(x) = 1 - 2/(e^{2|x|} + 1) in double, rounded once; for |x| < 2^-12 the float result is x
// itself (tanh x = x - x^3/3 and the correction is below half an ulp).
__device__ __forceinline__ float tanh_accurate(float x) {
  const float ax = fminf(fabsf(x), 10.f);         // beyond 10, 1 - 2e^{-2|x|} rounds to 1 (also for inf)
  const double e = exp_core(ax + ax);             // e^{2|x|} in [1, 4.9e8]
  const double t = fma(-2.0, rcp_newton(e + 1.0), 1.0);
  float y = copysignf(static_cast<float>(t), x);
  y = (fabsf(x) < 2.44140625e-4f) ? x : y;        // tiny arguments (and +-0) return x itself
  return (x == x) ? y : x;                        // NaN
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
    if (OP == SB200_POW) return static_cast<float>(pow(static_cast<double>(a), static_cast<double>(b)));
    if (OP == SB200_MAX) return std_max(a, b);
    return std_min(a, b);
  }
};

template <int OP>
struct UnaryFn {
  // Which tile code path the elementwise kernel uses for this functor (see ew_vec_kernel): for the
  // double-precision exp the per-group guarded form schedules markedly better (6.6 vs 5.5 TB/s).
  static constexpr bool kGuardedTile = (OP == SB200_EXP);
  __device__ __forceinline__ float operator()(float x) const {
    if (OP == SB200_ABS) return fabsf(x);
    if (OP == SB200_SQUARE) return __fmul_rn(x, x);
    if (OP == SB200_SQRT) return __fsqrt_rn(x);
    if (OP == SB200_LOG) return logf(x);   // within 1 ulp of glibc's logf on every input
    if (OP == SB200_EXP) return exp_accurate(x);
    if (OP == SB200_SIN) return static_cast<float>(sin(static_cast<double>(x)));
    if (OP == SB200_COS) return static_cast<float>(cos(static_cast<double>(x)));
    if (OP == SB200_TAN) return static_cast<float>(tan(static_cast<double>(x)));
    if (OP == SB200_ASIN) return static_cast<float>(asin(static_cast<double>(x)));
    if (OP == SB200_ACOS) return static_cast<float>(acos(static_cast<double>(x)));
    if (OP == SB200_ATAN) return static_cast<float>(atan(static_cast<double>(x)));
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
  float slope;
  __device__ __forceinline__ float operator()(float x) const {
    if (TYPE == SB200_RELU) return x > 0.f ? x : 0.f;
    if (TYPE == SB200_LEAKY) return x > 0.f ? x : __fmul_rn(slope, x);
    // 1 / (1 + exp(-x)): float add, then the correctly rounded reciprocal (== IEEE 1.0f / y)
    if (TYPE == SB200_SIGMOID) return rcp_correct(__fadd_rn(1.f, exp_accurate(-x)));
    if (TYPE == SB200_SOFTPLUS) {
      // log1p(exp(x)) with both steps in double; exp(x) first rounded to float like the reference.
      float e = exp_accurate(x);
      return static_cast<float>(log1p(static_cast<double>(e)));
    }
    if (TYPE == SB200_TANH) return tanh_accurate(x);
    if (TYPE == SB200_RELU6) return x < 0.f ? 0.f : (x > 6.f ? 6.f : x);
    if (TYPE == SB200_HARDSWISH)
      return x < -3.f ? 0.f : (x > 3.f ? x : __fdiv_rn(__fmul_rn(x, __fadd_rn(x, 3.f)), 6.f));
    // Gelu: 0.5f * x * (1 + erf(0.707107f * x)), left to right
    float t = __fmul_rn(0.707107f, x);
    float e = static_cast<float>(erf(static_cast<double>(t)));
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
