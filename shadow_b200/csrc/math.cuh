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
// CUDA's float functions document 1-4 ulp of error against the correctly rounded result; added to
// glibc's own error that can exceed the 2 ulp parity budget.  Where it matters the function is
// evaluated in double precision on a reduced argument and rounded once to float, which is
// correctly rounded except for rare double-rounding cases (so <= 1 ulp from glibc).

// e^x for a float-range x, in double: k = rint(x*log2(e)), r = x - k*ln2 in two steps
// (|r| <= 0.347), degree-9 Taylor polynomial by Horner (relative error < 1e-11), scaled by 2^k.
// exp_accurate() clamps the argument (overflow above 88.72 -> inf, underflow below -103.97 -> 0);
// denormal float results come out right because the scaling happens in double and the single
// conversion to float rounds into the denormal range.
__device__ __forceinline__ double exp_f64_core(double x) {
  const double kLog2e = 1.4426950408889634074, kLn2Hi = 6.93147180369123816490e-01,
               kLn2Lo = 1.90821492927058770002e-10;
  double k = rint(x * kLog2e);
  double r = fma(-k, kLn2Hi, x);
  r = fma(-k, kLn2Lo, r);
  double p = 2.75573192239858906526e-06;           // 1/9!
  p = fma(p, r, 2.48015873015873015873e-05);       // 1/8!
  p = fma(p, r, 1.98412698412698412698e-04);       // 1/7!
  p = fma(p, r, 1.38888888888888888889e-03);       // 1/6!
  p = fma(p, r, 8.33333333333333333333e-03);       // 1/5!
  p = fma(p, r, 4.16666666666666666667e-02);       // 1/4!
  p = fma(p, r, 1.66666666666666666667e-01);       // 1/3!
  p = fma(p, r, 0.5);
  p = fma(p, r, 1.0);
  p = fma(p, r, 1.0);
  // scale by 2^k through the exponent field: p is in [0.70, 1.42] and the caller clamps x so that
  // k stays in [-152, 130], far inside the double exponent range.
  int ki = static_cast<int>(k);
  return __hiloint2double(__double2hiint(p) + (ki << 20), __double2loint(p));
}

__device__ __forceinline__ float exp_accurate(float x) {
  if (!(x == x)) return x + x;                       // NaN
  double xd = static_cast<double>(x);
  if (xd > 90.0) return CUDART_INF_F;                // float overflow threshold is 88.7228
  if (xd < -105.0) return 0.f;                       // below the smallest denormal (-103.97)
  return static_cast<float>(exp_f64_core(xd));
}

// tanh(x) = (e^{2x} - 1) / (e^{2x} + 1) in double; for |x| < 2^-12 the float result is x itself
// (tanh x = x - x^3/3, the correction is below half an ulp).
__device__ __forceinline__ float tanh_accurate(float x) {
  float ax = fabsf(x);
  if (!(x == x)) return x + x;
  if (ax < 2.44140625e-4f) return x;
  if (ax > 10.f) return copysignf(1.f, x);           // 1 - 2e^{-20} rounds to 1 in float
  double e = exp_f64_core(2.0 * static_cast<double>(ax));   // e^{2|x|} in [1, 4.9e8]
  double t = (e - 1.0) / (e + 1.0);
  return copysignf(static_cast<float>(t), x);
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
  __device__ __forceinline__ float operator()(float x) const {
    if (OP == SB200_ABS) return fabsf(x);
    if (OP == SB200_SQUARE) return __fmul_rn(x, x);
    if (OP == SB200_SQRT) return __fsqrt_rn(x);
    if (OP == SB200_LOG) return static_cast<float>(log(static_cast<double>(x)));
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
  float slope;
  __device__ __forceinline__ float operator()(float x) const {
    if (TYPE == SB200_RELU) return x > 0.f ? x : 0.f;
    if (TYPE == SB200_LEAKY) return x > 0.f ? x : __fmul_rn(slope, x);
    if (TYPE == SB200_SIGMOID) return __fdiv_rn(1.f, __fadd_rn(1.f, exp_accurate(-x)));
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
struct PReluFn {       // x > 0 ? x : x * slope[c]
  __device__ __forceinline__ float operator()(float x, float s, float) const {
    return x > 0.f ? x : __fmul_rn(x, s);
  }
};

}  // namespace sb200
