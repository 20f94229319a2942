// Eltwise (N same-shape inputs folded by Prod / Sum-with-coefficients / Max / Min) and Axpy
// (out = y + alpha[n,c] * x).  The reference runs Eltwise as N-1 separate passes over the output
// (Blas::Mul / Max / Min in place) or N Saxpy passes after a Set(0); here one launch reads every
// input once and writes the output once: algorithmic bytes 4*(N+1) per element instead of
// roughly 12*(N-1).  Arithmetic follows the reference's order exactly: left-to-right folding,
// Sum as ((0 + c0*x0) + c1*x1) + ... with the multiply and the add rounded separately.
#include "common.cuh"
#include "math.cuh"

namespace sb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 2;
constexpr int kMaxInputs = 8;   // per launch; longer lists are chained through the output

enum { kEltProd = 0, kEltSum = 1, kEltMax = 2, kEltMin = 3 };

struct EltArgs {
  const float* in[kMaxInputs];
  float coeff[kMaxInputs];
  int n;
};

template <int OP>
__device__ __forceinline__ float fold(float acc, float x, float c) {
  if (OP == kEltProd) return __fmul_rn(acc, x);
  if (OP == kEltSum) return __fadd_rn(acc, __fmul_rn(c, x));
  if (OP == kEltMax) return std_max(acc, x);
  return std_min(acc, x);
}

// CONTINUE: the running value starts from what is already in y (a later launch of a long list).
template <int OP, bool CONTINUE, bool VEC>
__global__ void __launch_bounds__(kThreads)
eltwise_kernel(const __grid_constant__ EltArgs a, float* y, int64_t n) {
  constexpr int W = VEC ? 4 : 1;
  const int64_t units = VEC ? (n >> 2) : n;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kThreads * kUnroll + threadIdx.x;
  if (VEC && blockIdx.x == 0 && threadIdx.x < (n & 3)) {   // the last n % 4 elements, scalar
    const int64_t i = (units << 2) + threadIdx.x;
    float acc = CONTINUE ? y[i] : (OP == kEltSum ? 0.f : a.in[0][i]);
#pragma unroll
    for (int k = 0; k < kMaxInputs; ++k)
      if (k < a.n && (CONTINUE || OP == kEltSum || k > 0)) acc = fold<OP>(acc, a.in[k][i], a.coeff[k]);
    y[i] = acc;
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t v = base + static_cast<int64_t>(u) * kThreads;
    if (v >= units) continue;
    float x[kMaxInputs][W];
#pragma unroll
    for (int k = 0; k < kMaxInputs; ++k) {
      if (k < a.n) {
        if (VEC) {
          const float4 q = ld_stream(reinterpret_cast<const float4*>(a.in[k]) + v);
          x[k][0] = q.x; x[k][W > 1 ? 1 : 0] = q.y; x[k][W > 2 ? 2 : 0] = q.z; x[k][W > 3 ? 3 : 0] = q.w;
        } else {
          x[k][0] = ld_stream(a.in[k] + v);
        }
      }
    }
    float acc[W];
    if (CONTINUE) {
      if (VEC) {
        const float4 q = *(reinterpret_cast<const float4*>(y) + v);
        acc[0] = q.x; acc[W > 1 ? 1 : 0] = q.y; acc[W > 2 ? 2 : 0] = q.z; acc[W > 3 ? 3 : 0] = q.w;
      } else {
        acc[0] = y[v];
      }
    } else {
#pragma unroll
      for (int e = 0; e < W; ++e) acc[e] = (OP == kEltSum) ? 0.f : x[0][e];
    }
#pragma unroll
    for (int k = 0; k < kMaxInputs; ++k) {
      if (k < a.n && (CONTINUE || OP == kEltSum || k > 0)) {
#pragma unroll
        for (int e = 0; e < W; ++e) acc[e] = fold<OP>(acc[e], x[k][e], a.coeff[k]);
      }
    }
    if (VEC) st_stream(reinterpret_cast<float4*>(y) + v, make_float4(acc[0], acc[W > 1 ? 1 : 0], acc[W > 2 ? 2 : 0], acc[W > 3 ? 3 : 0]));
    else st_stream(y + v, acc[0]);
  }
}

template <int OP>
int launch_eltwise(const float* const* inputs, int n_inputs, const float* coeff, float* y, int64_t n,
                   cudaStream_t s) {
  bool vec = aligned16(y);
  for (int k = 0; k < n_inputs; ++k) vec = vec && aligned16(inputs[k]);
  const int64_t units = vec ? (n >> 2) : n;
  const unsigned grid = tile_grid(units, kThreads * kUnroll);
  for (int first = 0; first < n_inputs; first += kMaxInputs) {
    EltArgs a;
    a.n = (n_inputs - first < kMaxInputs) ? n_inputs - first : kMaxInputs;
    for (int k = 0; k < kMaxInputs; ++k) {
      a.in[k] = k < a.n ? inputs[first + k] : nullptr;
      a.coeff[k] = (k < a.n && coeff != nullptr) ? coeff[first + k] : 1.f;
    }
    if (first == 0) {
      if (vec) eltwise_kernel<OP, false, true><<<grid, kThreads, 0, s>>>(a, y, n);
      else eltwise_kernel<OP, false, false><<<grid, kThreads, 0, s>>>(a, y, n);
    } else {
      if (vec) eltwise_kernel<OP, true, true><<<grid, kThreads, 0, s>>>(a, y, n);
      else eltwise_kernel<OP, true, false><<<grid, kThreads, 0, s>>>(a, y, n);
    }
    int rc = after_launch("sb200_eltwise");
    if (rc != SB200_OK) return rc;
  }
  return SB200_OK;
}

// out[i] = y[i] + alpha[i / inner] * x[i]
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
axpy_kernel(const float* __restrict__ alpha, const float* x, const float* y, float* out, int64_t n, int64_t inner,
            FastDiv32 div_inner) {
  const int64_t units = VEC ? (n >> 2) : n;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kThreads * kUnroll + threadIdx.x;
  if (VEC && blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const int64_t i = (units << 2) + threadIdx.x;
    out[i] = __fadd_rn(y[i], __fmul_rn(__ldg(alpha + i / inner), x[i]));
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t v = base + static_cast<int64_t>(u) * kThreads;
    if (v >= units) continue;
    if (VEC) {
      const float4 xv = ld_stream(reinterpret_cast<const float4*>(x) + v);
      const float4 yv = ld_stream(reinterpret_cast<const float4*>(y) + v);
      const int64_t i = v << 2;
      int64_t row, r;
      if (n < (1ll << 32)) {
        uint32_t q, rem;
        div_inner.divmod(static_cast<uint32_t>(i), q, rem);
        row = q, r = rem;
      } else {
        row = i / inner, r = i - row * inner;
      }
      const float xs[4] = {xv.x, xv.y, xv.z, xv.w}, ys[4] = {yv.x, yv.y, yv.z, yv.w};
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o[e] = __fadd_rn(ys[e], __fmul_rn(__ldg(alpha + row), xs[e]));
        if (++r == inner) { r = 0; ++row; }
      }
      // the walk may step one row past the end after the very last element; alpha is read only
      // for e < 4 elements that exist (n % 4 == 0 here), so no read goes out of bounds
      st_stream(reinterpret_cast<float4*>(out) + v, make_float4(o[0], o[1], o[2], o[3]));
    } else {
      out[v] = __fadd_rn(y[v], __fmul_rn(__ldg(alpha + v / inner), x[v]));
    }
  }
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" {

int sb200_eltwise(const float* const* inputs, int n_inputs, const float* coeff, float* y, int64_t n,
                  int operation, void* stream) {
  if (inputs == nullptr || n_inputs < 2 || n_inputs > 1024 || n < 0 || operation < kEltProd || operation > kEltMin)
    return SB200_ERR_BAD_ARGUMENT;
  if (coeff != nullptr && operation != kEltSum) return SB200_ERR_BAD_ARGUMENT;
  if (n == 0) return SB200_OK;
  if (y == nullptr || (reinterpret_cast<uintptr_t>(y) & 3u)) return SB200_ERR_BAD_ARGUMENT;
  for (int k = 0; k < n_inputs; ++k)
    if (inputs[k] == nullptr || (reinterpret_cast<uintptr_t>(inputs[k]) & 3u)) return SB200_ERR_BAD_ARGUMENT;
  // two inputs folded by Prod / Max / Min are exactly Binary Mul / Max / Min (same operand order)
  if (n_inputs == 2 && operation != kEltSum)
    return sb200_binary(inputs[0], inputs[1], y, n, operation == kEltProd ? SB200_MUL : (operation == kEltMax ? SB200_MAX : SB200_MIN),
                        stream);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (operation) {
    case kEltProd: return launch_eltwise<kEltProd>(inputs, n_inputs, coeff, y, n, s);
    case kEltSum: return launch_eltwise<kEltSum>(inputs, n_inputs, coeff, y, n, s);
    case kEltMax: return launch_eltwise<kEltMax>(inputs, n_inputs, coeff, y, n, s);
    default: return launch_eltwise<kEltMin>(inputs, n_inputs, coeff, y, n, s);
  }
}

int sb200_axpy(const float* alpha, const float* x, const float* y, float* out, int64_t outer, int64_t inner,
               void* stream) {
  if (outer < 0 || inner < 1) return SB200_ERR_BAD_ARGUMENT;
  const int64_t n = outer * inner;
  if (n == 0) return SB200_OK;
  if (alpha == nullptr || x == nullptr || y == nullptr || out == nullptr) return SB200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(alpha)) & 3u)
    return SB200_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec = aligned16(x) && aligned16(y) && aligned16(out) && (n % 4 == 0);
  const FastDiv32 div(inner < (1ll << 32) ? static_cast<uint32_t>(inner) : 1u);
  if (vec) axpy_kernel<true><<<tile_grid(n >> 2, kThreads * kUnroll), kThreads, 0, s>>>(alpha, x, y, out, n, inner, div);
  else axpy_kernel<false><<<tile_grid(n, kThreads * kUnroll), kThreads, 0, s>>>(alpha, x, y, out, n, inner, div);
  return after_launch("sb200_axpy");
}

}  // extern "C"
