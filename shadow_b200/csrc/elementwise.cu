// Flat elementwise kernels: fill, unary, activate, binary (tensor,tensor) and (tensor,scalar), and
// the channel-indexed family (Scale / Bias / ScaleBias / PReLU).
//
// All of them are HBM-bound streams: 4 B read and 4 B written per element (12 B for the
// two-input binary).  One kernel shape serves them all:
//   * 128-bit accesses: a thread owns float4 groups; UNROLL independent groups are loaded before
//     any is used, so each thread keeps UNROLL*16 B (per input) in flight;
//   * a block owns ONE tile of THREADS*UNROLL consecutive float4 (16 KB per input) and the grid has
//     one block per tile.  Measured on B200, this beats a persistent grid-stride loop of
//     148*k blocks by 5-15 % (6.6 TB/s against 5.7-6.3 TB/s on a 512 MB negate): the hardware block
//     scheduler keeps every SM busy to the end and the access stream is less regular, while blocks
//     that stride in lock step over the tensor keep colliding on the same DRAM channels;
//   * pointers that are not 16-byte aligned (a sub-buffer at an odd element offset) are handled by
//     peeling `head` scalar elements when every pointer has the same misalignment, otherwise by
//     a scalar kernel; the last n%4 elements are scalar as well.  Head and tail are done by
//     block 0 inside the same launch.
#include "common.cuh"
#include "math.cuh"

namespace sb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

// Functors may ask for the guarded tile form through a static member kGuardedTile.
template <typename F, typename = void>
struct GuardedTileTrait { static constexpr bool value = false; };
template <typename F>
struct GuardedTileTrait<F, decltype(void(F::kGuardedTile))> { static constexpr bool value = F::kGuardedTile; };
template <typename F>
__host__ __device__ constexpr bool guarded_tile() { return GuardedTileTrait<F>::value; }

// Functors built on expf_like_glibc ask (static member kUsesExpfConsts) for its constants to be loaded
// once per thread and handed to eval(x, consts).
template <typename F, typename = void>
struct ExpfConstsTrait { static constexpr bool value = false; };
template <typename F>
struct ExpfConstsTrait<F, decltype(void(F::kUsesExpfConsts))> { static constexpr bool value = F::kUsesExpfConsts; };

// Calls f with as many operands as the kernel has inputs.
template <int NIN, typename F>
__device__ __forceinline__ float apply(const F& f, float a, float b) {
  if constexpr (NIN == 0) return f();
  else if constexpr (NIN == 1) return f(a);
  else return f(a, b);
}
template <int NIN, typename F>
__device__ __forceinline__ float4 apply4(const F& f, const float4& a, const float4& b) {
  return make_float4(apply<NIN>(f, a.x, b.x), apply<NIN>(f, a.y, b.y), apply<NIN>(f, a.z, b.z),
                     apply<NIN>(f, a.w, b.w));
}

// y = f()            (fill)
// y = f(x)           (unary / activate / binary-scalar)
// y = f(a, b)        (binary)
template <int NIN, typename F>
__global__ void __launch_bounds__(kThreads)
ew_vec_kernel(const float* a, const float* b, float* y, int64_t n, int head, F f) {
  // a/b may alias y (in-place): a group's loads precede its stores in the owning thread and no
  // other thread touches that group, so no __restrict__ is claimed.
  const int64_t nvec = (n - head) >> 2;
  const int tail = static_cast<int>(n - head - (nvec << 2));
  if (blockIdx.x == 0) {
    // scalar edges: elements [0, head) and the last `tail` ones
    int t = threadIdx.x;
    int64_t idx = -1;
    if (t < head) idx = t;
    else if (t >= 32 && t < 32 + tail) idx = head + (nvec << 2) + (t - 32);
    if (idx >= 0) {
      y[idx] = apply<NIN>(f, NIN >= 1 ? a[idx] : 0.f, NIN >= 2 ? b[idx] : 0.f);
    }
  }
  const float4* a4 = reinterpret_cast<const float4*>(a + head);
  const float4* b4 = reinterpret_cast<const float4*>(b + head);
  float4* y4 = reinterpret_cast<float4*>(y + head);
  constexpr int64_t kTile = static_cast<int64_t>(kThreads) * kUnroll;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
  float4 va[kUnroll] = {}, vb[kUnroll] = {};
  const int64_t first = base + threadIdx.x;
  if (!guarded_tile<F>() && base + kTile <= nvec) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (NIN >= 1) va[u] = ld_stream(a4 + first + u * kThreads);
      if (NIN >= 2) vb[u] = ld_stream(b4 + first + u * kThreads);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) st_stream(y4 + first + u * kThreads, apply4<NIN>(f, va[u], vb[u]));
  } else {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t v = first + u * kThreads;
      if (v < nvec) {
        if (NIN >= 1) va[u] = ld_stream(a4 + v);
        if (NIN >= 2) vb[u] = ld_stream(b4 + v);
      }
    }
    if constexpr (ExpfConstsTrait<F>::value) {
      const ExpfConsts c = load_expf_consts();
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t v = first + u * kThreads;
        if (v < nvec)
          st_stream(y4 + v, make_float4(f.eval(va[u].x, c), f.eval(va[u].y, c), f.eval(va[u].z, c), f.eval(va[u].w, c)));
      }
    } else {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t v = first + u * kThreads;
        if (v < nvec) st_stream(y4 + v, apply4<NIN>(f, va[u], vb[u]));
      }
    }
  }
}

// Scalar variant for pointers with different misalignments.
template <int NIN, typename F>
__global__ void __launch_bounds__(kThreads)
ew_scalar_kernel(const float* a, const float* b, float* y, int64_t n, F f) {
  constexpr int64_t kTile = static_cast<int64_t>(kThreads) * kUnroll;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
  float va[kUnroll] = {}, vb[kUnroll] = {};
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + threadIdx.x + u * kThreads;
    if (i < n) {
      if (NIN >= 1) va[u] = a[i];
      if (NIN >= 2) vb[u] = b[i];
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + threadIdx.x + u * kThreads;
    if (i < n) y[i] = apply<NIN>(f, va[u], vb[u]);
  }
}

// Number of leading scalar elements that brings `p` to a 16-byte boundary (p is 4-byte aligned).
inline int head_of(const void* p) {
  return static_cast<int>(((16u - (reinterpret_cast<uintptr_t>(p) & 15u)) & 15u) >> 2);
}

template <int NIN, typename F>
int launch_ew(const float* a, const float* b, float* y, int64_t n, F f, cudaStream_t stream,
              const char* what) {
  if (n == 0) return SB200_OK;
  if ((reinterpret_cast<uintptr_t>(y) & 3u) || (NIN >= 1 && (reinterpret_cast<uintptr_t>(a) & 3u)) ||
      (NIN >= 2 && (reinterpret_cast<uintptr_t>(b) & 3u)))
    return SB200_ERR_BAD_ARGUMENT;
  int head = head_of(y);
  bool same = (NIN < 1 || head_of(a) == head) && (NIN < 2 || head_of(b) == head);
  if (head > n) head = static_cast<int>(n);
  if (same) {
    const int64_t nvec = (n - head) >> 2;
    ew_vec_kernel<NIN, F><<<tile_grid(nvec, kThreads * kUnroll), kThreads, 0, stream>>>(a, b, y, n, head, f);
  } else {
    ew_scalar_kernel<NIN, F><<<tile_grid(n, kThreads * kUnroll), kThreads, 0, stream>>>(a, b, y, n, f);
  }
  return after_launch(what);
}

struct FillFn {
  float v;
  __device__ __forceinline__ float operator()() const { return v; }
};

template <int OP>
struct BinaryScalarFn {
  float alpha;
  __device__ __forceinline__ float operator()(float a) const { return BinaryFn<OP>()(a, alpha); }
};

// ---- channel-indexed family --------------------------------------------------------------------
// y[i] = f(x[i], p[c], q[c]) with c = (i / inner) % channels.  A thread owns 4 consecutive elements:
// it decodes (c, position inside the channel run) once and then walks, so any `inner` (also
// inner < 4 or not a multiple of 4) keeps 128-bit accesses on x and y.  p/q are small tables
// that stay in L1/L2 (read-only path).
template <bool HAS_P, bool HAS_Q, typename F>
__global__ void __launch_bounds__(kThreads)
chan_vec_kernel(const float* x, float* y, int64_t n, int head, const float* __restrict__ p,
                const float* __restrict__ q, int64_t inner, int64_t channels, int shared,
                FastDiv32 div_inner, FastDiv32 div_chan, F f) {
  const int64_t nvec = (n - head) >> 2;
  const int tail = static_cast<int>(n - head - (nvec << 2));
  if (blockIdx.x == 0) {
    int t = threadIdx.x;
    int64_t idx = -1;
    if (t < head) idx = t;
    else if (t >= 32 && t < 32 + tail) idx = head + (nvec << 2) + (t - 32);
    if (idx >= 0) {
      int64_t c = shared ? 0 : (idx / inner) % channels;
      y[idx] = f(x[idx], HAS_P ? __ldg(p + c) : 0.f, HAS_Q ? __ldg(q + c) : 0.f);
    }
  }
  const float4* x4 = reinterpret_cast<const float4*>(x + head);
  float4* y4 = reinterpret_cast<float4*>(y + head);
  const bool uniform4 = (head == 0) && ((inner & 3) == 0);
  constexpr int64_t kTile = static_cast<int64_t>(kThreads) * kUnroll;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
  float4 vx[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t v = base + threadIdx.x + u * kThreads;
    if (v < nvec) vx[u] = ld_stream(x4 + v);
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t v = base + threadIdx.x + u * kThreads;
    if (v < nvec) {
      const int64_t i = head + (v << 2);
      int64_t c, r;
      if (n < (1ll << 32) && channels < (1ll << 32)) {  // exact mul-hi division, host-computed constants
        uint32_t rw, rr, qq, cc;
        div_inner.divmod(static_cast<uint32_t>(i), rw, rr);
        div_chan.divmod(rw, qq, cc);
        r = rr, c = cc;
      } else {
        const int64_t row = i / inner;
        r = i - row * inner;
        c = row % channels;
      }
      if (uniform4) {   // inner % 4 == 0 and no head: the float4 lies inside one channel run
        const int64_t cc = shared ? 0 : c;
        const float ps = HAS_P ? __ldg(p + cc) : 0.f, qs = HAS_Q ? __ldg(q + cc) : 0.f;
        st_stream(y4 + v, make_float4(f(vx[u].x, ps, qs), f(vx[u].y, ps, qs), f(vx[u].z, ps, qs), f(vx[u].w, ps, qs)));
        continue;
      }
      float xs[4] = {vx[u].x, vx[u].y, vx[u].z, vx[u].w};
      float ys[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t cc = shared ? 0 : c;
        ys[j] = f(xs[j], HAS_P ? __ldg(p + cc) : 0.f, HAS_Q ? __ldg(q + cc) : 0.f);
        if (++r == inner) {
          r = 0;
          if (++c == channels) c = 0;
        }
      }
      st_stream(y4 + v, make_float4(ys[0], ys[1], ys[2], ys[3]));
    }
  }
}

template <bool HAS_P, bool HAS_Q, typename F>
__global__ void __launch_bounds__(kThreads)
chan_scalar_kernel(const float* x, float* y, int64_t n, const float* __restrict__ p,
                   const float* __restrict__ q, int64_t inner, int64_t channels, int shared, F f) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (i < n) {
    int64_t c = shared ? 0 : (i / inner) % channels;
    y[i] = f(x[i], HAS_P ? __ldg(p + c) : 0.f, HAS_Q ? __ldg(q + c) : 0.f);
  }
}

template <bool HAS_P, bool HAS_Q, typename F>
int launch_chan(const float* x, float* y, int64_t n, const float* p, const float* q, int64_t inner,
                int64_t channels, int shared, F f, cudaStream_t stream, const char* what) {
  if (n == 0) return SB200_OK;
  if ((reinterpret_cast<uintptr_t>(x) & 3u) || (reinterpret_cast<uintptr_t>(y) & 3u))
    return SB200_ERR_BAD_ARGUMENT;
  int head = head_of(y);
  if (head > n) head = static_cast<int>(n);
  if (head_of(x) == head_of(y)) {
    const int64_t nvec = (n - head) >> 2;
    chan_vec_kernel<HAS_P, HAS_Q, F><<<tile_grid(nvec, kThreads * kUnroll), kThreads, 0, stream>>>(
        x, y, n, head, p, q, inner, channels, shared,
        FastDiv32(inner < (1ll << 32) ? static_cast<uint32_t>(inner) : 1u),
        FastDiv32(channels < (1ll << 32) ? static_cast<uint32_t>(channels) : 1u), f);
  } else {
    chan_scalar_kernel<HAS_P, HAS_Q, F><<<tile_grid(n, kThreads), kThreads, 0, stream>>>(
        x, y, n, p, q, inner, channels, shared, f);
  }
  return after_launch(what);
}

template <int OP>
int unary_op(const float* x, float* y, int64_t n, cudaStream_t s) {
  return launch_ew<1>(x, nullptr, y, n, UnaryFn<OP>(), s, "sb200_unary");
}
template <int T>
int activate_op(const float* x, float* y, int64_t n, float slope, cudaStream_t s) {
  return launch_ew<1>(x, nullptr, y, n, ActivateFn<T>{slope}, s, "sb200_activate");
}
template <int OP>
int binary_scalar_op(const float* a, float alpha, float* y, int64_t n, cudaStream_t s) {
  return launch_ew<1>(a, nullptr, y, n, BinaryScalarFn<OP>{alpha}, s, "sb200_binary_scalar");
}
template <int OP>
int binary_op(const float* a, const float* b, float* y, int64_t n, cudaStream_t s) {
  return launch_ew<2>(a, b, y, n, BinaryFn<OP>(), s, "sb200_binary");
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" {

int sb200_fill(float* y, int64_t n, float val, void* stream) {
  if (n < 0 || (n > 0 && y == nullptr)) return SB200_ERR_BAD_ARGUMENT;
  return launch_ew<0>(nullptr, nullptr, y, n, FillFn{val}, static_cast<cudaStream_t>(stream), "sb200_fill");
}

int sb200_unary(const float* x, float* y, int64_t n, int operation, void* stream) {
  if (n < 0 || (n > 0 && (x == nullptr || y == nullptr))) return SB200_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (operation) {
    case SB200_ABS: return unary_op<SB200_ABS>(x, y, n, s);
    case SB200_SQUARE: return unary_op<SB200_SQUARE>(x, y, n, s);
    case SB200_SQRT: return unary_op<SB200_SQRT>(x, y, n, s);
    case SB200_LOG: return unary_op<SB200_LOG>(x, y, n, s);
    case SB200_EXP: return unary_op<SB200_EXP>(x, y, n, s);
    case SB200_SIN: return unary_op<SB200_SIN>(x, y, n, s);
    case SB200_COS: return unary_op<SB200_COS>(x, y, n, s);
    case SB200_TAN: return unary_op<SB200_TAN>(x, y, n, s);
    case SB200_ASIN: return unary_op<SB200_ASIN>(x, y, n, s);
    case SB200_ACOS: return unary_op<SB200_ACOS>(x, y, n, s);
    case SB200_ATAN: return unary_op<SB200_ATAN>(x, y, n, s);
    case SB200_FLOOR: return unary_op<SB200_FLOOR>(x, y, n, s);
    case SB200_CEIL: return unary_op<SB200_CEIL>(x, y, n, s);
    case SB200_NEG: return unary_op<SB200_NEG>(x, y, n, s);
    case SB200_RECIPROCAL: return unary_op<SB200_RECIPROCAL>(x, y, n, s);
    default: return SB200_ERR_BAD_ARGUMENT;
  }
}

int sb200_activate(const float* x, float* y, int64_t n, int type, float slope, void* stream) {
  if (n < 0 || (n > 0 && (x == nullptr || y == nullptr))) return SB200_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (type) {
    case SB200_RELU: return activate_op<SB200_RELU>(x, y, n, slope, s);
    case SB200_LEAKY: return activate_op<SB200_LEAKY>(x, y, n, slope, s);
    case SB200_SIGMOID: return activate_op<SB200_SIGMOID>(x, y, n, slope, s);
    case SB200_SOFTPLUS: return activate_op<SB200_SOFTPLUS>(x, y, n, slope, s);
    case SB200_TANH: return activate_op<SB200_TANH>(x, y, n, slope, s);
    case SB200_RELU6: return activate_op<SB200_RELU6>(x, y, n, slope, s);
    case SB200_HARDSWISH: return activate_op<SB200_HARDSWISH>(x, y, n, slope, s);
    case SB200_GELU: return activate_op<SB200_GELU>(x, y, n, slope, s);
    default: return SB200_ERR_BAD_ARGUMENT;  // PReLU (0) goes through sb200_prelu
  }
}

int sb200_prelu(const float* x, float* y, int64_t outer, int64_t channels, int64_t dim,
                const float* slope, int channel_shared, void* stream) {
  if (outer < 0 || channels < 1 || dim < 1 || slope == nullptr) return SB200_ERR_BAD_ARGUMENT;
  const int64_t n = outer * channels * dim;
  if (n > 0 && (x == nullptr || y == nullptr)) return SB200_ERR_BAD_ARGUMENT;
  // the reference indexes slope[(i/dim) % channels / div_factor] with div_factor = channels when the
  // slope is shared (index always 0) and 1 otherwise.
  return launch_chan<true, false>(x, y, n, slope, nullptr, dim, channels, channel_shared ? 1 : 0, PReluFn(),
                                  static_cast<cudaStream_t>(stream), "sb200_prelu");
}

int sb200_binary_scalar(const float* a, float alpha, float* y, int64_t n, int operation, void* stream) {
  if (n < 0 || (n > 0 && (a == nullptr || y == nullptr))) return SB200_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (operation) {
    case SB200_ADD: return binary_scalar_op<SB200_ADD>(a, alpha, y, n, s);
    case SB200_SUB: return binary_scalar_op<SB200_SUB>(a, alpha, y, n, s);
    case SB200_MUL: return binary_scalar_op<SB200_MUL>(a, alpha, y, n, s);
    case SB200_DIV: return binary_scalar_op<SB200_DIV>(a, alpha, y, n, s);
    case SB200_POW: return binary_scalar_op<SB200_POW>(a, alpha, y, n, s);
    case SB200_MAX: return binary_scalar_op<SB200_MAX>(a, alpha, y, n, s);
    case SB200_MIN: return binary_scalar_op<SB200_MIN>(a, alpha, y, n, s);
    default: return SB200_ERR_BAD_ARGUMENT;
  }
}

int sb200_binary(const float* a, const float* b, float* y, int64_t n, int operation, void* stream) {
  if (n < 0 || (n > 0 && (a == nullptr || b == nullptr || y == nullptr))) return SB200_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (operation) {
    case SB200_ADD: return binary_op<SB200_ADD>(a, b, y, n, s);
    case SB200_SUB: return binary_op<SB200_SUB>(a, b, y, n, s);
    case SB200_MUL: return binary_op<SB200_MUL>(a, b, y, n, s);
    case SB200_DIV: return binary_op<SB200_DIV>(a, b, y, n, s);
    case SB200_POW: return binary_op<SB200_POW>(a, b, y, n, s);
    case SB200_MAX: return binary_op<SB200_MAX>(a, b, y, n, s);
    case SB200_MIN: return binary_op<SB200_MIN>(a, b, y, n, s);
    default: return SB200_ERR_BAD_ARGUMENT;
  }
}

int sb200_batch_norm(const float* x, float* y, int64_t n, const float* mean, const float* variance,
                     int64_t channels, int64_t inner_num, float scale_factor, float eps, void* stream) {
  if (n < 0 || channels < 1 || inner_num < 1 || mean == nullptr || variance == nullptr) return SB200_ERR_BAD_ARGUMENT;
  if (n > 0 && (x == nullptr || y == nullptr)) return SB200_ERR_BAD_ARGUMENT;
  return launch_chan<true, true>(x, y, n, mean, variance, inner_num, channels, 0, BatchNormFn{scale_factor, eps},
                                 static_cast<cudaStream_t>(stream), "sb200_batch_norm");
}

int sb200_scale_bias(const float* x, float* y, int64_t n, const float* scale, const float* bias,
                     int64_t scale_num, int64_t inner_num, void* stream) {
  if (n < 0 || scale_num < 1 || inner_num < 1 || (scale == nullptr && bias == nullptr))
    return SB200_ERR_BAD_ARGUMENT;
  if (n > 0 && (x == nullptr || y == nullptr)) return SB200_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (scale != nullptr && bias != nullptr)
    return launch_chan<true, true>(x, y, n, scale, bias, inner_num, scale_num, 0, ScaleBiasFn(), s, "sb200_scale_bias");
  if (scale != nullptr)
    return launch_chan<true, false>(x, y, n, scale, nullptr, inner_num, scale_num, 0, ScaleFn(), s, "sb200_scale_bias");
  return launch_chan<false, true>(x, y, n, nullptr, bias, inner_num, scale_num, 0, BiasFn(), s, "sb200_scale_bias");
}

}  // extern "C"
