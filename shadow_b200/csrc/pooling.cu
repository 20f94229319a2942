// Pooling (max / average) over 2 or 3 spatial axes of x[planes, in_d, in_h, in_w] (2-D: in_d = 1).
//
// Window of output (d, h, w): starts at index*stride - pad per axis, ends at
// min(start + kernel, in + pad); the average divides by the size of that window BEFORE it is
// clipped to the tensor (padding counts), the maximum starts from the lowest float.
//   small windows (<= 64 elements, the usual 2x2 / 3x3 case): one thread per output walks its
//       window in the reference's order (d, then h, then w), so the float sum is bit-identical;
//       neighbouring threads read neighbouring windows, the overlap is served by L1/L2;
//   large windows (global pooling): one warp per output, lanes stride over the window and merge
//       by shuffles; the sum is accumulated in double (the reference adds floats one by one, so
//       the average matches it to the reduction tolerance, the maximum exactly).
// Algorithmic bytes: 4 * (|x| + |y|).
#include <float.h>

#include "common.cuh"
#include "math.cuh"

namespace sb200 {
namespace {

constexpr int kThreads = 256;

struct PoolGeom {
  int in_d, in_h, in_w, out_d, out_h, out_w;
  int k_d, k_h, k_w, s_d, s_h, s_w, p_d, p_h, p_w;
  FastDiv32 div_w, div_h, div_d;   // by out_w, out_h, out_d
};

struct Window {
  int d0, d1, h0, h1, w0, w1;   // clipped to the tensor
  int pool_size;                // before clipping
};

__device__ __forceinline__ Window window_of(const PoolGeom& g, int od, int oh, int ow) {
  Window w;
  int ds = od * g.s_d - g.p_d, hs = oh * g.s_h - g.p_h, ws = ow * g.s_w - g.p_w;
  int de = min(ds + g.k_d, g.in_d + g.p_d), he = min(hs + g.k_h, g.in_h + g.p_h), we = min(ws + g.k_w, g.in_w + g.p_w);
  w.pool_size = (de - ds) * (he - hs) * (we - ws);
  w.d0 = max(ds, 0), w.h0 = max(hs, 0), w.w0 = max(ws, 0);
  w.d1 = min(de, g.in_d), w.h1 = min(he, g.in_h), w.w1 = min(we, g.in_w);
  return w;
}

// output index -> (plane, od, oh, ow); requires the output count < 2^32
__device__ __forceinline__ void decode(const PoolGeom& g, uint32_t i, uint32_t& plane, int& od, int& oh, int& ow) {
  uint32_t q, r;
  g.div_w.divmod(i, q, r);
  ow = static_cast<int>(r);
  g.div_h.divmod(q, q, r);
  oh = static_cast<int>(r);
  g.div_d.divmod(q, plane, r);
  od = static_cast<int>(r);
}

template <bool AVG>
__global__ void __launch_bounds__(kThreads)
pool_thread_kernel(const float* __restrict__ x, float* y, uint32_t count, const __grid_constant__ PoolGeom g) {
  const int64_t i64 = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (i64 >= count) return;
  const uint32_t i = static_cast<uint32_t>(i64);
  uint32_t plane;
  int od, oh, ow;
  decode(g, i, plane, od, oh, ow);
  const Window w = window_of(g, od, oh, ow);
  const float* xp = x + static_cast<int64_t>(plane) * g.in_d * g.in_h * g.in_w;
  float max_val = -FLT_MAX, sum_val = 0.f;
  for (int pd = w.d0; pd < w.d1; ++pd)
    for (int ph = w.h0; ph < w.h1; ++ph) {
      const float* row = xp + (static_cast<int64_t>(pd) * g.in_h + ph) * g.in_w;
      for (int pw = w.w0; pw < w.w1; ++pw) {
        const float v = __ldg(row + pw);
        if (AVG) sum_val = __fadd_rn(sum_val, v);
        else max_val = std_max(max_val, v);
      }
    }
  y[i] = AVG ? __fdiv_rn(sum_val, static_cast<float>(w.pool_size)) : max_val;
}

template <bool AVG>
__global__ void __launch_bounds__(kThreads)
pool_warp_kernel(const float* __restrict__ x, float* y, uint32_t count, const __grid_constant__ PoolGeom g) {
  const uint32_t i = static_cast<uint32_t>((static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5);   // one warp per output
  const int lane = threadIdx.x & 31;
  if (i >= count) return;
  uint32_t plane;
  int od, oh, ow;
  decode(g, i, plane, od, oh, ow);
  const Window w = window_of(g, od, oh, ow);
  const float* xp = x + static_cast<int64_t>(plane) * g.in_d * g.in_h * g.in_w;
  const int nw = w.w1 - w.w0, nh = w.h1 - w.h0, nd = w.d1 - w.d0;
  const int n = (nw > 0 && nh > 0 && nd > 0) ? nw * nh * nd : 0;
  float max_val = -FLT_MAX;
  double sum_val = 0.0;
  for (int e = lane; e < n; e += 32) {
    const int pw = e % nw, t = e / nw;
    const int ph = t % nh, pd = t / nh;
    const float v = ld_stream(xp + (static_cast<int64_t>(w.d0 + pd) * g.in_h + (w.h0 + ph)) * g.in_w + (w.w0 + pw));
    if (AVG) sum_val += static_cast<double>(v);
    else max_val = std_max(max_val, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    if (AVG) sum_val += __shfl_xor_sync(0xffffffffu, sum_val, o);
    else max_val = std_max(max_val, __shfl_xor_sync(0xffffffffu, max_val, o));
  }
  if (lane == 0) y[i] = AVG ? __fdiv_rn(static_cast<float>(sum_val), static_cast<float>(w.pool_size)) : max_val;
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" int sb200_pooling(const float* x, float* y, int64_t planes, const int* in_dhw, const int* out_dhw,
                             const int* kernel, const int* stride, const int* pad, int pool_type, void* stream) {
  if (in_dhw == nullptr || out_dhw == nullptr || kernel == nullptr || stride == nullptr || pad == nullptr || planes < 0 ||
      pool_type < 0 || pool_type > 1)
    return SB200_ERR_BAD_ARGUMENT;
  for (int a = 0; a < 3; ++a)
    if (in_dhw[a] < 1 || out_dhw[a] < 1 || kernel[a] < 1 || stride[a] < 1 || pad[a] < 0) return SB200_ERR_BAD_ARGUMENT;
  if (planes == 0) return SB200_OK;
  if (x == nullptr || y == nullptr || x == y) return SB200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 3u) return SB200_ERR_BAD_ARGUMENT;
  const int64_t out_plane = static_cast<int64_t>(out_dhw[0]) * out_dhw[1] * out_dhw[2];
  const int64_t count = planes * out_plane;
  const int64_t in_count = planes * in_dhw[0] * in_dhw[1] * static_cast<int64_t>(in_dhw[2]);
  if (count >= (1ll << 31) || in_count > (1ll << 40)) return SB200_ERR_UNSUPPORTED;
  PoolGeom g;
  g.in_d = in_dhw[0], g.in_h = in_dhw[1], g.in_w = in_dhw[2];
  g.out_d = out_dhw[0], g.out_h = out_dhw[1], g.out_w = out_dhw[2];
  g.k_d = kernel[0], g.k_h = kernel[1], g.k_w = kernel[2];
  g.s_d = stride[0], g.s_h = stride[1], g.s_w = stride[2];
  g.p_d = pad[0], g.p_h = pad[1], g.p_w = pad[2];
  g.div_w = FastDiv32(static_cast<uint32_t>(g.out_w));
  g.div_h = FastDiv32(static_cast<uint32_t>(g.out_h));
  g.div_d = FastDiv32(static_cast<uint32_t>(g.out_d));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t window = static_cast<int64_t>(kernel[0]) * kernel[1] * kernel[2];
  const uint32_t n = static_cast<uint32_t>(count);
  if (window <= 64) {
    const unsigned blocks = static_cast<unsigned>((count + kThreads - 1) / kThreads);
    if (pool_type == 1) pool_thread_kernel<true><<<blocks, kThreads, 0, s>>>(x, y, n, g);
    else pool_thread_kernel<false><<<blocks, kThreads, 0, s>>>(x, y, n, g);
  } else {
    const int64_t blocks = (count * 32 + kThreads - 1) / kThreads;
    if (blocks >= (1ll << 31)) return SB200_ERR_UNSUPPORTED;
    if (pool_type == 1) pool_warp_kernel<true><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(x, y, n, g);
    else pool_warp_kernel<false><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(x, y, n, g);
  }
  return after_launch("sb200_pooling");
}
