// Pooling (max / average) over 2 or 3 spatial axes of x[planes, in_d, in_h, in_w] (2-D: in_d = 1).
//
// Window of output (d, h, w): starts at index*stride - pad per axis, ends at
// min(start + kernel, in + pad); the average divides by the size of that window BEFORE it is
// clipped to the tensor (padding counts), the maximum starts from the lowest float.
//   small windows (<= 64 elements, the usual 2x2 / 3x3 case): one thread per output walks its
//       window in the reference's order (d, then h, then w), so the float sum is bit-identical.
//       2-D: the input rows a block needs are ONE contiguous range of the tensor (a band of rows of
//       one plane, or several whole planes when planes are small); the block brings it into shared
//       memory with 16-byte asynchronous copies (coalesced, no register staging) and the windows
//       are read from there, so global memory sees 128-bit accesses only and every output store is
//       coalesced (pool_smem_kernel).  3-D, bands wider than the shared-memory budget and
//       misaligned bases: windows read through L1/L2 (pool_thread_kernel);
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

// 2-D pooling from a shared-memory copy of the block's input.
// Block b = (group, band): planes [group*G, group*G + g) and output rows [band*TH, band*TH + rows) of
// them (G > 1 only with whole planes: NB == 1, TH == out_h).  Three layouts of the copy:
//   kPoolFlat      the contiguous float range [in_start, in_end) of x as it lies in memory (the copy starts at
//                  in_start rounded down to a multiple of 4 floats); windows that leave the tensor are clipped;
//   kPoolFlatFree  the same when no window of the geometry leaves the tensor: no clipping code at all;
//   kPoolPadded    one band of one plane (G == 1, in_w a multiple of 4) laid out WITH its padding: tile rows
//                  of `pitch` floats, the tensor's columns starting at column `lead`, everything else holding
//                  the neutral value (lowest float for max; +0 for the average, which leaves a float sum
//                  unchanged bit for bit: the running sum starts at +0 and never becomes -0) - so every
//                  window, also one over an edge, is the same unrolled walk without a test.
enum { kPoolFlat = 0, kPoolFlatFree = 1, kPoolPadded = 2 };
struct PoolTile {
  int G, TH, NB;          // planes per block, output rows per band, bands per plane
  int pitch, lead;        // kPoolPadded: floats per tile row, tile column of tensor column 0 (both multiples of 4)
  FastDiv32 div_w4;       // by in_w / 4
  FastDiv32 div_nb;       // by NB
  int64_t planes;
  int64_t total_in;       // planes * in_h * in_w
};

// KH x KW > 0: the window extents as compile-time constants (must equal g.k_h, g.k_w): an unrolled walk
// with all loads ahead of the arithmetic; KH == 0: run-time loops.
template <bool AVG, int KH, int KW, int MODE>
__global__ void __launch_bounds__(kThreads)
pool_smem_kernel(const float* __restrict__ x, float* y, const __grid_constant__ PoolGeom g, const __grid_constant__ PoolTile q) {
  extern __shared__ __align__(16) float pool_sm[];
  const int t = threadIdx.x;
  uint32_t group, band_u;
  q.div_nb.divmod(blockIdx.x, group, band_u);
  const int band = static_cast<int>(band_u);
  const int64_t p0 = static_cast<int64_t>(group) * q.G;
  const int n_planes = static_cast<int>((q.planes - p0) < q.G ? (q.planes - p0) : q.G);
  const int oh0 = band * q.TH;
  const int rows = (q.G > 1) ? n_planes * g.out_h : min(q.TH, g.out_h - oh0);
  const int plane_in = g.in_h * g.in_w;   // fits an int (checked by the planner)
  const int in_w = g.in_w, in_h = g.in_h;
  const uint32_t sm_addr = static_cast<uint32_t>(__cvta_generic_to_shared(pool_sm));
  int origin;      // kPoolFlat*: index in pool_sm of element (0, 0) of the block's first plane
  if (MODE == kPoolPadded) {
    const int tile_rows = (rows - 1) * g.s_h + g.k_h, h_first = oh0 * g.s_h - g.p_h;
    const float neutral = AVG ? 0.f : -FLT_MAX;
    const float4 fill = make_float4(neutral, neutral, neutral, neutral);
    const int hr0 = max(h_first, 0), hr1 = max(min(h_first + tile_rows, in_h), hr0);
    // neutral values where the copy below does not write: tile rows above and below the tensor's rows, and the
    // columns left and right of the tensor's columns in the rows between (disjoint from the copy: no barrier)
    float4* sm4 = reinterpret_cast<float4*>(pool_sm);
    const int pitch4 = q.pitch >> 2, top4 = (hr0 - h_first) * pitch4, mid_end4 = (hr1 - h_first) * pitch4;
    for (int j = t; j < top4; j += kThreads) sm4[j] = fill;
    for (int j = mid_end4 + t; j < tile_rows * pitch4; j += kThreads) sm4[j] = fill;
    const int left4 = q.lead >> 2, right0 = left4 + (in_w >> 2), side4 = left4 + (pitch4 - right0);
    for (int j = t; j < (hr1 - hr0) * side4; j += kThreads) {   // a few cells per row: most threads skip this loop
      const int r = j / side4, b = j - r * side4;
      sm4[top4 + r * pitch4 + (b < left4 ? b : right0 + (b - left4))] = fill;
    }
    const int w4 = in_w >> 2, n_vec = (hr1 - hr0) * w4;
    const float4* src = reinterpret_cast<const float4*>(x + p0 * plane_in + static_cast<int64_t>(hr0) * in_w);
    const uint32_t dst0 = sm_addr + 4u * static_cast<uint32_t>((hr0 - h_first) * q.pitch + q.lead);
    for (int j = t; j < n_vec; j += kThreads) {
      uint32_t r, c4;
      q.div_w4.divmod(static_cast<uint32_t>(j), r, c4);
      cp_async16(dst0 + 4u * (r * q.pitch) + 16u * c4, src + j);
    }
    cp_async_commit();
    origin = 0;
  } else {
    int h_lo = 0, h_hi = in_h;
    if (q.G == 1) {
      h_lo = max(oh0 * g.s_h - g.p_h, 0);
      h_hi = min(min((oh0 + rows - 1) * g.s_h - g.p_h + g.k_h, in_h + g.p_h), in_h);
      h_hi = max(h_hi, h_lo);
    }
    const int64_t in_start = p0 * plane_in + static_cast<int64_t>(h_lo) * in_w;
    const int64_t in_end = (q.G > 1) ? (p0 + n_planes) * plane_in : p0 * plane_in + static_cast<int64_t>(h_hi) * in_w;
    const int64_t a0 = in_start & ~static_cast<int64_t>(3);
    // whole float4 that lie inside the tensor; what is left of the range (at most 3 floats) by scalar loads
    int64_t vec_end = (in_end + 3) & ~static_cast<int64_t>(3);
    const int64_t tensor_vec_end = q.total_in & ~static_cast<int64_t>(3);
    if (vec_end > tensor_vec_end) vec_end = tensor_vec_end;
    const int n_vec = vec_end > a0 ? static_cast<int>((vec_end - a0) >> 2) : 0;
    const float4* src = reinterpret_cast<const float4*>(x + a0);
    for (int j = t; j < n_vec; j += kThreads) cp_async16(sm_addr + 16u * j, src + j);
    cp_async_commit();
    const int n_in = static_cast<int>(in_end - a0);
    for (int i = 4 * n_vec + t; i < n_in; i += kThreads) pool_sm[i] = __ldg(x + a0 + i);
    origin = static_cast<int>(in_start - a0) - h_lo * in_w;
  }
  cp_async_wait<0>();
  __syncthreads();

  const int n_out = rows * g.out_w;
  float* yb = y + (p0 * g.out_h + oh0) * static_cast<int64_t>(g.out_w);
  // local output o = row * out_w + ow, walked with a stride of kThreads without a division per output
  uint32_t row, ow;
  g.div_w.divmod(static_cast<uint32_t>(t), row, ow);
  const uint32_t d_row = g.div_w.div(kThreads), d_ow = kThreads - d_row * g.out_w;
  // row stride of the copy, and what to add to hs * stride + ws to reach the window's first element
  const int stride = (MODE == kPoolPadded) ? q.pitch : in_w;
  const int first = (MODE == kPoolPadded) ? (g.p_h - oh0 * g.s_h) * q.pitch + q.lead : origin;
  for (int o = t; o < n_out; o += kThreads) {
    uint32_t pl = 0, oh = static_cast<uint32_t>(oh0) + row;
    if (q.G > 1) g.div_h.divmod(row, pl, oh);
    const int hs = static_cast<int>(oh) * g.s_h - g.p_h, ws = static_cast<int>(ow) * g.s_w - g.p_w;
    const int off = first + static_cast<int>(pl) * plane_in;
    float max_val = -FLT_MAX, sum_val = 0.f;
    int pool_size = KH * KW;
    const bool whole = MODE != kPoolFlat || (hs >= 0 && hs + KH <= in_h && ws >= 0 && ws + KW <= in_w);
    if (MODE != kPoolFlatFree && AVG) pool_size = (min(hs + g.k_h, in_h + g.p_h) - hs) * (min(ws + g.k_w, in_w + g.p_w) - ws);
    if (KH > 0 && whole) {
      const float* rp = pool_sm + (off + hs * stride + ws);
      float v[KH > 0 ? KH * KW : 1];
#pragma unroll
      for (int i = 0; i < KH; ++i)
#pragma unroll
        for (int j = 0; j < KW; ++j) v[i * KW + j] = rp[i * stride + j];
#pragma unroll
      for (int e = 0; e < KH * KW; ++e) {
        if (AVG) sum_val = __fadd_rn(sum_val, v[e]);
        else max_val = std_max(max_val, v[e]);
      }
    } else if (KH > 0) {
      // kPoolFlat, a window over an edge: the same unrolled walk with one predicate per row and per column
      // (an element is taken exactly when it lies inside the tensor)
      const int rbase = off + hs * in_w + ws;
      bool col_ok[KW > 0 ? KW : 1];
#pragma unroll
      for (int j = 0; j < KW; ++j) col_ok[j] = static_cast<unsigned>(ws + j) < static_cast<unsigned>(in_w);
#pragma unroll
      for (int i = 0; i < KH; ++i) {
        const bool row_ok = static_cast<unsigned>(hs + i) < static_cast<unsigned>(in_h);
#pragma unroll
        for (int j = 0; j < KW; ++j) {
          if (row_ok && col_ok[j]) {
            const float v = pool_sm[rbase + i * in_w + j];
            if (AVG) sum_val = __fadd_rn(sum_val, v);
            else max_val = std_max(max_val, v);
          }
        }
      }
    } else {
      int h0 = hs, h1 = hs + g.k_h, w0 = ws, w1 = ws + g.k_w;
      if (MODE == kPoolFlat) h0 = max(h0, 0), h1 = min(h1, in_h), w0 = max(w0, 0), w1 = min(w1, in_w);
      if (MODE == kPoolFlatFree) pool_size = g.k_h * g.k_w;
      for (int ph = h0; ph < h1; ++ph) {
        const int ro = off + ph * stride;
        for (int pw = w0; pw < w1; ++pw) {
          const float v = pool_sm[ro + pw];
          if (AVG) sum_val = __fadd_rn(sum_val, v);
          else max_val = std_max(max_val, v);
        }
      }
    }
    st_stream(yb + o, AVG ? __fdiv_rn(sum_val, static_cast<float>(pool_size)) : max_val);
    ow += d_ow;
    row += d_row;
    if (ow >= static_cast<uint32_t>(g.out_w)) ow -= g.out_w, ++row;
  }
}

// Shared-memory budget of one pool_smem_kernel block.  Measured on [256*64, 112, 112] and [1024*2048, 7, 7]: 56 KB
// (four blocks per SM, 12 outputs per thread) beats 24 KB (eight blocks, 4 outputs per thread) by 3-17 % - the
// kernel is bound by instruction issue, and the per-thread set-up is shared by more outputs.
constexpr int kPoolSmemBudget = 56 * 1024;
constexpr int kPoolSmemMax = 100 * 1024;

// Chooses the layout and planes per block or rows per band; false when one output row's input does not fit.
inline bool plan_pool_tile(const PoolGeom& g, int64_t planes, PoolTile& q, int& mode, int& smem_bytes) {
  const int64_t plane_bytes = static_cast<int64_t>(g.in_h) * g.in_w * 4;
  if (plane_bytes >= (1ll << 32)) return false;   // the kernel indexes a plane with an int
  q.planes = planes;
  q.total_in = planes * g.in_h * g.in_w;
  q.pitch = q.lead = 0;
  q.div_w4 = FastDiv32(static_cast<uint32_t>(g.in_w / 4 > 0 ? g.in_w / 4 : 1));
  // exclusive end, in tensor coordinates, of the last window along each axis before clipping
  const int64_t reach_h = static_cast<int64_t>(g.out_h - 1) * g.s_h - g.p_h + g.k_h;
  const int64_t reach_w = static_cast<int64_t>(g.out_w - 1) * g.s_w - g.p_w + g.k_w;
  const bool all_inside = g.p_h == 0 && g.p_w == 0 && reach_h <= g.in_h && reach_w <= g.in_w;
  mode = all_inside ? kPoolFlatFree : kPoolFlat;
  int64_t bytes;
  if (plane_bytes * 2 <= kPoolSmemBudget) {
    q.G = static_cast<int>(kPoolSmemBudget / plane_bytes);
    // whole passes of the block's threads over its outputs: a last pass with a few outputs leaves most threads idle
    const int64_t out_plane = static_cast<int64_t>(g.out_h) * g.out_w;
    const int64_t passes = q.G * out_plane / kThreads;
    if (passes >= 1 && passes * kThreads / out_plane >= 1) q.G = static_cast<int>(passes * kThreads / out_plane);
    if (q.G > planes) q.G = static_cast<int>(planes);
    q.NB = 1, q.TH = g.out_h;
    if (static_cast<int64_t>(q.G) * g.out_h * g.out_w >= (1ll << 30)) return false;
    bytes = (static_cast<int64_t>(q.G) * g.in_h * g.in_w + 8) * 4;
  } else {
    q.G = 1;
    int64_t row_floats = g.in_w;
    if (!all_inside && (g.in_w & 3) == 0) {
      mode = kPoolPadded;
      q.lead = (g.p_w + 3) & ~3;
      const int64_t pitch = (q.lead + (reach_w > g.in_w ? reach_w : g.in_w) + 3) & ~static_cast<int64_t>(3);
      if (pitch >= (1 << 20)) return false;
      q.pitch = static_cast<int>(pitch);
      row_floats = pitch;
    }
    const int64_t row_bytes = row_floats * 4;
    // input rows of a band of th output rows: (th - 1) * s_h + k_h
    int64_t th = (kPoolSmemBudget / row_bytes - g.k_h) / g.s_h + 1;
    if (kPoolSmemBudget / row_bytes < g.k_h) th = 1;
    if (th > g.out_h) th = g.out_h;
    q.NB = static_cast<int>((g.out_h + th - 1) / th);
    q.TH = (g.out_h + q.NB - 1) / q.NB;
    q.NB = (g.out_h + q.TH - 1) / q.TH;
    int64_t in_rows = static_cast<int64_t>(q.TH - 1) * g.s_h + g.k_h;
    if (mode != kPoolPadded && in_rows > g.in_h) in_rows = g.in_h;
    bytes = (in_rows * row_floats + 8) * 4;
  }
  if (bytes > kPoolSmemMax) return false;
  q.div_nb = FastDiv32(static_cast<uint32_t>(q.NB));
  smem_bytes = static_cast<int>(bytes);
  const int64_t blocks = ((planes + q.G - 1) / q.G) * q.NB;
  return blocks < (1ll << 31);
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
  PoolTile q;
  int smem_bytes = 0, mode = kPoolFlat;
  if (window <= 64 && g.in_d == 1 && g.out_d == 1 && g.k_d == 1 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
      plan_pool_tile(g, planes, q, mode, smem_bytes)) {
    const unsigned blocks = static_cast<unsigned>(((planes + q.G - 1) / q.G) * q.NB);
    const bool avg = pool_type == 1;
#define SB200_POOL_M(KH, KW, MODE)                                                                             \
  do {                                                                                                         \
    static unsigned long long done_avg = 0, done_max = 0;                                                      \
    if (avg) {                                                                                                 \
      allow_dynamic_smem(pool_smem_kernel<true, KH, KW, MODE>, kPoolSmemMax, &done_avg);                       \
      pool_smem_kernel<true, KH, KW, MODE><<<blocks, kThreads, smem_bytes, s>>>(x, y, g, q);                   \
    } else {                                                                                                   \
      allow_dynamic_smem(pool_smem_kernel<false, KH, KW, MODE>, kPoolSmemMax, &done_max);                      \
      pool_smem_kernel<false, KH, KW, MODE><<<blocks, kThreads, smem_bytes, s>>>(x, y, g, q);                  \
    }                                                                                                          \
  } while (0)
#define SB200_POOL(KH, KW)                                                                                     \
  do {                                                                                                         \
    if (mode == kPoolPadded) SB200_POOL_M(KH, KW, kPoolPadded);                                                \
    else if (mode == kPoolFlatFree) SB200_POOL_M(KH, KW, kPoolFlatFree);                                       \
    else SB200_POOL_M(KH, KW, kPoolFlat);                                                                      \
  } while (0)
    if (g.k_h == 2 && g.k_w == 2) SB200_POOL(2, 2);
    else if (g.k_h == 3 && g.k_w == 3) SB200_POOL(3, 3);
    else if (g.k_h == 7 && g.k_w == 7) SB200_POOL(7, 7);   // global pooling of 7x7 planes
    else SB200_POOL(0, 0);
#undef SB200_POOL
#undef SB200_POOL_M
  } else if (window <= 64) {
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
