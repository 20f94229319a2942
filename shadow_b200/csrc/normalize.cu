// Normalize: y = x / max(||x||_p, eps), the p-norm taken over the middle axis of x viewed as
// [outer, dim, inner].
//
// The reference makes two passes with a scratch blob of outer*inner norms; here one launch reads
// the tensor, keeps the norms on chip and writes the result (the second read of a block's patch
// comes from L2): 8 algorithmic bytes per element, no scratch.  Thread layout as in the strided
// softmax: P planes x G row groups x W columns per block, so consecutive threads read
// consecutive addresses for any `inner` (inner == 1 included, where the G row groups of a row
// are the consecutive lanes).
// Arithmetic follows the reference term by term: |x| (p = 1), the float product |x|*|x| (p = 2)
// or powf(|x|, p), accumulated in double; the norm is (float)sum, sqrtf((float)sum) or
// powf((float)sum, 1/p); every output is the correctly rounded float quotient x / max(norm, eps).
// Only the order of the double additions differs (tree instead of left to right), which moves
// the float norm by at most one ulp, and rarely.
#include <float.h>

#include "colwalk.cuh"
#include "common.cuh"
#include "math.cuh"

namespace sb200 {
namespace {

// kSsdChannel / kSsdSpatial: SSDNormalize (sum of float squares in double; see sb200_ssd_normalize)
enum { kNormL1 = 1, kNormL2 = 2, kNormLp = 0, kSsdChannel = 3, kSsdSpatial = 4 };
enum { kScaleNone = 0, kScaleShared = 1, kScaleChannel = 2 };

struct SsdScale {
  const float* scale;      // one value (shared) or one per channel
  FastDiv32 div_spatial;   // kSsdSpatial: channel of flattened position r is r / spatial
};

template <int MODE>
__device__ __forceinline__ double norm_term(float v, float p) {
  const float a = fabsf(v);
  if (MODE == kNormL1) return static_cast<double>(a);
  if (MODE == kNormL2 || MODE == kSsdChannel || MODE == kSsdSpatial) return static_cast<double>(__fmul_rn(a, a));
  return static_cast<double>(powf(a, p));
}

template <int MODE, int kT, int kU, int SCALE>
__global__ void __launch_bounds__(kT, 1024 / kT)
normalize_plane_kernel(const float* x, float* y, int64_t outer, int dim, int64_t inner, int W, int G, int P,
                       int64_t ntile, float p, float eps, const __grid_constant__ SsdScale ssd) {
  __shared__ double sm_acc[kT];
  const int t = threadIdx.x;
  const int sidx = t % W, pg = t / W;
  const int g = pg % G, pl = pg / G;
  const int64_t bn = blockIdx.x / ntile, tile = blockIdx.x - bn * ntile;
  const int64_t n = bn * P + pl;
  const int64_t col = tile * W + sidx;
  const bool live = (pl < P) && (n < outer) && (col < inner);
  const int64_t origin = live ? (n * dim + g) * inner + col : 0;
  const float* xp = x + origin;
  float* yp = y + origin;
  const int64_t step = static_cast<int64_t>(G) * inner;
  const int cnt = live ? (dim - g + G - 1) / G : 0;   // rows of this thread
  double acc = 0.0;
  {
    const float* q = xp;
    int k = 0;
    for (; k + kU <= cnt; k += kU, q += kU * step) {
      float v[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) v[u] = q[u * step];   // default caching: stays in L2 for pass 2
#pragma unroll
      for (int u = 0; u < kU; ++u) acc += norm_term<MODE>(v[u], p);
    }
    for (; k < cnt; ++k, q += step) acc += norm_term<MODE>(*q, p);
  }
  sm_acc[t] = acc;
  __syncthreads();
  if (!live) return;
  const int first = pl * G * W + sidx;
  double sum = 0.0;
  for (int k = 0; k < G; ++k) sum += sm_acc[first + k * W];
  float d, factor = 0.f;
  if (MODE == kSsdChannel) {
    d = static_cast<float>(sqrt(sum + static_cast<double>(eps)));
  } else if (MODE == kSsdSpatial) {
    d = __fsqrt_rn(__fadd_rn(static_cast<float>(sum), eps));
    factor = __fdiv_rn(1.f, d);
  } else {
    float val = static_cast<float>(sum);
    if (MODE == kNormL2) val = __fsqrt_rn(val);
    if (MODE == kNormLp) val = powf(val, __fdiv_rn(1.f, p));
    d = (val < eps) ? eps : val;   // std::max(val, eps)
  }
  const bool d_ok = (d >= 0x1p-60f) && (d <= 0x1p60f);
  const float rcp = __frcp_rn(d);
  const float shared_scale = (SCALE == kScaleShared) ? __ldg(ssd.scale) : 1.f;
  // row index r of the value -> output
  auto finish = [&](float v, int r) {
    float o = (MODE == kSsdSpatial) ? __fmul_rn(v, factor) : div_exact(v, d, rcp, d_ok);
    if (SCALE == kScaleShared) o = __fmul_rn(o, shared_scale);
    if (SCALE == kScaleChannel)
      o = __fmul_rn(o, __ldg(ssd.scale + (MODE == kSsdSpatial ? ssd.div_spatial.div(static_cast<uint32_t>(r)) : static_cast<uint32_t>(r))));
    return o;
  };
  const float* q = xp;
  float* o = yp;
  int k = 0;
  for (; k + kU <= cnt; k += kU, q += kU * step, o += kU * step) {
    float v[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) v[u] = ld_stream(q + u * step);
#pragma unroll
    for (int u = 0; u < kU; ++u) st_stream(o + u * step, finish(v[u], g + (k + u) * G));
  }
  for (; k < cnt; ++k, q += step, o += step) st_stream(o, finish(ld_stream(q), g + k * G));
}

// What turns a norm's double sum into the divisor (and, for kSsdSpatial, the factor).
template <int MODE>
__device__ __forceinline__ float norm_divisor(double sum, float p, float eps) {
  if (MODE == kSsdChannel) return static_cast<float>(sqrt(sum + static_cast<double>(eps)));
  if (MODE == kSsdSpatial) return __fsqrt_rn(__fadd_rn(static_cast<float>(sum), eps));
  float val = static_cast<float>(sum);
  if (MODE == kNormL2) val = __fsqrt_rn(val);
  if (MODE == kNormLp) val = powf(val, __fdiv_rn(1.f, p));
  return (val < eps) ? eps : val;   // std::max(val, eps)
}

// The same operator on the fixed-column 128-bit walk (colwalk.cuh; inner > 1): float4 loads and
// stores, four double accumulators per thread (one per lane = column), column sums through shared
// memory in partial-row order, then the patch again from L2 and one float4 store per float4.
template <int MODE, int SCALE, int U, int NB>
__global__ void __launch_bounds__(1024, 1)
normalize_colvec_kernel(const float* x, float* y, const __grid_constant__ ColWalk q, float p, float eps,
                        const __grid_constant__ SsdScale ssd) {
  // during pass 1 the memory is the threads' copy rings (colwalk_stream); afterwards it holds the
  // per-lane partial sums
  extern __shared__ double sm_sum[];   // [blockDim * 4]
  const ColLane L = colwalk_thread(q, threadIdx.x, blockIdx.x);
  const float4* xp = reinterpret_cast<const float4*>(x) + L.first4;
  float4* yp = reinterpret_cast<float4*>(y) + L.first4;
  const int64_t step = L.step4;
  const int cnt = L.cnt;
  double acc[4] = {0.0, 0.0, 0.0, 0.0};
  colwalk_stream<U, NB>(xp, step, cnt, reinterpret_cast<float4*>(sm_sum) + threadIdx.x,
                        [&](const float4 (&v)[U], int, int valid) {
#pragma unroll
                          for (int u = 0; u < U; ++u) {
                            if (u < valid) {
                              acc[0] += norm_term<MODE>(v[u].x, p), acc[1] += norm_term<MODE>(v[u].y, p);
                              acc[2] += norm_term<MODE>(v[u].z, p), acc[3] += norm_term<MODE>(v[u].w, p);
                            }
                          }
                        });
  __syncthreads();   // all rings drained: the memory now takes the partials
  if (L.slot >= 0) {
#pragma unroll
    for (int e = 0; e < 4; ++e) sm_sum[L.slot + e] = acc[e];
  }
  __syncthreads();
  // one thread per (plane, column): partial rows in order; the divisor (a float) is left in row 0
  const int planes = q.tiled ? 1 : q.P;
  const int plane_slots = 4 * q.tact;
  for (int c = threadIdx.x; c < planes * q.ncols; c += blockDim.x) {
    const int pl = static_cast<int>(q.div_ncols.div(static_cast<uint32_t>(c)));
    double* col = sm_sum + pl * plane_slots + (c - pl * q.ncols);
    double sum = col[0];
    for (int r = 1; r < q.R; ++r) sum += col[r * q.ncols];
    col[0] = static_cast<double>(norm_divisor<MODE>(sum, p, eps));
  }
  __syncthreads();
  if (cnt == 0) return;
  float d[4], rcp[4];
  bool ok[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    d[e] = static_cast<float>(sm_sum[L.plane_base + colwalk_col(q, L, e)]);
    ok[e] = (d[e] >= 0x1p-60f) && (d[e] <= 0x1p60f);
    rcp[e] = __frcp_rn(d[e]);
  }
  const float shared_scale = (SCALE == kScaleShared) ? __ldg(ssd.scale) : 1.f;
  // row (index along dim) of lane e at step k: row0 (+1 when the lane wrapped into the next row)
  // + k * rows_per_step
  int row[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) row[e] = L.row0 + ((!q.tiled && L.rem0 + e >= q.ncols) ? 1 : 0);
  auto out4 = [&](const float4& v, int k) {
    float o[4] = {v.x, v.y, v.z, v.w};
    div_exact4(o, d, rcp, ok);
    if (SCALE == kScaleShared) {
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = __fmul_rn(o[e], shared_scale);
    }
    if (SCALE == kScaleChannel) {
      const int base = k * q.rows_per_step;
      if (q.tiled) {   // the four lanes of a tiled layout sit in one row: one scale for the float4
        const float sc = __ldg(ssd.scale + row[0] + base);
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = __fmul_rn(o[e], sc);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = __fmul_rn(o[e], __ldg(ssd.scale + row[e] + base));
      }
    }
    return make_float4(o[0], o[1], o[2], o[3]);
  };
  const float4* ptr = xp;
  float4* out = yp;
  int k = 0;
  for (; k + U <= cnt; k += U, ptr += U * step, out += U * step) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = ld_stream(ptr + u * step);
#pragma unroll
    for (int u = 0; u < U; ++u) st_stream(out + u * step, out4(v[u], k + u));
  }
  if (k < cnt) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (k + u < cnt) v[u] = ld_stream(ptr + u * step);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (k + u < cnt) st_stream(out + u * step, out4(v[u], k + u));
  }
}

// inner == 1 with rows of up to 32768 floats (a multiple of 4, 16-byte aligned): the row lives in
// the registers of TPR threads (NV float4 each): one 128-bit read, a shuffle / shared-memory sum
// of the doubles, one 128-bit write.  No second read at all.
template <int TPR>
__device__ __forceinline__ double row_sum(double v, double* red) {
  if (TPR <= 32) {
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
  } else {
    constexpr int WPR = TPR / 32;
    v = warp_reduce(v, OpAddD());
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int first = (warp / WPR) * WPR;
    double r = (lane < WPR) ? red[first + lane] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
  }
}

template <int MODE, int SCALE, int TPR, int NV, int BLOCK>
__global__ void __launch_bounds__(BLOCK)
normalize_rows_kernel(const float* x, float* y, int64_t rows, int units_per_row, float p, float eps,
                      const __grid_constant__ SsdScale ssd) {
  constexpr int RPB = BLOCK / TPR;
  __shared__ double red[BLOCK / 32];
  const int t = threadIdx.x % TPR;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * RPB + threadIdx.x / TPR;
  const bool live = r < rows;   // dead rows still take part in the barrier
  const float4* xr = reinterpret_cast<const float4*>(x) + r * units_per_row;
  float4* yr = reinterpret_cast<float4*>(y) + r * units_per_row;
  float4 v[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int u = t + i * TPR;
    v[i] = (live && u < units_per_row) ? ld_stream(xr + u) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  double a0 = 0.0, a1 = 0.0;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int u = t + i * TPR;
    if (live && u < units_per_row) {
      a0 += norm_term<MODE>(v[i].x, p), a1 += norm_term<MODE>(v[i].y, p);
      a0 += norm_term<MODE>(v[i].z, p), a1 += norm_term<MODE>(v[i].w, p);
    }
  }
  const double sum = row_sum<TPR>(a0 + a1, red);
  const float d = norm_divisor<MODE>(sum, p, eps);
  const bool d_ok = (d >= 0x1p-60f) && (d <= 0x1p60f);
  const float rcp = __frcp_rn(d);
  const float factor = (MODE == kSsdSpatial) ? __fdiv_rn(1.f, d) : 0.f;
  const float shared_scale = (SCALE == kScaleShared) ? __ldg(ssd.scale) : 1.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int u = t + i * TPR;
    if (live && u < units_per_row) {
      float o[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      if (MODE != kSsdSpatial) div_exact4(o, d, rcp, d_ok);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (MODE == kSsdSpatial) o[e] = __fmul_rn(o[e], factor);
        if (SCALE == kScaleShared) o[e] = __fmul_rn(o[e], shared_scale);
        if (SCALE == kScaleChannel) o[e] = __fmul_rn(o[e], __ldg(ssd.scale + ssd.div_spatial.div(static_cast<uint32_t>(4 * u + e))));
      }
      st_stream(yr + u, make_float4(o[0], o[1], o[2], o[3]));
    }
  }
}

template <int MODE, int SCALE, int TPR, int NV>
void launch_norm_rows(const float* x, float* y, int64_t rows, int units, float p, float eps, const SsdScale& ssd, cudaStream_t s) {
  constexpr int BLOCK = TPR < 256 ? 256 : TPR;
  constexpr int RPB = BLOCK / TPR;
  const int64_t blocks = (rows + RPB - 1) / RPB;
  normalize_rows_kernel<MODE, SCALE, TPR, NV, BLOCK><<<static_cast<unsigned>(blocks), BLOCK, 0, s>>>(x, y, rows, units, p, eps, ssd);
}

// Rows in registers when the geometry allows; false = not launched.
template <int MODE, int SCALE>
bool try_norm_rows(const float* x, float* y, int64_t rows, int64_t dim, float p, float eps, const SsdScale& ssd, cudaStream_t s) {
  if (dim % 4 != 0 || dim / 4 > 1024 * 8 || !aligned16(x) || !aligned16(y)) return false;
  if ((rows + 7) / 8 >= (1ll << 31)) return false;
  const int units = static_cast<int>(dim / 4);
#define SB200_TRY(TPR, NV) \
  if (units <= TPR * NV) { launch_norm_rows<MODE, SCALE, TPR, NV>(x, y, rows, units, p, eps, ssd, s); return true; }
  SB200_TRY(32, 1) SB200_TRY(32, 2) SB200_TRY(32, 4) SB200_TRY(128, 4) SB200_TRY(256, 4) SB200_TRY(1024, 4) SB200_TRY(1024, 8)
#undef SB200_TRY
  return false;
}

template <int MODE, int SCALE>
void launch_colvec(const float* x, float* y, const ColWalk& cw, float p, float eps, const SsdScale& ssd, cudaStream_t s) {
  constexpr int U = 4, NB = 2;
  size_t smem = colwalk_smem(cw, sizeof(double));
  if (smem < colwalk_ring_bytes(cw, U, NB)) smem = colwalk_ring_bytes(cw, U, NB);
  static unsigned long long attr_done = 0;   // per instantiation, one bit per device
  allow_dynamic_smem(normalize_colvec_kernel<MODE, SCALE, U, NB>, 1024 * U * NB * 16, &attr_done);
  normalize_colvec_kernel<MODE, SCALE, U, NB><<<cw.grid, cw.threads, smem, s>>>(x, y, cw, p, eps, ssd);
}

struct PlaneGeo {
  int64_t outer, inner, ntile;
  int dim, W, G, P, T;
  unsigned grid;
};

int plan_plane(int64_t outer, int64_t dim, int64_t inner, PlaneGeo* q) {
  if (dim >= (1ll << 31)) return SB200_ERR_UNSUPPORTED;
  q->outer = outer, q->inner = inner, q->dim = static_cast<int>(dim);
  q->W = static_cast<int>(inner < 256 ? inner : 256);
  q->ntile = (inner + q->W - 1) / q->W;
  // 512-thread blocks when every thread still gets full batches of rows, else 256
  q->T = (dim >= 256 && dim >= 16 * (512 / q->W)) ? 512 : 256;
  // row groups: as many as leave each thread about 16 rows; the rest of the block packs planes
  int G = q->T / q->W;
  const int g16 = static_cast<int>((dim + 15) / 16);
  if (G > g16) G = g16;
  int P = q->T / (G * q->W);
  if (P > outer) P = static_cast<int>(outer);
  q->G = G, q->P = P;
  const int64_t blocks = ((outer + P - 1) / P) * q->ntile;
  if (blocks >= (1ll << 31)) return SB200_ERR_UNSUPPORTED;
  q->grid = static_cast<unsigned>(blocks);
  return SB200_OK;
}

template <int MODE, int SCALE>
void launch_plane(const float* x, float* y, const PlaneGeo& q, float p, float eps, const SsdScale& ssd, cudaStream_t s) {
  if (q.T == 512)
    normalize_plane_kernel<MODE, 512, 16, SCALE><<<q.grid, 512, 0, s>>>(x, y, q.outer, q.dim, q.inner, q.W, q.G, q.P, q.ntile, p, eps, ssd);
  else
    normalize_plane_kernel<MODE, 256, 8, SCALE><<<q.grid, 256, 0, s>>>(x, y, q.outer, q.dim, q.inner, q.W, q.G, q.P, q.ntile, p, eps, ssd);
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" int sb200_normalize(const float* x, float* y, int64_t outer, int64_t dim, int64_t inner, float p,
                               float eps, void* stream) {
  if (outer < 0 || dim < 1 || inner < 1) return SB200_ERR_BAD_ARGUMENT;
  if (outer == 0) return SB200_OK;
  if (x == nullptr || y == nullptr) return SB200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 3u) return SB200_ERR_BAD_ARGUMENT;
  if (dim >= (1ll << 31) || outer * dim > (1ll << 40) / inner) return SB200_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const SsdScale none{nullptr, FastDiv32()};
  ColWalk cw;
  if (inner == 1) {
    const bool done = (p == 1.f)   ? try_norm_rows<kNormL1, kScaleNone>(x, y, outer, dim, p, eps, none, s)
                      : (p == 2.f) ? try_norm_rows<kNormL2, kScaleNone>(x, y, outer, dim, p, eps, none, s)
                                   : try_norm_rows<kNormLp, kScaleNone>(x, y, outer, dim, p, eps, none, s);
    if (done) return after_launch("sb200_normalize");
  } else if (plan_colwalk(x, y, outer, dim, inner, &cw)) {
    if (p == 1.f) launch_colvec<kNormL1, kScaleNone>(x, y, cw, p, eps, none, s);
    else if (p == 2.f) launch_colvec<kNormL2, kScaleNone>(x, y, cw, p, eps, none, s);
    else launch_colvec<kNormLp, kScaleNone>(x, y, cw, p, eps, none, s);
    return after_launch("sb200_normalize");
  }
  PlaneGeo geo;
  const int rc = plan_plane(outer, dim, inner, &geo);
  if (rc != SB200_OK) return rc;
  if (p == 1.f) launch_plane<kNormL1, kScaleNone>(x, y, geo, p, eps, none, s);
  else if (p == 2.f) launch_plane<kNormL2, kScaleNone>(x, y, geo, p, eps, none, s);
  else launch_plane<kNormLp, kScaleNone>(x, y, geo, p, eps, none, s);
  return after_launch("sb200_normalize");
}

extern "C" int sb200_ssd_normalize(const float* x, float* y, int64_t batch, int64_t channels, int64_t spatial,
                                   int across_spatial, float eps, const float* scale, int channel_shared, void* stream) {
  if (batch < 0 || channels < 1 || spatial < 1) return SB200_ERR_BAD_ARGUMENT;
  if (batch == 0) return SB200_OK;
  if (x == nullptr || y == nullptr) return SB200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(scale)) & 3u)
    return SB200_ERR_BAD_ARGUMENT;
  if (channels * spatial >= (1ll << 31)) return SB200_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const SsdScale ssd{scale, FastDiv32(static_cast<uint32_t>(spatial))};
  const int sm = scale == nullptr ? kScaleNone : (channel_shared ? kScaleShared : kScaleChannel);
  ColWalk cw;
  if (across_spatial || spatial == 1) {
    // one norm per sample over a row of the [batch, channels*spatial] view
    const int64_t row = channels * spatial;
    bool done;
    if (across_spatial) {
      done = sm == kScaleNone     ? try_norm_rows<kSsdSpatial, kScaleNone>(x, y, batch, row, 2.f, eps, ssd, s)
             : sm == kScaleShared ? try_norm_rows<kSsdSpatial, kScaleShared>(x, y, batch, row, 2.f, eps, ssd, s)
                                  : try_norm_rows<kSsdSpatial, kScaleChannel>(x, y, batch, row, 2.f, eps, ssd, s);
    } else {
      done = sm == kScaleNone     ? try_norm_rows<kSsdChannel, kScaleNone>(x, y, batch, row, 2.f, eps, ssd, s)
             : sm == kScaleShared ? try_norm_rows<kSsdChannel, kScaleShared>(x, y, batch, row, 2.f, eps, ssd, s)
                                  : try_norm_rows<kSsdChannel, kScaleChannel>(x, y, batch, row, 2.f, eps, ssd, s);
    }
    if (done) return after_launch("sb200_ssd_normalize");
  } else if (plan_colwalk(x, y, batch, channels, spatial, &cw)) {
    if (sm == kScaleNone) launch_colvec<kSsdChannel, kScaleNone>(x, y, cw, 2.f, eps, ssd, s);
    else if (sm == kScaleShared) launch_colvec<kSsdChannel, kScaleShared>(x, y, cw, 2.f, eps, ssd, s);
    else launch_colvec<kSsdChannel, kScaleChannel>(x, y, cw, 2.f, eps, ssd, s);
    return after_launch("sb200_ssd_normalize");
  }
  PlaneGeo geo;
  // across_spatial: one norm per sample over all of [channels, spatial] (a row of the [batch, C*S]
  // view); else one norm per (sample, position) over the channels
  const int rc = across_spatial ? plan_plane(batch, channels * spatial, 1, &geo) : plan_plane(batch, channels, spatial, &geo);
  if (rc != SB200_OK) return rc;
#define SB200_SSD(MODE)                                                                  \
  if (sm == kScaleNone) launch_plane<MODE, kScaleNone>(x, y, geo, 2.f, eps, ssd, s);      \
  else if (sm == kScaleShared) launch_plane<MODE, kScaleShared>(x, y, geo, 2.f, eps, ssd, s); \
  else launch_plane<MODE, kScaleChannel>(x, y, geo, 2.f, eps, ssd, s);
  if (across_spatial) { SB200_SSD(kSsdSpatial) }
  else { SB200_SSD(kSsdChannel) }
#undef SB200_SSD
  return after_launch("sb200_ssd_normalize");
}
