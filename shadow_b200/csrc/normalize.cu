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
  PlaneGeo geo;
  const int rc = plan_plane(outer, dim, inner, &geo);
  if (rc != SB200_OK) return rc;
  const SsdScale none{nullptr, FastDiv32()};
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
  PlaneGeo geo;
  // across_spatial: one norm per sample over all of [channels, spatial] (a row of the [batch, C*S]
  // view); else one norm per (sample, position) over the channels
  const int rc = across_spatial ? plan_plane(batch, channels * spatial, 1, &geo) : plan_plane(batch, channels, spatial, &geo);
  if (rc != SB200_OK) return rc;
  const SsdScale ssd{scale, FastDiv32(static_cast<uint32_t>(spatial))};
  const int sm = scale == nullptr ? kScaleNone : (channel_shared ? kScaleShared : kScaleChannel);
#define SB200_SSD(MODE)                                                                  \
  if (sm == kScaleNone) launch_plane<MODE, kScaleNone>(x, y, geo, 2.f, eps, ssd, s);      \
  else if (sm == kScaleShared) launch_plane<MODE, kScaleShared>(x, y, geo, 2.f, eps, ssd, s); \
  else launch_plane<MODE, kScaleChannel>(x, y, geo, 2.f, eps, ssd, s);
  if (across_spatial) { SB200_SSD(kSsdSpatial) }
  else { SB200_SSD(kSsdChannel) }
#undef SB200_SSD
  return after_launch("sb200_ssd_normalize");
}
