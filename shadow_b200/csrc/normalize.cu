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

enum { kNormL1 = 1, kNormL2 = 2, kNormLp = 0 };

template <int MODE>
__device__ __forceinline__ double norm_term(float v, float p) {
  const float a = fabsf(v);
  if (MODE == kNormL1) return static_cast<double>(a);
  if (MODE == kNormL2) return static_cast<double>(__fmul_rn(a, a));
  return static_cast<double>(powf(a, p));
}

template <int MODE, int kT, int kU>
__global__ void __launch_bounds__(kT, 1024 / kT)
normalize_plane_kernel(const float* x, float* y, int64_t outer, int dim, int64_t inner, int W, int G, int P,
                       int64_t ntile, float p, float eps) {
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
  float val = static_cast<float>(sum);
  if (MODE == kNormL2) val = __fsqrt_rn(val);
  if (MODE == kNormLp) val = powf(val, __fdiv_rn(1.f, p));
  const float d = (val < eps) ? eps : val;   // std::max(val, eps)
  const bool d_ok = (d >= 0x1p-60f) && (d <= 0x1p60f);
  const float rcp = __frcp_rn(d);
  const float* q = xp;
  float* o = yp;
  int k = 0;
  for (; k + kU <= cnt; k += kU, q += kU * step, o += kU * step) {
    float v[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) v[u] = ld_stream(q + u * step);
#pragma unroll
    for (int u = 0; u < kU; ++u) st_stream(o + u * step, div_exact(v[u], d, rcp, d_ok));
  }
  for (; k < cnt; ++k, q += step, o += step) st_stream(o, div_exact(ld_stream(q), d, rcp, d_ok));
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
  const int W = static_cast<int>(inner < 256 ? inner : 256);
  const int64_t ntile = (inner + W - 1) / W;
  // 512-thread blocks when every thread still gets full batches of rows, else 256
  const int T = (dim >= 256 && dim >= 16 * (512 / W)) ? 512 : 256;
  // row groups: as many as leave each thread about 16 rows; the rest of the block packs planes
  int G = T / W;
  const int g16 = static_cast<int>((dim + 15) / 16);
  if (G > g16) G = g16;
  int P = T / (G * W);
  if (P > outer) P = static_cast<int>(outer);
  const int64_t blocks = ((outer + P - 1) / P) * ntile;
  if (blocks >= (1ll << 31)) return SB200_ERR_UNSUPPORTED;
  const unsigned grid = static_cast<unsigned>(blocks);
  const int d = static_cast<int>(dim);
#define SB200_NORM(MODE)                                                                                       \
  if (T == 512) normalize_plane_kernel<MODE, 512, 16><<<grid, 512, 0, s>>>(x, y, outer, d, inner, W, G, P, ntile, p, eps); \
  else normalize_plane_kernel<MODE, 256, 8><<<grid, 256, 0, s>>>(x, y, outer, d, inner, W, G, P, ntile, p, eps);
  if (p == 1.f) { SB200_NORM(kNormL1) }
  else if (p == 2.f) { SB200_NORM(kNormL2) }
  else { SB200_NORM(kNormLp) }
#undef SB200_NORM
  return after_launch("sb200_normalize");
}
