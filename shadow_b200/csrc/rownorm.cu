// Row normalisation shared by LayerNorm, GroupNorm and InstanceNorm: x viewed as [rows, inner]
// (contiguous rows),
//     mean = sum(alpha*x), v = x - mean, var = sum(alpha*v*v), y = v / sqrt(var + eps)
// with alpha = 1/inner, optionally followed by y*scale[k] + bias[k] (k = position in the row for
// LayerNorm, the channel for GroupNorm / InstanceNorm).
//
// The reference runs this as Set + Sgemv + SubtractMeanAndSquare + Sgemv + DivideVariance
// (+ ScaleBias): six launches, about 36 bytes of traffic per element and a scratch of
// count + inner + 2*rows floats.  Here a row lives in the registers of TPR threads: one 128-bit
// read, three in-register steps, one 128-bit write, no scratch: 8 algorithmic bytes per element.
// Rows longer than 32768 floats take a block-per-row kernel that re-reads the row (from L2).
// Arithmetic follows the reference CPU term by term: every term alpha*x (and alpha*(v*v)) is
// rounded to float and accumulated in double (Blas::BlasSgemv on the CPU), mean and variance
// are rounded to float, the quotient is the correctly rounded float division, scale and bias are
// a separately rounded multiply and add.  Only the order of the double additions differs.
#include <float.h>

#include "common.cuh"
#include "math.cuh"

namespace sb200 {
namespace {

enum { kAffineNone = 0, kAffinePosition = 1, kAffineChannel = 2 };

struct Affine {
  const float* scale;
  const float* bias;
  int mode;
  uint32_t groups;           // channel mode: rows cycle through `groups` groups ...
  uint32_t chan_per_group;   // ... of this many channels ...
  FastDiv32 div_spatial;     // ... of this many elements each
};

// index into scale / bias of element j of row `row`
__device__ __forceinline__ uint32_t affine_index(const Affine& a, int64_t row, uint32_t j) {
  if (a.mode == kAffinePosition) return j;
  return static_cast<uint32_t>(row % a.groups) * a.chan_per_group + a.div_spatial.div(j);
}

__device__ __forceinline__ float affine_apply(const Affine& a, float v, uint32_t k) {
  return __fadd_rn(__fmul_rn(v, __ldg(a.scale + k)), __ldg(a.bias + k));
}

// Sum of `v` over the TPR consecutive threads that share a row; every thread of the row gets it.
template <int TPR>
__device__ __forceinline__ double row_sum(double v, double* red) {
  if (TPR <= 32) {
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
  } else {
    constexpr int WPR = TPR / 32;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int first = (warp / WPR) * WPR;
    double r = (lane < WPR) ? red[first + lane] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
  }
}

// Rows in registers.  VEC: units are float4 (inner % 4 == 0, aligned), else single floats.
template <int TPR, int NV, bool VEC, int BLOCK>
__global__ void __launch_bounds__(BLOCK)
rownorm_rows_kernel(const float* x, float* y, int64_t rows, int units_per_row, float alpha, float eps,
                    const __grid_constant__ Affine aff) {
  constexpr int RPB = BLOCK / TPR;
  constexpr int W = VEC ? 4 : 1;
  __shared__ double red[BLOCK / 32];
  const int t = threadIdx.x % TPR;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * RPB + threadIdx.x / TPR;
  const bool live = row < rows;   // dead rows still take part in the barriers
  const int64_t row_off = row * static_cast<int64_t>(units_per_row) * W;
  float v[NV][W];
  double acc = 0.0;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int u = t + i * TPR;
    if (live && u < units_per_row) {
      if (VEC) {
        float4 q = ld_stream(reinterpret_cast<const float4*>(x + row_off) + u);
        v[i][0] = q.x; v[i][W > 1 ? 1 : 0] = q.y; v[i][W > 2 ? 2 : 0] = q.z; v[i][W > 3 ? 3 : 0] = q.w;
      } else {
        v[i][0] = ld_stream(x + row_off + u);
      }
#pragma unroll
      for (int e = 0; e < W; ++e) acc += static_cast<double>(__fmul_rn(alpha, v[i][e]));
    }
  }
  const float mean = static_cast<float>(row_sum<TPR>(acc, red));
  acc = 0.0;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int u = t + i * TPR;
    if (live && u < units_per_row) {
#pragma unroll
      for (int e = 0; e < W; ++e) {
        v[i][e] = __fsub_rn(v[i][e], mean);
        acc += static_cast<double>(__fmul_rn(alpha, __fmul_rn(v[i][e], v[i][e])));
      }
    }
  }
  const float var = static_cast<float>(row_sum<TPR>(acc, red));
  const float d = __fsqrt_rn(__fadd_rn(var, eps));
  const bool d_ok = (d >= 0x1p-60f) && (d <= 0x1p60f);
  const float rcp = __frcp_rn(d);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int u = t + i * TPR;
    if (live && u < units_per_row) {
      float o[W];
#pragma unroll
      for (int e = 0; e < W; ++e) {
        o[e] = div_exact(v[i][e], d, rcp, d_ok);
        if (aff.mode != kAffineNone) o[e] = affine_apply(aff, o[e], affine_index(aff, row, static_cast<uint32_t>(u * W + e)));
      }
      if (VEC) st_stream(reinterpret_cast<float4*>(y + row_off) + u, make_float4(o[0], o[W > 1 ? 1 : 0], o[W > 2 ? 2 : 0], o[W > 3 ? 3 : 0]));
      else st_stream(y + row_off + u, o[0]);
    }
  }
}

// Any row length: one block per row (grid-strided), three passes over the row.
__global__ void __launch_bounds__(256)
rownorm_long_rows_kernel(const float* x, float* y, int64_t rows, int64_t inner, float alpha, float eps,
                         const __grid_constant__ Affine aff) {
  __shared__ double red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * inner;
    float* yr = y + row * inner;
    double acc = 0.0;
    for (int64_t i = threadIdx.x; i < inner; i += 256) acc += static_cast<double>(__fmul_rn(alpha, xr[i]));
    const float mean = static_cast<float>(block_reduce(acc, OpAddD(), 0.0, red));
    acc = 0.0;
    for (int64_t i = threadIdx.x; i < inner; i += 256) {
      const float c = __fsub_rn(xr[i], mean);
      acc += static_cast<double>(__fmul_rn(alpha, __fmul_rn(c, c)));
    }
    const float var = static_cast<float>(block_reduce(acc, OpAddD(), 0.0, red));
    const float d = __fsqrt_rn(__fadd_rn(var, eps));
    const bool d_ok = (d >= 0x1p-60f) && (d <= 0x1p60f);
    const float rcp = __frcp_rn(d);
    for (int64_t i = threadIdx.x; i < inner; i += 256) {
      float o = div_exact(__fsub_rn(xr[i], mean), d, rcp, d_ok);
      if (aff.mode != kAffineNone) o = affine_apply(aff, o, affine_index(aff, row, static_cast<uint32_t>(i)));
      yr[i] = o;
    }
    __syncthreads();
  }
}

template <int TPR, int NV, bool VEC>
void launch_rows(const float* x, float* y, int64_t rows, int units, float alpha, float eps, const Affine& aff,
                 cudaStream_t s) {
  constexpr int BLOCK = TPR < 256 ? 256 : TPR;
  constexpr int RPB = BLOCK / TPR;
  const int64_t blocks = (rows + RPB - 1) / RPB;
  rownorm_rows_kernel<TPR, NV, VEC, BLOCK><<<static_cast<unsigned>(blocks), BLOCK, 0, s>>>(x, y, rows, units, alpha, eps, aff);
}

template <bool VEC>
bool pick_rows(const float* x, float* y, int64_t rows, int units, float alpha, float eps, const Affine& aff,
               cudaStream_t s) {
#define SB200_TRY(TPR, NV) \
  if (units <= TPR * NV) { launch_rows<TPR, NV, VEC>(x, y, rows, units, alpha, eps, aff, s); return true; }
  SB200_TRY(32, 1) SB200_TRY(32, 2) SB200_TRY(32, 4)
  SB200_TRY(64, 4) SB200_TRY(128, 4) SB200_TRY(256, 4) SB200_TRY(512, 4) SB200_TRY(1024, 4)
  SB200_TRY(1024, 8)
#undef SB200_TRY
  return false;
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" int sb200_row_norm(const float* x, float* y, int64_t rows, int64_t inner, float eps, const float* scale,
                              const float* bias, int affine_mode, int64_t groups, int64_t channels_per_group,
                              int64_t spatial, void* stream) {
  if (rows < 0 || inner < 1 || affine_mode < kAffineNone || affine_mode > kAffineChannel) return SB200_ERR_BAD_ARGUMENT;
  if (rows == 0) return SB200_OK;
  if (x == nullptr || y == nullptr) return SB200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 3u) return SB200_ERR_BAD_ARGUMENT;
  if (inner >= (1ll << 31) || rows >= (1ll << 31) || rows > (1ll << 40) / inner) return SB200_ERR_UNSUPPORTED;
  Affine aff;
  aff.scale = scale, aff.bias = bias, aff.mode = affine_mode, aff.groups = 1, aff.chan_per_group = 1;
  if (affine_mode != kAffineNone) {
    if (scale == nullptr || bias == nullptr) return SB200_ERR_BAD_ARGUMENT;
    if (affine_mode == kAffineChannel) {
      if (groups < 1 || channels_per_group < 1 || spatial < 1 || channels_per_group * spatial != inner ||
          groups * channels_per_group >= (1ll << 31))
        return SB200_ERR_BAD_ARGUMENT;
      aff.groups = static_cast<uint32_t>(groups), aff.chan_per_group = static_cast<uint32_t>(channels_per_group);
      aff.div_spatial = FastDiv32(static_cast<uint32_t>(spatial));
    }
  }
  const float alpha = 1.f / static_cast<float>(inner);   // the reference's 1.f / inner_num
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  bool done = false;
  if (inner % 4 == 0 && aligned16(x) && aligned16(y) && inner / 4 <= 1024 * 8)
    done = pick_rows<true>(x, y, rows, static_cast<int>(inner / 4), alpha, eps, aff, s);
  else if (inner <= 1024 * 8)
    done = pick_rows<false>(x, y, rows, static_cast<int>(inner), alpha, eps, aff, s);
  if (!done) rownorm_long_rows_kernel<<<stream_grid(rows, 8), 256, 0, s>>>(x, y, rows, inner, alpha, eps, aff);
  return after_launch("sb200_row_norm");
}
