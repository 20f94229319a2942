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
// Rows of 8192 .. 57344 floats are staged once in shared memory (rownorm_smem_rows_kernel); longer or
// unaligned ones take a block-per-row kernel that re-reads the row (from L2).
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
  int vec_ok;                // scale and bias are 16-byte aligned
  uint32_t groups;           // channel mode: rows cycle through `groups` groups ...
  uint32_t chan_per_group;   // ... of this many channels ...
  FastDiv32 div_spatial;     // ... of this many elements each
};

// first channel of the group that row `row` belongs to (channel mode)
__device__ __forceinline__ uint32_t channel_base(const Affine& a, int64_t row) {
  return a.mode == kAffineChannel ? static_cast<uint32_t>(row % a.groups) * a.chan_per_group : 0u;
}

// index into scale / bias of element j of a row whose group starts at channel `base`
__device__ __forceinline__ uint32_t affine_index(const Affine& a, uint32_t base, uint32_t j) {
  if (a.mode == kAffinePosition) return j;
  return base + a.div_spatial.div(j);
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

// The four terms of one float4, added as floats (pairwise) before they join the double accumulator: one
// conversion and one double addition per float4 instead of four of each.  Each pre-sum is off by at most 2^-24
// of its own size, far inside the tolerance a different addition order already needs (a float ulp of the mean).
__device__ __forceinline__ double sum4_terms(float a, float b, float c, float d) {
  return static_cast<double>(__fadd_rn(__fadd_rn(a, b), __fadd_rn(c, d)));
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
      if constexpr (W == 4) {
        acc += sum4_terms(__fmul_rn(alpha, v[i][0]), __fmul_rn(alpha, v[i][1]), __fmul_rn(alpha, v[i][2]), __fmul_rn(alpha, v[i][3]));
      } else {
#pragma unroll
        for (int e = 0; e < W; ++e) acc += static_cast<double>(__fmul_rn(alpha, v[i][e]));
      }
    }
  }
  const float mean = static_cast<float>(row_sum<TPR>(acc, red));
  acc = 0.0;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int u = t + i * TPR;
    if (live && u < units_per_row) {
#pragma unroll
      for (int e = 0; e < W; ++e) v[i][e] = __fsub_rn(v[i][e], mean);
      if constexpr (W == 4) {
        acc += sum4_terms(__fmul_rn(alpha, __fmul_rn(v[i][0], v[i][0])), __fmul_rn(alpha, __fmul_rn(v[i][1], v[i][1])),
                          __fmul_rn(alpha, __fmul_rn(v[i][2], v[i][2])), __fmul_rn(alpha, __fmul_rn(v[i][3], v[i][3])));
      } else {
#pragma unroll
        for (int e = 0; e < W; ++e) acc += static_cast<double>(__fmul_rn(alpha, __fmul_rn(v[i][e], v[i][e])));
      }
    }
  }
  const float var = static_cast<float>(row_sum<TPR>(acc, red));
  const float d = __fsqrt_rn(__fadd_rn(var, eps));
  const bool d_ok = (d >= 0x1p-60f) && (d <= 0x1p60f);
  const float rcp = __frcp_rn(d);
  const uint32_t base = channel_base(aff, row);
  // position mode with float4 units: scale and bias are read as float4 too (vec_affine: both 16-byte aligned)
  const bool vec_affine = VEC && aff.mode == kAffinePosition && aff.vec_ok;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int u = t + i * TPR;
    if (live && u < units_per_row) {
      float o[W];
      if constexpr (W == 4) {
#pragma unroll
        for (int e = 0; e < W; ++e) o[e] = v[i][e];
        div_exact4(o, d, rcp, d_ok);
      } else {
#pragma unroll
        for (int e = 0; e < W; ++e) o[e] = div_exact(v[i][e], d, rcp, d_ok);
      }
      if (vec_affine) {
        const float4 sc = __ldg(reinterpret_cast<const float4*>(aff.scale) + u), bs = __ldg(reinterpret_cast<const float4*>(aff.bias) + u);
        o[0] = __fadd_rn(__fmul_rn(o[0], sc.x), bs.x);
        o[W > 1 ? 1 : 0] = __fadd_rn(__fmul_rn(o[W > 1 ? 1 : 0], sc.y), bs.y);
        o[W > 2 ? 2 : 0] = __fadd_rn(__fmul_rn(o[W > 2 ? 2 : 0], sc.z), bs.z);
        o[W > 3 ? 3 : 0] = __fadd_rn(__fmul_rn(o[W > 3 ? 3 : 0], sc.w), bs.w);
      } else if (aff.mode != kAffineNone) {
#pragma unroll
        for (int e = 0; e < W; ++e) o[e] = affine_apply(aff, o[e], affine_index(aff, base, static_cast<uint32_t>(u * W + e)));
      }
      if (VEC) st_stream(reinterpret_cast<float4*>(y + row_off) + u, make_float4(o[0], o[W > 1 ? 1 : 0], o[W > 2 ? 2 : 0], o[W > 3 ? 3 : 0]));
      else st_stream(y + row_off + u, o[0]);
    }
  }
}

// Long rows: one block per row (grid-strided), three passes over the row; the second and third
// read come from L2 (the grid is sized so that the rows in flight fit there).  Used for rows that
// would need a 1024-thread block in the register kernel (one resident block per SM, no overlap
// of one row's load with another's arithmetic) and for rows too long for registers at all.
template <bool VEC, int T>
__global__ void __launch_bounds__(T)
rownorm_long_rows_kernel(const float* x, float* y, int64_t rows, int64_t inner, float alpha, float eps,
                         const __grid_constant__ Affine aff) {
  constexpr int W = VEC ? 4 : 1;
  __shared__ double red[32];
  const int64_t units = inner / W;
  auto load = [&](const float* xr, int64_t u, float (&v)[W]) {
    if (VEC) {
      const float4 q = *(reinterpret_cast<const float4*>(xr) + u);
      v[0] = q.x; v[W > 1 ? 1 : 0] = q.y; v[W > 2 ? 2 : 0] = q.z; v[W > 3 ? 3 : 0] = q.w;
    } else {
      v[0] = xr[u];
    }
  };
  // kB units per thread and step, loaded together so that they are in flight together
  constexpr int kB = 4;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * inner;
    float* yr = y + row * inner;
    double acc = 0.0;
    for (int64_t u0 = threadIdx.x; u0 < units; u0 += T * kB) {
      float v[kB][W];
#pragma unroll
      for (int k = 0; k < kB; ++k)
        if (u0 + k * T < units) load(xr, u0 + k * T, v[k]);
#pragma unroll
      for (int k = 0; k < kB; ++k)
        if (u0 + k * T < units) {
#pragma unroll
          for (int e = 0; e < W; ++e) acc += static_cast<double>(__fmul_rn(alpha, v[k][e]));
        }
    }
    const float mean = static_cast<float>(block_reduce(acc, OpAddD(), 0.0, red));
    acc = 0.0;
    for (int64_t u0 = threadIdx.x; u0 < units; u0 += T * kB) {
      float v[kB][W];
#pragma unroll
      for (int k = 0; k < kB; ++k)
        if (u0 + k * T < units) load(xr, u0 + k * T, v[k]);
#pragma unroll
      for (int k = 0; k < kB; ++k)
        if (u0 + k * T < units) {
#pragma unroll
          for (int e = 0; e < W; ++e) {
            const float c = __fsub_rn(v[k][e], mean);
            acc += static_cast<double>(__fmul_rn(alpha, __fmul_rn(c, c)));
          }
        }
    }
    const float var = static_cast<float>(block_reduce(acc, OpAddD(), 0.0, red));
    const float d = __fsqrt_rn(__fadd_rn(var, eps));
    const bool d_ok = (d >= 0x1p-60f) && (d <= 0x1p60f);
    const float rcp = __frcp_rn(d);
    const uint32_t base = channel_base(aff, row);
    for (int64_t u0 = threadIdx.x; u0 < units; u0 += T * kB) {
      float v[kB][W];
#pragma unroll
      for (int k = 0; k < kB; ++k)
        if (u0 + k * T < units) load(xr, u0 + k * T, v[k]);
#pragma unroll
      for (int k = 0; k < kB; ++k) {
        const int64_t u = u0 + k * T;
        if (u < units) {
          float o[W];
#pragma unroll
          for (int e = 0; e < W; ++e) o[e] = __fsub_rn(v[k][e], mean);
          if constexpr (W == 4) {
            div_exact4(o, d, rcp, d_ok);
          } else {
            o[0] = div_exact(o[0], d, rcp, d_ok);
          }
          if (aff.mode != kAffineNone) {
#pragma unroll
            for (int e = 0; e < W; ++e) o[e] = affine_apply(aff, o[e], affine_index(aff, base, static_cast<uint32_t>(u * W + e)));
          }
          if (VEC) st_stream(reinterpret_cast<float4*>(yr) + u, make_float4(o[0], o[W > 1 ? 1 : 0], o[W > 2 ? 2 : 0], o[W > 3 ? 3 : 0]));
          else st_stream(yr + u, o[0]);
        }
      }
    }
    __syncthreads();
  }
}

// Rows of 8192 .. 57344 floats (a multiple of 4, 16-byte aligned): the row is staged ONCE in shared
// memory by 16-byte asynchronous copies (all of them issued together: the whole row is in flight, no
// registers involved), the three steps read it from there, and the result goes out in 128-bit
// stores: 8 bytes of traffic per element, no second or third read through the L2.  Rows of up to
// 110 KB leave room for two blocks of 512 threads per SM, so one block's copy-in overlaps the other's
// arithmetic and stores (measured on 100 KB rows: 0.48 of 8 TB/s; one 1024-thread block per SM that
// prefetches its next row into a second buffer: 0.42; the block-per-row kernel below: 0.34); longer
// rows get one block of 1024 threads per SM.  Blocks walk the rows grid-strided.
template <int T>
__global__ void __launch_bounds__(T)
rownorm_smem_rows_kernel(const float* x, float* y, int64_t rows, int units, float alpha, float eps,
                         const __grid_constant__ Affine aff) {
  extern __shared__ float4 row_buf[];   // [units]
  __shared__ double red[32];
  const uint32_t buf0 = static_cast<uint32_t>(__cvta_generic_to_shared(row_buf));
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float4* xr = reinterpret_cast<const float4*>(x) + row * units;
    for (int u = threadIdx.x; u < units; u += T) cp_async16(buf0 + 16u * static_cast<uint32_t>(u), xr + u);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    const float4* buf = row_buf;
    float4* yr = reinterpret_cast<float4*>(y) + row * units;
    double acc = 0.0;
    for (int u = threadIdx.x; u < units; u += T) {
      const float4 q = buf[u];
      acc += sum4_terms(__fmul_rn(alpha, q.x), __fmul_rn(alpha, q.y), __fmul_rn(alpha, q.z), __fmul_rn(alpha, q.w));
    }
    const float mean = static_cast<float>(block_reduce(acc, OpAddD(), 0.0, red));
    acc = 0.0;
    for (int u = threadIdx.x; u < units; u += T) {
      const float4 q = buf[u];
      const float c0 = __fsub_rn(q.x, mean), c1 = __fsub_rn(q.y, mean), c2 = __fsub_rn(q.z, mean), c3 = __fsub_rn(q.w, mean);
      acc += sum4_terms(__fmul_rn(alpha, __fmul_rn(c0, c0)), __fmul_rn(alpha, __fmul_rn(c1, c1)),
                        __fmul_rn(alpha, __fmul_rn(c2, c2)), __fmul_rn(alpha, __fmul_rn(c3, c3)));
    }
    const float var = static_cast<float>(block_reduce(acc, OpAddD(), 0.0, red));
    const float d = __fsqrt_rn(__fadd_rn(var, eps));
    const bool d_ok = (d >= 0x1p-60f) && (d <= 0x1p60f);
    const float rcp = __frcp_rn(d);
    const uint32_t base = channel_base(aff, row);
    for (int u = threadIdx.x; u < units; u += T) {
      const float4 q = buf[u];
      float o[4] = {__fsub_rn(q.x, mean), __fsub_rn(q.y, mean), __fsub_rn(q.z, mean), __fsub_rn(q.w, mean)};
      div_exact4(o, d, rcp, d_ok);
      if (aff.mode == kAffineChannel) {
        // long rows: the four lanes of a float4 almost always share a channel - one index, one scale, one bias
        const uint32_t k0 = affine_index(aff, base, static_cast<uint32_t>(4 * u)), k3 = affine_index(aff, base, static_cast<uint32_t>(4 * u + 3));
        if (k0 == k3) {
          const float sc = __ldg(aff.scale + k0), bs = __ldg(aff.bias + k0);
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] = __fadd_rn(__fmul_rn(o[e], sc), bs);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] = affine_apply(aff, o[e], affine_index(aff, base, static_cast<uint32_t>(4 * u + e)));
        }
      } else if (aff.mode != kAffineNone) {
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = affine_apply(aff, o[e], affine_index(aff, base, static_cast<uint32_t>(4 * u + e)));
      }
      st_stream(yr + u, make_float4(o[0], o[1], o[2], o[3]));
    }
    __syncthreads();   // the buffer is free for the next row
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
  SB200_TRY(64, 4) SB200_TRY(128, 4) SB200_TRY(128, 6) SB200_TRY(128, 7) SB200_TRY(256, 4) SB200_TRY(256, 6) SB200_TRY(512, 4)
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
  aff.vec_ok = (scale != nullptr && bias != nullptr && aligned16(scale) && aligned16(bias)) ? 1 : 0;
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
  const bool vec = inner % 4 == 0 && aligned16(x) && aligned16(y);
  bool done = false;
  if (vec) done = pick_rows<true>(x, y, rows, static_cast<int>(inner / 4), alpha, eps, aff, s);
  else if (inner <= 512 * 4) done = pick_rows<false>(x, y, rows, static_cast<int>(inner), alpha, eps, aff, s);
  if (!done && vec && inner * 4 <= 224 * 1024) {
    // the row fits the shared memory of a block
    const size_t bytes = static_cast<size_t>(inner) * 4;
    static unsigned long long attr_done_512 = 0, attr_done_1024 = 0;   // one bit per device
    allow_dynamic_smem(rownorm_smem_rows_kernel<512>, 110 * 1024, &attr_done_512);
    allow_dynamic_smem(rownorm_smem_rows_kernel<1024>, 224 * 1024, &attr_done_1024);
    if (bytes <= 110 * 1024)
      rownorm_smem_rows_kernel<512><<<stream_grid(rows, 2), 512, bytes, s>>>(x, y, rows, static_cast<int>(inner / 4), alpha, eps, aff);
    else
      rownorm_smem_rows_kernel<1024><<<stream_grid(rows, 1), 1024, bytes, s>>>(x, y, rows, static_cast<int>(inner / 4), alpha, eps, aff);
    done = true;
  }
  if (!done) {
    // rows in flight (grid x row bytes) are kept near 48 MB so that the re-reads hit L2
    int64_t per_sm = (48ll << 20) / (inner * 4) / sm_count();
    per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
    const unsigned grid = stream_grid(rows, static_cast<int>(per_sm));
    // rows this long leave room for few blocks (their re-reads must stay in L2): large blocks keep the SM busy
    if (inner >= 32768) {
      if (vec) rownorm_long_rows_kernel<true, 1024><<<grid, 1024, 0, s>>>(x, y, rows, inner, alpha, eps, aff);
      else rownorm_long_rows_kernel<false, 1024><<<grid, 1024, 0, s>>>(x, y, rows, inner, alpha, eps, aff);
    } else if (vec) {
      rownorm_long_rows_kernel<true, 256><<<grid, 256, 0, s>>>(x, y, rows, inner, alpha, eps, aff);
    } else {
      rownorm_long_rows_kernel<false, 256><<<grid, 256, 0, s>>>(x, y, rows, inner, alpha, eps, aff);
    }
  }
  return after_launch("sb200_row_norm");
}
