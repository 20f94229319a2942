// Softmax over the middle axis of x viewed as [outer, dim, inner].
//
// The reference makes four launches and six passes over memory (max, exp, sum, divide) with a
// workspace of outer*inner floats.  Here the tensor is read once and written once, no scratch:
//   inner == 1 (rows): a row lives in the registers of TPR threads (TPR = 32..1024, up to 8 float4
//       per thread, so rows up to 32768 floats): one 128-bit read, warp-shuffle / shared-memory
//       max and sum, one 128-bit write.  Longer rows use a block-per-row kernel that re-reads the
//       row (from L2) for the second and third step.
//   inner > 1 (strided): the threads of a block tile the contiguous [dim, inner] planes as P
//       planes x G row groups x W columns (W = min(inner, 256)), so reads are contiguous for any
//       `inner`; pass 1 keeps an online (max, sum) per thread, pass 2 re-reads the patch and
//       writes.  The profiler shows the second read served by the L2 (DRAM read bytes = tensor
//       size), and the kernel bound by instruction issue and load latency rather than DRAM
//       (0.50 of 8 TB/s on [1536,1000,7,7]).  Variants that hold the patch on chip were built and
//       measured slower: the patch in shared memory filled by asynchronous copies (one 196 KB
//       block per SM: no overlap between consecutive patches, 66 instructions per element), a
//       per-thread shared-memory ring of asynchronous copies, and a cluster/DSMEM row split.
// Arithmetic: float max, expf(x - max), float sum (tree order instead of the reference's
// left-to-right order), then one correctly rounded reciprocal per row and a multiply per element
// instead of the reference's per-element division (an IEEE float division costs ~60 issue slots on
// this part and capped the row kernel; the result differs by at most 1 ulp, inside the softmax
// tolerance of 1e-5*log2(n) relative).  Algorithmic bytes: 8 per element.
#include <float.h>

#include "colwalk.cuh"
#include "common.cuh"
#include "math.cuh"

namespace sb200 {
namespace {

// Reduce `v` over the TPR consecutive threads that share a row.  `red` is shared scratch with one
// slot per warp of the block.  Every thread of the row gets the result.
template <int TPR, typename Op>
__device__ __forceinline__ float row_reduce(float v, Op op, float identity, float* red) {
  if (TPR <= 32) {
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
  } else {
    constexpr int WPR = TPR / 32;  // warps per row
    v = warp_reduce(v, op);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int first = (warp / WPR) * WPR;
    float r = (lane < WPR) ? red[first + lane] : identity;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = op(r, __shfl_xor_sync(0xffffffffu, r, o));
    return r;
  }
}

// Rows in registers.  VEC: units are float4 (dim % 4 == 0, aligned), else single floats.
// Each thread owns NV units: unit index = lane_in_row + i*TPR.
template <int TPR, int NV, bool VEC, int BLOCK>
__global__ void __launch_bounds__(BLOCK)
softmax_rows_kernel(const float* x, float* y, int64_t rows, int units_per_row) {
  constexpr int RPB = BLOCK / TPR;  // rows per block
  constexpr int W = VEC ? 4 : 1;
  __shared__ float red[BLOCK / 32];
  const int t = threadIdx.x % TPR;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * RPB + threadIdx.x / TPR;
  const bool live = row < rows;   // dead rows still take part in the barriers
  const int64_t row_off = row * static_cast<int64_t>(units_per_row) * W;
  float v[NV][W];
  float m = -FLT_MAX;
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
      for (int e = 0; e < W; ++e) m = std_max(v[i][e], m);
    }
  }
  m = row_reduce<TPR>(m, OpMaxF(), -FLT_MAX, red);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int u = t + i * TPR;
    if (live && u < units_per_row) {
#pragma unroll
      for (int e = 0; e < W; ++e) {
        v[i][e] = expf(__fsub_rn(v[i][e], m));
        sum = __fadd_rn(sum, v[i][e]);
      }
    }
  }
  sum = row_reduce<TPR>(sum, OpAddF(), 0.f, red);
  const float inv = __frcp_rn(sum);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int u = t + i * TPR;
    if (live && u < units_per_row) {
      if (VEC) {
        float4 q = make_float4(__fmul_rn(v[i][0], inv), __fmul_rn(v[i][W > 1 ? 1 : 0], inv),
                               __fmul_rn(v[i][W > 2 ? 2 : 0], inv), __fmul_rn(v[i][W > 3 ? 3 : 0], inv));
        st_stream(reinterpret_cast<float4*>(y + row_off) + u, q);
      } else {
        st_stream(y + row_off + u, __fmul_rn(v[i][0], inv));
      }
    }
  }
}

// Any row length: one block per row (grid-strided), three passes over the row.
__global__ void __launch_bounds__(256)
softmax_long_rows_kernel(const float* x, float* y, int64_t rows, int64_t dim) {
  __shared__ float red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * dim;
    float* yr = y + row * dim;
    float m = -FLT_MAX;
    for (int64_t i = threadIdx.x; i < dim; i += 256) m = std_max(xr[i], m);
    m = block_reduce(m, OpMaxF(), -FLT_MAX, red);
    float sum = 0.f;
    for (int64_t i = threadIdx.x; i < dim; i += 256) sum = __fadd_rn(sum, expf(__fsub_rn(xr[i], m)));
    sum = block_reduce(sum, OpAddF(), 0.f, red);
    const float inv = __frcp_rn(sum);
    for (int64_t i = threadIdx.x; i < dim; i += 256) yr[i] = __fmul_rn(expf(__fsub_rn(xr[i], m)), inv);
    __syncthreads();
  }
}

// Strided softmax, plane layout.  The threads of a block are laid out as P planes x G row groups
// x W columns (W = min(inner, 256)), so consecutive threads read consecutive addresses whatever
// `inner` is - no lane is wasted on a ragged `inner` such as 49 - and P > 1 packs planes too small
// to occupy a block.  Thread (p, g, s) owns rows g, g+G, ... of column s of plane p.
//   pass 1: U independent loads in flight per thread; the batch maximum is taken first and the
//       running sum re-referenced at most once per batch (the usual online-softmax rescale), so a
//       row costs one max, one subtract, one multiply, one 2^x and one add.  The sum only feeds
//       the denominator, whose tolerance is far looser than one exponential's, hence the hardware
//       2^x unit (about 2 ulp) instead of expf;
//   merge of the G row groups through shared memory: exact maximum, sums re-referenced with expf;
//   pass 2: re-reads the patch - the block read it a moment ago, and the patches in flight
//       (resident blocks x dim x W x 4 bytes) are sized to stay inside the L2, so DRAM sees one
//       read and one write per element (measured: dram read = tensor size) - and writes
//       expf(x - max) * (1/sum) with the accurate expf.
// The kernel is bound by instruction issue, not by DRAM: every element costs two address
// computations, two loads, a store and two exponentials of 4-byte granularity.
// exp(d) for d <= 0 (the softmax numerator): 2^(d*log2 e) on the hardware 2^x unit with the rounding
// error of the product d*log2 e and of the constant carried in a low word and applied as a
// first-order correction.  Measured against the double-precision exp on 2^26 arguments in
// [-100, 0]: at most 2.6 ulp (CUDA's expf: 1.9), at 8 instructions instead of about 14.  The
// argument is clamped at -150 (result 0) so that -inf does not produce inf*0; a NaN argument gives
// 0 here, which is harmless because a column holding a NaN has a NaN sum and therefore NaN outputs.
__device__ __forceinline__ float exp_nonpos(float d) {
  const float kHi = 1.4426950216293335f;      // float(log2 e)
  const float kLo = 1.9259629911266175e-8f;   // log2 e - kHi
  d = fmaxf(d, -150.f);
  const float t = __fmul_rn(d, kHi);
  float lo = __fmaf_rn(d, kHi, -t);
  lo = __fmaf_rn(d, kLo, lo);
  float r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(t));
  return __fmaf_rn(r, __fmul_rn(lo, 0.6931471805599453f), r);
}

// Idx: int32_t when a [dim, inner] plane (times the unroll) is addressable with 32-bit element
// offsets (the usual case: cheaper address arithmetic), else int64_t.
template <int T, int U, typename Idx>
__global__ void __launch_bounds__(T, 1024 / T)
softmax_plane_kernel(const float* x, float* y, int64_t outer, int dim, int64_t inner, int W, int G, int P,
                     int64_t ntile) {
  __shared__ float sm_m[T], sm_l[T];
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
  const Idx step = static_cast<Idx>(G * inner);
  const int cnt = live ? (dim - g + G - 1) / G : 0;   // rows of this thread
  constexpr float kLog2e = 1.4426950408889634f;
  auto exp2_fast = [](float d) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
    return r;
  };
  float m = -FLT_MAX, l = 0.f;
  {
    const float* p = xp;
    int k = 0;
    for (; k + U <= cnt; k += U, p += U * step) {
      float v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = p[u * step];   // default caching: stays in L2 for pass 2
      float bm = v[0];
#pragma unroll
      for (int u = 1; u < U; ++u) bm = fmaxf(bm, v[u]);
      if (bm > m) {   // new maximum: bring the running sum to the new reference point
        l = l * exp2_fast((m - bm) * kLog2e);
        m = bm;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) l = l + exp2_fast((v[u] - m) * kLog2e);
    }
    for (; k < cnt; ++k, p += step) {
      const float val = *p;
      if (val > m) {
        l = l * exp2_fast((m - val) * kLog2e);
        m = val;
      }
      l = l + exp2_fast((val - m) * kLog2e);
    }
  }
  sm_m[t] = m;
  sm_l[t] = l;
  __syncthreads();
  if (live) {
    const int first = pl * G * W + sidx;
    float M = -FLT_MAX, L = 0.f;
    for (int k = 0; k < G; ++k) M = std_max(sm_m[first + k * W], M);
    for (int k = 0; k < G; ++k) L = __fadd_rn(L, __fmul_rn(sm_l[first + k * W], expf(__fsub_rn(sm_m[first + k * W], M))));
    const float inv = __frcp_rn(L);
    const float* p = xp;
    float* q = yp;
    int k = 0;
    for (; k + U <= cnt; k += U, p += U * step, q += U * step) {
      float v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = ld_stream(p + u * step);
#pragma unroll
      for (int u = 0; u < U; ++u) st_stream(q + u * step, __fmul_rn(exp_nonpos(__fsub_rn(v[u], M)), inv));
    }
    for (; k < cnt; ++k, p += step, q += step) st_stream(q, __fmul_rn(exp_nonpos(__fsub_rn(ld_stream(p), M)), inv));
  }
}

// ---- exponentials against an integer reference ---------------------------------------------------
// softmax is invariant under a common shift of a column, and in the base-2 domain any shift works
// as long as sum and numerators use it alike.  The kernels below therefore never subtract a float
// maximum: a column's reference is an INTEGER c (about log2(e) * max), a term is
// 2^(x*log2(e) - c) - one fused multiply-add and one pass through the hardware 2^x unit - and
// partial sums taken against different references are brought together by exact powers of two.
// Error of a term: the fused multiply-add rounds once at magnitude |x*log2(e) - c| (below 2^-19
// absolute for the terms that matter, 6.6e-7 relative in the result) plus the unit's 2^-22: under
// 1e-6 relative, a tenth of the softmax bar at its tightest (1e-5 for n = 2).  NaN stays NaN, -inf
// gives 0.  The numerators carry a bias of 2^24 that the reciprocal of the sum takes back, so that
// the unit (which flushes results below 2^-126) is exact down to 2^-150 and outputs in the
// denormal range come out right.
constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kNumeratorBias = 24.f;
__device__ __forceinline__ float ex2_ftz(float t) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}
// 2^d for an integer-valued float d <= 0, exact (0 below 2^-126).
__device__ __forceinline__ float pow2_int(float d) {
  const int k = static_cast<int>(fmaxf(d, -127.f));
  return __int_as_float((127 + k) << 23);   // k = -127 gives +0
}

// Running (reference, sum) of one lane.  `take` adds a batch of U values: the reference moves up
// (to the batch maximum, rounded to an integer) only when the batch would otherwise produce terms
// above 2^8, which after the first batch is rare; a move rescales the sum by an exact power of two.
struct LaneSum {
  float c, l;
  __device__ __forceinline__ void init() { c = -3.0e38f, l = 0.f; }
};

template <int U>
__device__ __forceinline__ void lanes_take(LaneSum (&s)[4], const float4 (&v)[U]) {
  float bm[4] = {v[0].x, v[0].y, v[0].z, v[0].w};
#pragma unroll
  for (int u = 1; u < U; ++u) bm[0] = fmaxf(bm[0], v[u].x), bm[1] = fmaxf(bm[1], v[u].y), bm[2] = fmaxf(bm[2], v[u].z), bm[3] = fmaxf(bm[3], v[u].w);
  const float over = fmaxf(fmaxf(__fmaf_rn(bm[0], kLog2eF, -s[0].c), __fmaf_rn(bm[1], kLog2eF, -s[1].c)),
                           fmaxf(__fmaf_rn(bm[2], kLog2eF, -s[2].c), __fmaf_rn(bm[3], kLog2eF, -s[3].c)));
  if (over > 8.f) {   // one branch per batch; rarely taken after a thread's first batch
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // never move down: a batch of small values must not blow the sum up
      const float cn = fmaxf(s[e].c, rintf(fminf(__fmul_rn(bm[e], kLog2eF), 3.0e38f)));
      s[e].l = __fmul_rn(s[e].l, pow2_int(__fsub_rn(s[e].c, cn)));
      s[e].c = cn;
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    s[0].l = __fadd_rn(s[0].l, ex2_ftz(__fmaf_rn(v[u].x, kLog2eF, -s[0].c)));
    s[1].l = __fadd_rn(s[1].l, ex2_ftz(__fmaf_rn(v[u].y, kLog2eF, -s[1].c)));
    s[2].l = __fadd_rn(s[2].l, ex2_ftz(__fmaf_rn(v[u].z, kLog2eF, -s[2].c)));
    s[3].l = __fadd_rn(s[3].l, ex2_ftz(__fmaf_rn(v[u].w, kLog2eF, -s[3].c)));
  }
}

// Strided softmax on the fixed-column 128-bit walk (colwalk.cuh), two passes: every load and store
// is a float4, a thread's four lanes stay on four fixed columns, offsets are 32-bit.
//   pass 1: U float4 in flight per thread; per element one fused multiply-add, one 2^x, one add
//           (lanes_take);
//   merge:  column references (maximum of the lanes' integers), every thread brings its four sums to
//           its columns' references by an exact power of two, column sums in a fixed order;
//   pass 2: the float4 again (from L2: the block read its patch a moment ago), one fused
//           multiply-add, one 2^x, one multiplication by the reciprocal of the sum, one float4 store.
template <int U>
__global__ void __launch_bounds__(1024, 1)
softmax_colvec_kernel(const float* x, float* y, const __grid_constant__ ColWalk q) {
  extern __shared__ float4 sm_dyn[];
  float* sm_c = reinterpret_cast<float*>(sm_dyn);   // [blockDim * 4]
  float* sm_l = sm_c + blockDim.x * 4;              // [blockDim * 4]
  const ColLane L = colwalk_thread(q, threadIdx.x, blockIdx.x);
  const float4* xp = reinterpret_cast<const float4*>(x) + L.first4;
  float4* yp = reinterpret_cast<float4*>(y) + L.first4;
  const uint32_t step = static_cast<uint32_t>(L.step4);   // a patch spans fewer than 2^31 float4
  const int cnt = L.cnt;
  const int full = cnt / U, rem = cnt - full * U;
  LaneSum s[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) s[e].init();
  {
    uint32_t off = 0;
    for (int b = 0; b < full; ++b, off += U * step) {
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = xp[off + u * step];   // default caching: stays in L2 for pass 2
      lanes_take<U>(s, v);
    }
    if (rem > 0) {   // last, partial batch: absent float4 read as -inf (their 2^x is 0)
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        v[u] = (u < rem) ? xp[off + u * step] : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
      lanes_take<U>(s, v);
    }
  }
  if (L.slot >= 0) *reinterpret_cast<float4*>(sm_c + L.slot) = make_float4(s[0].c, s[1].c, s[2].c, s[3].c);
  __syncthreads();
  colwalk_merge(q, sm_c, OpMaxF(), -3.0e38f);   // column references, left in row 0
  __syncthreads();
  float c[4];
  if (L.slot >= 0) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      c[e] = sm_c[L.plane_base + colwalk_col(q, L, e)];
      sm_l[L.slot + e] = __fmul_rn(s[e].l, pow2_int(__fsub_rn(s[e].c, c[e])));
    }
  }
  __syncthreads();
  colwalk_merge(q, sm_l, OpAddF(), 0.f);   // column sums, left in row 0
  __syncthreads();
  if (cnt == 0) return;
  float inv[4], k[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    inv[e] = __fmul_rn(__frcp_rn(sm_l[L.plane_base + colwalk_col(q, L, e)]), 0x1p-24f);   // takes the bias back
    k[e] = __fsub_rn(kNumeratorBias, c[e]);
  }
  auto out4 = [&](const float4& v) {
    return make_float4(__fmul_rn(ex2_ftz(__fmaf_rn(v.x, kLog2eF, k[0])), inv[0]), __fmul_rn(ex2_ftz(__fmaf_rn(v.y, kLog2eF, k[1])), inv[1]),
                       __fmul_rn(ex2_ftz(__fmaf_rn(v.z, kLog2eF, k[2])), inv[2]), __fmul_rn(ex2_ftz(__fmaf_rn(v.w, kLog2eF, k[3])), inv[3]));
  };
  uint32_t off = 0;
  for (int b = 0; b < full; ++b, off += U * step) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = ld_stream(xp + (off + u * step));
#pragma unroll
    for (int u = 0; u < U; ++u) st_stream(yp + (off + u * step), out4(v[u]));
  }
  if (rem > 0) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (u < rem) v[u] = ld_stream(xp + (off + u * step));
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (u < rem) st_stream(yp + (off + u * step), out4(v[u]));
  }
}

// Strided softmax with the block's patch held in registers (fixed-column walk, at most NV float4 per
// thread, blocks of 512 threads or fewer so that two or more share an SM): the tensor is read ONCE -
// no second pass over L2 - and each exponential is computed once, for the sum and for the output
// alike.  All of a thread's loads are issued before the first is used: NV*16 bytes per thread in flight.
//   1. load; per-lane maximum; column maxima through shared memory;
//   2. e = 2^24 * 2^(x*log2(e) - c), c the column's integer reference, kept in the registers; per-lane
//      sums; column sums -> reciprocal (which takes the 2^24 back);
//   3. e * (1/sum), one float4 store per float4.
// Combining a column's partials: tiled layouts with 8 row groups or fewer read the other groups'
// partials of their own four columns directly (one 128-bit shared-memory load per group, no second
// barrier); the others go through colwalk_merge.
template <typename Op>
__device__ __forceinline__ float4 colreg_combine(const ColWalk& q, const ColLane& L, float* sm, const float4& mine, Op op,
                                                 float identity) {
  if (L.slot >= 0) *reinterpret_cast<float4*>(sm + L.slot) = mine;
  __syncthreads();
  float4 r = make_float4(identity, identity, identity, identity);
  if (q.tiled && q.R <= 8) {
    if (L.slot >= 0) {
      const float* col = sm + L.col0;   // [R][4*W4]: this thread's four columns, row group g at g*ncols
      r = *reinterpret_cast<const float4*>(col);
      for (int g = 1; g < q.R; ++g) {
        const float4 o = *reinterpret_cast<const float4*>(col + g * q.ncols);
        r.x = op(r.x, o.x), r.y = op(r.y, o.y), r.z = op(r.z, o.z), r.w = op(r.w, o.w);
      }
    }
    return r;
  }
  colwalk_merge(q, sm, op, identity);
  __syncthreads();
  if (L.slot >= 0) {
    const float* p = sm + L.plane_base;
    r = make_float4(p[colwalk_col(q, L, 0)], p[colwalk_col(q, L, 1)], p[colwalk_col(q, L, 2)], p[colwalk_col(q, L, 3)]);
  }
  return r;
}

template <int NV>
__global__ void __launch_bounds__(512, 2)
softmax_colreg_kernel(const float* x, float* y, const __grid_constant__ ColWalk q) {
  extern __shared__ float4 sm_dyn[];
  float* sm_m = reinterpret_cast<float*>(sm_dyn);   // [blockDim * 4]
  float* sm_l = sm_m + blockDim.x * 4;              // [blockDim * 4]
  const ColLane L = colwalk_thread(q, threadIdx.x, blockIdx.x);
  const float4* xp = reinterpret_cast<const float4*>(x) + L.first4;
  const uint32_t step = static_cast<uint32_t>(L.step4);   // a patch spans fewer than 2^31 float4
  const int cnt = L.cnt;   // <= NV; the guards below are uniform across a warp except at a patch's edge
  float4 v[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i)
    if (i < cnt) v[i] = ld_stream(xp + i * step);
  float4 m = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (i < cnt) m.x = fmaxf(m.x, v[i].x), m.y = fmaxf(m.y, v[i].y), m.z = fmaxf(m.z, v[i].z), m.w = fmaxf(m.w, v[i].w);
  }
  m = colreg_combine(q, L, sm_m, m, OpMaxF(), -FLT_MAX);
  // integer reference of each column, with the numerators' bias folded in
  const float4 k = make_float4(__fsub_rn(kNumeratorBias, rintf(__fmul_rn(m.x, kLog2eF))), __fsub_rn(kNumeratorBias, rintf(__fmul_rn(m.y, kLog2eF))),
                               __fsub_rn(kNumeratorBias, rintf(__fmul_rn(m.z, kLog2eF))), __fsub_rn(kNumeratorBias, rintf(__fmul_rn(m.w, kLog2eF))));
  float4 l = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (i < cnt) {
      v[i].x = ex2_ftz(__fmaf_rn(v[i].x, kLog2eF, k.x)), v[i].y = ex2_ftz(__fmaf_rn(v[i].y, kLog2eF, k.y));
      v[i].z = ex2_ftz(__fmaf_rn(v[i].z, kLog2eF, k.z)), v[i].w = ex2_ftz(__fmaf_rn(v[i].w, kLog2eF, k.w));
      l.x = __fadd_rn(l.x, v[i].x), l.y = __fadd_rn(l.y, v[i].y), l.z = __fadd_rn(l.z, v[i].z), l.w = __fadd_rn(l.w, v[i].w);
    }
  }
  l = colreg_combine(q, L, sm_l, l, OpAddF(), 0.f);
  if (cnt == 0) return;
  // the sums carry the numerators' bias, so their reciprocals take it back
  const float4 inv = make_float4(__frcp_rn(l.x), __frcp_rn(l.y), __frcp_rn(l.z), __frcp_rn(l.w));
  float4* yp = reinterpret_cast<float4*>(y) + L.first4;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (i < cnt)
      st_stream(yp + i * step, make_float4(__fmul_rn(v[i].x, inv.x), __fmul_rn(v[i].y, inv.y), __fmul_rn(v[i].z, inv.z),
                                           __fmul_rn(v[i].w, inv.w)));
  }
}

// ---- strided softmax with the plane resident in shared memory, planes pipelined through it -------
// For planes of about 100..200 KB (too long a column for a block's registers, e.g. [1000,7,7]): ONE
// persistent block per SM keeps the whole plane in shared memory, cut into chunks of 5 * tact float4
// (tact = k periods of the fixed-column walk, so thread t owns float4 t, t + tact, ... of every chunk
// and its four lanes stay on four columns).  The chunks are brought in by bulk asynchronous copies
// (cp.async.bulk global -> shared, one block's own memory only, completion counted on one mbarrier per chunk; no
// registers involved), so the tensor is read from DRAM once and never re-read through the L2:
//   pass 1 takes the chunks in order as they land (running sums against integer references,
//          lanes_take), the column references and sums meet through shared memory;
//   pass 2 reads chunk c from shared memory, writes its outputs with 128-bit stores and, after a
//          block barrier, hands the chunk's memory to the copy of chunk c of the block's NEXT plane:
//          the next plane streams in while this one streams out, and its pass 1 finds all but the
//          last chunks already there.
// Every wait on an mbarrier is bounded: a wait that runs out (it never should: the copies were
// issued by this block) raises a flag that sb200_softmax_ring_timeouts() reports, and the block
// stops after giving its outstanding copies one more bounded wait.
__device__ unsigned int g_ring_timeouts = 0;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false when the phase did not complete within about half a second (2^30 SM clocks).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity))
    if (clock64() - start > (1ll << 30)) return false;
  return true;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

constexpr int kRingM = 5;   // float4 per thread and chunk

struct RingGeo {
  int64_t outer, plane4;   // planes; float4 per plane
  int tact;                // working threads; a chunk holds kRingM * tact float4 (thread t owns float4 t, t + tact, ...)
  int chunks;              // chunks per plane (the last one may be partial)
  int R, ncols;            // partial rows per column held by the block (k * rows per period); columns (inner)
  FastDiv32 div_inner;
  ColWalk merge;           // what colwalk_merge needs: one plane, R partial rows of ncols columns
};

template <int T>
__global__ void __launch_bounds__(T, 1)
softmax_ring_kernel(const float* x, float* y, const __grid_constant__ RingGeo g) {
  extern __shared__ float4 sm_dyn[];
  float4* ring = sm_dyn;                                                    // [chunks][kRingM * tact]
  float* sm_c = reinterpret_cast<float*>(ring + static_cast<size_t>(g.chunks) * kRingM * g.tact);   // [4 * tact]
  float* sm_l = sm_c + 4 * g.tact;                                          // [4 * tact]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm_l + 4 * g.tact);          // [chunks]
  __shared__ int give_up;
  const int t = threadIdx.x;
  const uint32_t ring_addr = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
  const uint32_t bar_addr = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  const int chunk4 = kRingM * g.tact;
  const uint32_t chunk_bytes = static_cast<uint32_t>(chunk4) * 16u;
  auto bytes_of = [&](int c) {   // the last chunk of a plane may be short
    const int64_t left = g.plane4 - static_cast<int64_t>(c) * chunk4;
    return left >= chunk4 ? chunk_bytes : static_cast<uint32_t>(left) * 16u;
  };
  auto fetch = [&](int64_t plane, int c) {   // one thread: announce the bytes, start the copy
    const uint32_t bar = bar_addr + 8u * static_cast<uint32_t>(c), bytes = bytes_of(c);
    mbar_expect_tx(bar, bytes);
    bulk_copy_g2s(ring_addr + static_cast<uint32_t>(c) * chunk_bytes,
                  reinterpret_cast<const float4*>(x) + plane * g.plane4 + static_cast<int64_t>(c) * chunk4, bytes, bar);
  };
  if (t == 0) {
    give_up = 0;
    for (int c = 0; c < g.chunks; ++c) mbar_init(bar_addr + 8u * static_cast<uint32_t>(c), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (t == 0 && blockIdx.x < g.outer)
    for (int c = 0; c < g.chunks; ++c) fetch(blockIdx.x, c);
  // this thread's place in the column bookkeeping (flat layout, one plane per block)
  const bool worker = t < g.tact;
  uint32_t row_unused, rem0;
  g.div_inner.divmod(static_cast<uint32_t>(4 * (worker ? t : 0)), row_unused, rem0);
  int col[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    col[e] = static_cast<int>(rem0) + e;
    if (col[e] >= g.ncols) col[e] -= g.ncols;
  }
  const ColWalk& q = g.merge;
  uint32_t parity = 0;
  bool failed = false;
  for (int64_t plane = blockIdx.x; plane < g.outer; plane += gridDim.x, parity ^= 1u) {
    // ---- pass 1: chunks in order, as they land
    LaneSum s[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) s[e].init();
    for (int c = 0; c < g.chunks && !failed; ++c) {
      if (!mbar_wait(bar_addr + 8u * static_cast<uint32_t>(c), parity)) { failed = true; break; }
      float4 v[kRingM];
#pragma unroll
      for (int u = 0; u < kRingM; ++u) {
        const int j = u * g.tact + t;   // float4 inside the chunk
        v[u] = (worker && static_cast<int64_t>(c) * chunk4 + j < g.plane4)
                   ? ring[static_cast<size_t>(c) * chunk4 + j]
                   : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);   // absent: 2^x of -inf is 0
      }
      if (worker) lanes_take<kRingM>(s, v);
    }
    if (failed) give_up = 1;   // (every thread that saw it writes the same value)
    __syncthreads();
    if (give_up) break;
    // ---- column references and sums through shared memory (as in softmax_colvec_kernel)
    if (worker) *reinterpret_cast<float4*>(sm_c + 4 * t) = make_float4(s[0].c, s[1].c, s[2].c, s[3].c);
    __syncthreads();
    colwalk_merge(q, sm_c, OpMaxF(), -3.0e38f);
    __syncthreads();
    float cref[4];
    if (worker) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        cref[e] = sm_c[col[e]];
        sm_l[4 * t + e] = __fmul_rn(s[e].l, pow2_int(__fsub_rn(s[e].c, cref[e])));
      }
    }
    __syncthreads();
    colwalk_merge(q, sm_l, OpAddF(), 0.f);
    __syncthreads();
    float inv[4], k[4];
    if (worker) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        inv[e] = __fmul_rn(__frcp_rn(sm_l[col[e]]), 0x1p-24f);   // takes the numerators' bias back
        k[e] = __fsub_rn(kNumeratorBias, cref[e]);
      }
    }
    // ---- pass 2: out of shared memory; each chunk's memory goes to the next plane as soon as it is done
    const int64_t next = plane + gridDim.x;
    float4* yp = reinterpret_cast<float4*>(y) + plane * g.plane4;
    for (int c = 0; c < g.chunks; ++c) {
      if (worker) {
        float4 v[kRingM];
#pragma unroll
        for (int u = 0; u < kRingM; ++u) v[u] = ring[static_cast<size_t>(c) * chunk4 + u * g.tact + t];   // (stale bytes past the plane's end are not stored)
#pragma unroll
        for (int u = 0; u < kRingM; ++u) {
          const int64_t i4 = static_cast<int64_t>(c) * chunk4 + u * g.tact + t;
          if (i4 < g.plane4)
            st_stream(yp + i4, make_float4(__fmul_rn(ex2_ftz(__fmaf_rn(v[u].x, kLog2eF, k[0])), inv[0]), __fmul_rn(ex2_ftz(__fmaf_rn(v[u].y, kLog2eF, k[1])), inv[1]),
                                           __fmul_rn(ex2_ftz(__fmaf_rn(v[u].z, kLog2eF, k[2])), inv[2]), __fmul_rn(ex2_ftz(__fmaf_rn(v[u].w, kLog2eF, k[3])), inv[3])));
        }
      }
      if (next < g.outer) {
        __syncthreads();   // every thread has read chunk c
        if (t == 0) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // order the reads before the copy that overwrites them
          fetch(next, c);
        }
      }
    }
  }
  if (give_up) {
    // copies of this block may still be in flight: give each one more bounded wait, then report
    if (t == 0) {
      for (int c = 0; c < g.chunks; ++c) mbar_wait(bar_addr + 8u * static_cast<uint32_t>(c), parity);
      atomicAdd(&g_ring_timeouts, 1u);
    }
  }
}

// Plans the resident-plane kernel; false when it does not apply.
bool plan_ring(const void* x, const void* y, int64_t outer, int64_t dim, int64_t inner, RingGeo* g, size_t* smem) {
  if (!aligned16(x) || !aligned16(y) || (dim * inner) % 4 != 0 || inner < 2) return false;
  const int64_t plane4 = dim * inner / 4;
  const int64_t g4 = (inner % 4 == 0) ? 4 : ((inner % 2 == 0) ? 2 : 1);
  const int64_t p = inner / g4;
  const int rp = static_cast<int>(4 / g4);
  if (p > 512 || plane4 * 16 < 96 * 1024 || outer < 2ll * sm_count()) return false;
  const int64_t k = 512 / p;
  const int64_t tact = k * p;
  const int64_t chunks = (plane4 + kRingM * tact - 1) / (kRingM * tact);
  const size_t bytes = static_cast<size_t>(chunks) * kRingM * tact * 16 + 2 * 4 * tact * sizeof(float) + static_cast<size_t>(chunks) * 8;
  if (bytes > 226 * 1024 || chunks > 4096) return false;
  g->outer = outer, g->plane4 = plane4, g->tact = static_cast<int>(tact), g->chunks = static_cast<int>(chunks);
  g->R = static_cast<int>(k) * rp, g->ncols = static_cast<int>(inner);
  g->div_inner = FastDiv32(static_cast<uint32_t>(inner));
  g->merge = ColWalk{};
  g->merge.tiled = 0, g->merge.P = 1, g->merge.tact = g->tact, g->merge.ncols = g->ncols, g->merge.R = g->R;
  g->merge.lpc_shift = g->R >= 8 ? 3 : (g->R >= 4 ? 2 : (g->R >= 2 ? 1 : 0));
  g->merge.div_ncols = FastDiv32(static_cast<uint32_t>(inner));
  *smem = bytes;
  return true;
}

template <int NV>
void launch_colreg(const float* x, float* y, const ColWalk& cw, size_t smem, cudaStream_t s) {
  softmax_colreg_kernel<NV><<<cw.grid, cw.threads, smem, s>>>(x, y, cw);
}

template <int TPR, int NV, bool VEC>
void launch_rows(const float* x, float* y, int64_t rows, int units, cudaStream_t s) {
  constexpr int BLOCK = TPR < 256 ? 256 : TPR;
  constexpr int RPB = BLOCK / TPR;
  const int64_t blocks = (rows + RPB - 1) / RPB;
  softmax_rows_kernel<TPR, NV, VEC, BLOCK><<<static_cast<unsigned>(blocks), BLOCK, 0, s>>>(x, y, rows, units);
}

template <bool VEC>
bool pick_rows(const float* x, float* y, int64_t rows, int units, cudaStream_t s) {
  // smallest TPR whose per-thread unit count fits; NV rounded up to 1, 2, 4 or 8
#define SB200_TRY(TPR, NV) \
  if (units <= TPR * NV) { launch_rows<TPR, NV, VEC>(x, y, rows, units, s); return true; }
  SB200_TRY(32, 1) SB200_TRY(32, 2) SB200_TRY(32, 4)
  SB200_TRY(64, 4) SB200_TRY(128, 4) SB200_TRY(256, 4) SB200_TRY(512, 4) SB200_TRY(1024, 4)
  SB200_TRY(1024, 8)
#undef SB200_TRY
  return false;
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" long long sb200_softmax_ring_timeouts(void) {
  unsigned int n = 0;
  if (cudaMemcpyFromSymbol(&n, g_ring_timeouts, sizeof(n)) != cudaSuccess) return -1;
  return static_cast<long long>(n);
}

extern "C" int sb200_softmax(const float* x, float* y, int64_t outer, int64_t dim, int64_t inner,
                             void* stream) {
  if (outer < 0 || dim < 1 || inner < 1) return SB200_ERR_BAD_ARGUMENT;
  if (outer == 0) return SB200_OK;
  if (x == nullptr || y == nullptr) return SB200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 3u) return SB200_ERR_BAD_ARGUMENT;
  if (outer * dim > (1ll << 40) / inner) return SB200_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (inner == 1) {
    const int64_t rows = outer;
    if (rows >= (1ll << 31)) return SB200_ERR_UNSUPPORTED;
    bool done = false;
    if (dim % 4 == 0 && aligned16(x) && aligned16(y) && dim / 4 <= 1024 * 8)
      done = pick_rows<true>(x, y, rows, static_cast<int>(dim / 4), s);
    else if (dim <= 1024 * 8)
      done = pick_rows<false>(x, y, rows, static_cast<int>(dim), s);
    if (!done) {
      const unsigned grid = stream_grid(rows, 8);
      softmax_long_rows_kernel<<<grid, 256, 0, s>>>(x, y, rows, dim);
    }
    return after_launch("sb200_softmax");
  }
  if (dim >= (1ll << 31)) return SB200_ERR_UNSUPPORTED;
  ColWalk cw;
  if (plan_colwalk(x, y, outer, dim, inner, &cw, kWalkResident, 12)) {
    // the patch fits the registers of a block: one read, one write
    const size_t smem = 2 * colwalk_smem(cw, sizeof(float));
    const int64_t share = cw.tiled ? cw.dim : cw.plane4 / cw.period4;   // rows or periods per block
    const int64_t per_step = cw.tiled ? cw.G : cw.tact / cw.period4;
    const int64_t most = (share + per_step - 1) / per_step;
    if (most <= 4) launch_colreg<4>(x, y, cw, smem, s);
    else if (most <= 8) launch_colreg<8>(x, y, cw, smem, s);
    else launch_colreg<12>(x, y, cw, smem, s);
    return after_launch("sb200_softmax");
  }
  {
    RingGeo rg;
    size_t ring_smem = 0;
    if (plan_ring(x, y, outer, dim, inner, &rg, &ring_smem)) {
      static unsigned long long attr_done = 0;   // one bit per device
      allow_dynamic_smem(softmax_ring_kernel<512>, 226 * 1024, &attr_done);
      softmax_ring_kernel<512><<<stream_grid(outer, 1), 512, ring_smem, s>>>(x, y, rg);
      return after_launch("sb200_softmax");
    }
  }
  if (plan_colwalk(x, y, outer, dim, inner, &cw)) {
    softmax_colvec_kernel<6><<<cw.grid, cw.threads, 2 * colwalk_smem(cw, sizeof(float)), s>>>(x, y, cw);
    return after_launch("sb200_softmax");
  }
  const int W = static_cast<int>(inner < 256 ? inner : 256);
  const int64_t ntile = (inner + W - 1) / W;
  // block size: 512 threads when every thread still gets full batches of rows, else 256
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
  const int rows_per_thread = static_cast<int>(dim / G);
  const int d = static_cast<int>(dim);
  const bool small = dim * inner < (1ll << 27);   // 16 rows' worth of offsets still fit 32 bits
#define SB200_PLANE(TT, UU)                                                                                  \
  do {                                                                                                       \
    if (small) softmax_plane_kernel<TT, UU, int32_t><<<grid, TT, 0, s>>>(x, y, outer, d, inner, W, G, P, ntile); \
    else softmax_plane_kernel<TT, UU, int64_t><<<grid, TT, 0, s>>>(x, y, outer, d, inner, W, G, P, ntile);   \
  } while (0)
  if (T == 512) SB200_PLANE(512, 16);
  else if (rows_per_thread >= 16) SB200_PLANE(256, 16);
  else SB200_PLANE(256, 4);
#undef SB200_PLANE
  return after_launch("sb200_softmax");
}
