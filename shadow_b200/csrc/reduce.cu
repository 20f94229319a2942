// Axis reductions (Prod / Sum / Max / Min / Avg / L1 / L2 over any set of axes).
//
// Host side: drop size-1 dims, merge neighbouring dims of the same kind (reduced / kept).  What is
// left alternates between kept (K) and reduced (R) dims and picks the strategy:
//   R, K R, R K R   -> "inner-reduced" family: contiguous runs of the innermost reduced dim.
//        few elements per output  -> one warp per output (warp-shuffle tree);
//        many elements per output -> grid (splits x outputs) of blocks, block tree reduction,
//                                    cross-block partials in caller scratch + a finishing kernel.
//   R K, K R K      -> "inner-kept" family: lanes run along the contiguous kept dim, rows of the
//                      block walk the reduced dim, shared-memory combine across rows, optional
//                      split of the reduced dim over blocks (partials + finishing kernel).
//   anything deeper -> generic kernel, one block per output with mixed-radix decoding.
// No index tables exist anywhere (the reference uploads one int per reduced element per call).
//
// Arithmetic mirrors the reference CPU loops: double accumulators for Prod/Sum/Avg/L1/L2 (L2 squares
// in float first), float std::max/std::min chains from -FLT_MAX/+FLT_MAX for Max/Min (NaNs are
// skipped because they never win the comparison).  The combination ORDER differs from the
// reference's sequential loop (tree instead of left-to-right) but is fixed for a given geometry, so
// results are reproducible; double accumulation keeps the difference far below float resolution.
// Algorithmic bytes: 4*(|x| + |y|); scratch traffic is splits*outputs*8 B, negligible.
#include <float.h>

#include <cstdio>
#include <initializer_list>
#include <mutex>
#include <type_traits>

#include "colwalk.cuh"
#include "common.cuh"
#include "math.cuh"

namespace sb200 {
namespace {

constexpr int kMaxDims = 8;
constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kTargetWaves = 10;  // grids of the split kernels aim at this many waves of resident blocks
constexpr int kMinTiles = 2;      // ... but never fewer than this many tile iterations per block

// Number of reduced elements with its reciprocal (both doubles, computed on the host).
struct Divisor {
  double n, inv;
  Divisor() : n(1.0), inv(1.0) {}
  explicit Divisor(double v) : n(v), inv(1.0 / v) {}
};

// ---- per-operation arithmetic --------------------------------------------------------------------
template <int OP>
struct RedOp {
  static constexpr bool kFloatAcc = (OP == SB200_RED_MAX || OP == SB200_RED_MIN);
  using Acc = typename std::conditional<kFloatAcc, float, double>::type;
  __device__ __forceinline__ static Acc init() {
    if (OP == SB200_RED_PROD) return Acc(1);
    if (OP == SB200_RED_MAX) return Acc(-FLT_MAX);
    if (OP == SB200_RED_MIN) return Acc(FLT_MAX);
    return Acc(0);
  }
  __device__ __forceinline__ static Acc step(Acc a, float x) {
    if (OP == SB200_RED_PROD) return a * static_cast<Acc>(x);
    if (OP == SB200_RED_MAX) return (a < x) ? static_cast<Acc>(x) : a;   // std::max(val, x)
    if (OP == SB200_RED_MIN) return (x < a) ? static_cast<Acc>(x) : a;   // std::min(val, x)
    if (OP == SB200_RED_L1) return a + static_cast<Acc>(fabsf(x));
    if (OP == SB200_RED_L2) { float ax = fabsf(x); return a + static_cast<Acc>(__fmul_rn(ax, ax)); }
    return a + static_cast<Acc>(x);
  }
  __device__ __forceinline__ static Acc merge(Acc a, Acc b) {
    if (OP == SB200_RED_PROD) return a * b;
    if (OP == SB200_RED_MAX) return (a < b) ? b : a;
    if (OP == SB200_RED_MIN) return (b < a) ? b : a;
    return a + b;
  }
  __device__ __forceinline__ static float finish(Acc a, Divisor count) {
    if (OP == SB200_RED_AVG) {
      // a / n in double, correctly rounded, without the ~50-instruction division: with inv = RN(1/n)
      // from the host, q = RN(a*inv), r = a - n*q (exact in an fma), q' = RN(q + r*inv) is the
      // correctly rounded quotient (Markstein's theorem; n is a small integer, never all-ones).
      const double ad = static_cast<double>(a);
      double q = ad * count.inv;
      const double r = fma(-q, count.n, ad);
      q = fma(r, count.inv, q);
      // inf / nan sums give nan in r: fall back to the plain product for them
      return static_cast<float>(r == r ? q : ad * count.inv);
    }
    if (OP == SB200_RED_L2) return __fsqrt_rn(static_cast<float>(a));
    return static_cast<float>(a);
  }
  struct Merge {
    __device__ __forceinline__ Acc operator()(Acc a, Acc b) const { return merge(a, b); }
  };
};

// Where a block's result goes: the final float, or a double partial at part[split*n_out + out].
template <int OP, bool TO_PART>
__device__ __forceinline__ void emit(typename RedOp<OP>::Acc acc, float* y, double* part, int64_t out,
                                     int64_t split, int64_t n_out, Divisor count) {
  if (TO_PART) part[split * n_out + out] = static_cast<double>(acc);
  else y[out] = RedOp<OP>::finish(acc, count);
}

template <int OP>
__device__ __forceinline__ typename RedOp<OP>::Acc step4(typename RedOp<OP>::Acc a, const float4& v) {
  a = RedOp<OP>::step(a, v.x);
  a = RedOp<OP>::step(a, v.y);
  a = RedOp<OP>::step(a, v.z);
  return RedOp<OP>::step(a, v.w);
}

// ---- inner-reduced family: x viewed as [R0, K, R1], output k = reduce over (r0, r1) ---------------
// `units` are float4 when VEC (R1 % 4 == 0 and 16-byte aligned base), single floats otherwise.
struct GeomA {
  int64_t K;            // outputs
  uint32_t R0;          // outer reduced extent (1 if absent)
  uint32_t R1u;         // inner reduced extent in units
  int64_t row_elems;    // R1 in elements (distance between consecutive k)
  int64_t r0_stride;    // K*R1 elements
  FastDiv32 div_r1u;
  int64_t n_units;      // R0 * R1u
  int64_t chunk_units;  // units per split (block kernel)
  Divisor count;         // divisor for Avg
};

template <int OP, bool VEC, bool TO_PART>
__global__ void __launch_bounds__(kThreads)
redA_warp_kernel(const float* __restrict__ x, float* y, double* part, const __grid_constant__ GeomA g) {
  using R = RedOp<OP>;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * kThreads) >> 5;
  const uint32_t n = static_cast<uint32_t>(g.n_units);
  for (int64_t k = warp; k < g.K; k += nwarps) {
    const float* base = x + k * g.row_elems;
    typename R::Acc acc = R::init();
    for (uint32_t j0 = 0; j0 < n; j0 += 32 * kUnroll) {
      float4 v4[kUnroll];
      float v1[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const uint32_t j = j0 + u * 32 + lane;
        if (j < n) {
          uint32_t r0 = 0, c = j;
          if (g.R0 > 1) g.div_r1u.divmod(j, r0, c);
          const float* p = base + static_cast<int64_t>(r0) * g.r0_stride;
          if (VEC) v4[u] = ld_stream(reinterpret_cast<const float4*>(p) + c);
          else v1[u] = ld_stream(p + c);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const uint32_t j = j0 + u * 32 + lane;
        if (j < n) {
          if (VEC) acc = step4<OP>(acc, v4[u]);
          else acc = R::step(acc, v1[u]);
        }
      }
    }
    acc = warp_reduce(acc, typename R::Merge());
    if (lane == 0) emit<OP, TO_PART>(acc, y, part, k, 0, g.K, g.count);
  }
}

// Short rows (R0 == 1, at most 256 units per row): a block of T threads owns `rows_per_block`
// consecutive rows, i.e. one contiguous chunk of up to T*UPT units.  Phase 1 loads the chunk with
// UPT independent 128-bit loads per thread (coalesced, no per-row structure) and leaves one partial
// per unit in shared memory; phase 2 gives every row to 8 lanes that combine its partials in a
// fixed order.  Tile shapes were measured on [1024*512, 196]: double accumulators run best with
// small tiles (128 threads x 3 units: 6.1 TB/s against 4.7 TB/s for 256 x 7), float ones with 256 x 3.
template <int OP>
struct RowsTile {
  static constexpr int kT = RedOp<OP>::kFloatAcc ? 256 : 128;
  static constexpr int kUPT = 3;
  static constexpr int kUnits = kT * kUPT;
};
constexpr int kRowsMaxUnitsPerRow = 256;

template <int OP, bool VEC, bool TO_PART>
__global__ void __launch_bounds__(RowsTile<OP>::kT)
redA_rows_kernel(const float* __restrict__ x, float* y, double* part, int64_t K, int r1u,
                 int rows_per_block, Divisor count) {
  using R = RedOp<OP>;
  using Acc = typename R::Acc;
  constexpr int T = RowsTile<OP>::kT, UPT = RowsTile<OP>::kUPT;
  __shared__ Acc partial[T * UPT];
  const int t = threadIdx.x;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_block;
  const int rows = static_cast<int>((K - row0) < rows_per_block ? (K - row0) : rows_per_block);
  const int n_units = rows * r1u;
  const float* base = x + row0 * r1u * (VEC ? 4 : 1);
  float4 v4[UPT];
  float v1[UPT];
#pragma unroll
  for (int i = 0; i < UPT; ++i) {
    const int idx = i * T + t;
    if (idx < n_units) {
      if (VEC) v4[i] = ld_stream(reinterpret_cast<const float4*>(base) + idx);
      else v1[i] = ld_stream(base + idx);
    }
  }
#pragma unroll
  for (int i = 0; i < UPT; ++i) {
    const int idx = i * T + t;
    if (idx < n_units) {
      if (VEC) {
        // two independent pairs, then their merge: shorter dependency chain than four steps in a row
        const Acc lo = R::step(R::step(R::init(), v4[i].x), v4[i].y);
        const Acc hi = R::step(R::step(R::init(), v4[i].z), v4[i].w);
        partial[idx] = R::merge(lo, hi);
      } else {
        partial[idx] = R::step(R::init(), v1[i]);
      }
    }
  }
  __syncthreads();
  const int lane8 = t & 7, group = (t >> 3) & 3, warp = t >> 5;
  for (int rb = warp * 4; rb < rows; rb += (T / 32) * 4) {   // warp-uniform trip count
    const int r = rb + group;
    Acc a = R::init();
    if (r < rows) {
      const Acc* p = partial + r * r1u;
      for (int j = lane8; j < r1u; j += 8) a = R::merge(a, p[j]);
    }
    a = R::merge(a, __shfl_xor_sync(0xffffffffu, a, 4));
    a = R::merge(a, __shfl_xor_sync(0xffffffffu, a, 2));
    a = R::merge(a, __shfl_xor_sync(0xffffffffu, a, 1));
    if (r < rows && lane8 == 0) emit<OP, TO_PART>(a, y, part, row0 + r, 0, K, count);
  }
}

// grid = (K, splits).  Block (k, s) reduces units [s*chunk, (s+1)*chunk) of output k.
template <int OP, bool VEC, bool TO_PART>
__global__ void __launch_bounds__(kThreads)
redA_block_kernel(const float* __restrict__ x, float* y, double* part, const __grid_constant__ GeomA g) {
  using R = RedOp<OP>;
  __shared__ typename R::Acc smem[32];
  const int64_t k = blockIdx.x, s = blockIdx.y;
  const float* base = x + k * g.row_elems;
  const int64_t begin = s * g.chunk_units;
  int64_t end = begin + g.chunk_units;
  if (end > g.n_units) end = g.n_units;
  // One accumulator per unroll slot: the slots' chains are independent, and a full tile takes the
  // unguarded path so that its kUnroll loads are all issued before the first is consumed.
  typename R::Acc accs[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) accs[u] = R::init();
  constexpr int64_t kTile = static_cast<int64_t>(kThreads) * kUnroll;
  auto address = [&](int64_t j, int64_t* c) {
    const float* p = base;
    *c = j;
    if (g.R0 > 1) {
      uint32_t r0, cc;
      g.div_r1u.divmod(static_cast<uint32_t>(j), r0, cc);   // n_units < 2^32 whenever R0 > 1
      p += static_cast<int64_t>(r0) * g.r0_stride;
      *c = cc;
    }
    return p;
  };
  int64_t j0 = begin;
  for (; j0 + kTile <= end; j0 += kTile) {
    float4 v4[kUnroll];
    float v1[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t c;
      const float* p = address(j0 + u * kThreads + threadIdx.x, &c);
      if (VEC) v4[u] = ld_stream(reinterpret_cast<const float4*>(p) + c);
      else v1[u] = ld_stream(p + c);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (VEC) accs[u] = step4<OP>(accs[u], v4[u]);
      else accs[u] = R::step(accs[u], v1[u]);
    }
  }
  for (int64_t j = j0 + threadIdx.x; j < end; j += kThreads) {   // ragged last tile
    int64_t c;
    const float* p = address(j, &c);
    if (VEC) accs[0] = step4<OP>(accs[0], ld_stream(reinterpret_cast<const float4*>(p) + c));
    else accs[0] = R::step(accs[0], ld_stream(p + c));
  }
  typename R::Acc acc = accs[0];
#pragma unroll
  for (int u = 1; u < kUnroll; ++u) acc = R::merge(acc, accs[u]);
  acc = block_reduce(acc, typename R::Merge(), R::init(), smem);
  if (threadIdx.x == 0) emit<OP, TO_PART>(acc, y, part, k, s, g.K, g.count);
}

// ---- inner-kept family: x viewed as [K0, R, K1], output (k0, k1) = reduce over r ------------------
struct GeomB {
  int64_t K0, R, K1;    // elements
  int64_t K1u;          // K1 in units (float4 when VEC)
  int64_t nbx;          // blocks along K1
  int64_t r_chunk;      // rows per split
  int64_t n_out;        // K0*K1
  Divisor count;
};

// blockIdx.x = k0*nbx + bx, blockIdx.y = split.  TX lanes along K1, TY = kThreads/TX rows along R.
template <int OP, int TX, bool VEC, bool TO_PART>
__global__ void __launch_bounds__(kThreads)
redB_kernel(const float* __restrict__ x, float* y, double* part, const __grid_constant__ GeomB g) {
  using R = RedOp<OP>;
  using Acc = typename R::Acc;
  constexpr int TY = kThreads / TX;
  constexpr int W = VEC ? 4 : 1;
  __shared__ Acc smem[kThreads / 32][TX * W + 1];
  const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
  const int64_t k0 = blockIdx.x / g.nbx, bx = blockIdx.x - k0 * g.nbx;
  const int64_t s = blockIdx.y;
  const int64_t col = bx * TX + tx;  // unit index along K1
  const bool active = col < g.K1u;
  const int64_t r_begin = s * g.r_chunk;
  int64_t r_end = r_begin + g.r_chunk;
  if (r_end > g.R) r_end = g.R;
  Acc acc[W];
#pragma unroll
  for (int e = 0; e < W; ++e) acc[e] = R::init();
  if (active) {
    const float* base = x + k0 * g.R * g.K1 + col * W;
    auto take = [&](const float4& q4, float q1) {
      if (VEC) {
        acc[0] = R::step(acc[0], q4.x);
        acc[W > 1 ? 1 : 0] = R::step(acc[W > 1 ? 1 : 0], q4.y);
        acc[W > 2 ? 2 : 0] = R::step(acc[W > 2 ? 2 : 0], q4.z);
        acc[W > 3 ? 3 : 0] = R::step(acc[W > 3 ? 3 : 0], q4.w);
      } else {
        acc[0] = R::step(acc[0], q1);
      }
    };
    int64_t r0 = r_begin + ty;
    // full steps: kUnroll rows per thread, loads issued together and unguarded
    for (; r0 + static_cast<int64_t>(kUnroll - 1) * TY < r_end; r0 += static_cast<int64_t>(TY) * kUnroll) {
      float4 v4[kUnroll];
      float v1[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const float* p = base + (r0 + static_cast<int64_t>(u) * TY) * g.K1;
        if (VEC) v4[u] = ld_stream(reinterpret_cast<const float4*>(p));
        else v1[u] = ld_stream(p);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) take(v4[u], v1[u]);
    }
    for (; r0 < r_end; r0 += TY) {   // remaining rows
      const float* p = base + r0 * g.K1;
      if (VEC) take(ld_stream(reinterpret_cast<const float4*>(p)), 0.f);
      else take(make_float4(0.f, 0.f, 0.f, 0.f), ld_stream(p));
    }
  }
  // rows that share a warp (lanes with equal tx) are merged with shuffles; the per-warp results go
  // through shared memory and the first TX*W threads merge the warps in index order
  constexpr int kWarps = kThreads / 32;
  constexpr int kRowsPerWarp = 32 / TX;   // TX is 8, 16 or 32
#pragma unroll
  for (int e = 0; e < W; ++e) {
#pragma unroll
    for (int o = TX; o < 32; o <<= 1) acc[e] = R::merge(acc[e], __shfl_xor_sync(0xffffffffu, acc[e], o));
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane < TX) {
#pragma unroll
    for (int e = 0; e < W; ++e) smem[warp][lane * W + e] = acc[e];
  }
  (void)kRowsPerWarp;
  __syncthreads();
  if (threadIdx.x < TX * W) {
    const int c = threadIdx.x;
    const int64_t colu = bx * TX + c / W;
    if (colu < g.K1u) {
      Acc a = smem[0][c];
#pragma unroll
      for (int r = 1; r < kWarps; ++r) a = R::merge(a, smem[r][c]);
      const int64_t out = k0 * g.K1 + colu * W + (c % W);
      emit<OP, TO_PART>(a, y, part, out, s, g.n_out, g.count);
    }
  }
}

// Inner-kept family on the fixed-column 128-bit walk (colwalk.cuh): x viewed as [K0, R, K1] is a
// stack of K0 planes; every access is a float4 whatever K1 is (K1 = 196: no idle lanes, where the
// TX-lane tiles of redB_kernel leave 7 of 56 idle), a thread's four lanes are four fixed columns,
// and the block combines the partial rows of a column through shared memory in row order.  Used
// when the planes alone give enough blocks (no split of R over blocks).
template <int OP, int U, int NB, bool TO_PART>
__global__ void __launch_bounds__(512, 3)
redC_kernel(const float* __restrict__ x, float* y, double* part, const __grid_constant__ ColWalk q, int64_t n_out,
            Divisor count) {
  using R = RedOp<OP>;
  using Acc = typename R::Acc;
  extern __shared__ double sm_raw[];
  Acc* sm = reinterpret_cast<Acc*>(sm_raw);   // [blockDim * 4], after the walk (the ring lives here during it)
  const ColLane L = colwalk_thread(q, threadIdx.x, blockIdx.x);
  Acc acc[4] = {R::init(), R::init(), R::init(), R::init()};
  colwalk_stream<U, NB>(reinterpret_cast<const float4*>(x) + L.first4, L.step4, L.cnt,
                        reinterpret_cast<float4*>(sm_raw) + threadIdx.x, [&](const float4 (&v)[U], int, int valid) {
#pragma unroll
                          for (int u = 0; u < U; ++u) {
                            if (u < valid) {
                              acc[0] = R::step(acc[0], v[u].x), acc[1] = R::step(acc[1], v[u].y);
                              acc[2] = R::step(acc[2], v[u].z), acc[3] = R::step(acc[3], v[u].w);
                            }
                          }
                        });
  __syncthreads();   // every thread is done with its ring slots: the memory now holds the partials
  if (L.slot >= 0) {
#pragma unroll
    for (int e = 0; e < 4; ++e) sm[L.slot + e] = acc[e];
  }
  __syncthreads();
  const int planes = q.tiled ? 1 : q.P;
  const int plane_slots = 4 * q.tact;
  const int64_t tile_n = blockIdx.x / q.ntile, tile = blockIdx.x - tile_n * q.ntile;
  const int64_t K1 = q.tiled ? q.row4 * 4 : q.ncols;
  for (int c = threadIdx.x; c < planes * q.ncols; c += blockDim.x) {
    const int pl = static_cast<int>(q.div_ncols.div(static_cast<uint32_t>(c)));
    const int cc = c - pl * q.ncols;
    const int64_t n = q.tiled ? tile_n : static_cast<int64_t>(blockIdx.x) * q.P + pl;
    const int64_t col = q.tiled ? tile * q.ncols + cc : cc;
    if (n >= q.outer || col >= K1) continue;
    const Acc* p = sm + pl * plane_slots + cc;
    Acc a = p[0];
    for (int r = 1; r < q.R; ++r) a = R::merge(a, p[r * q.ncols]);
    emit<OP, TO_PART>(a, y, part, n * K1 + col, 0, n_out, count);
  }
}

// ---- generic: any alternation of kept / reduced dims ----------------------------------------------
struct GeomG {
  int nk, nr;                                  // kept / reduced dim counts (outermost first)
  int64_t k_extent[kMaxDims], k_stride[kMaxDims];
  int64_t r_extent[kMaxDims], r_stride[kMaxDims];
  int64_t n_out, n_red;
  Divisor count;
};

template <int OP, bool TO_PART>
__global__ void __launch_bounds__(kThreads)
redG_kernel(const float* __restrict__ x, float* y, double* part, const __grid_constant__ GeomG g) {
  using R = RedOp<OP>;
  __shared__ typename R::Acc smem[32];
  for (int64_t o = blockIdx.x; o < g.n_out; o += gridDim.x) {
    int64_t off = 0, cc = o;
    for (int d = g.nk - 1; d >= 0; --d) {
      int64_t q = cc / g.k_extent[d];
      off += (cc - q * g.k_extent[d]) * g.k_stride[d];
      cc = q;
    }
    typename R::Acc acc = R::init();
    for (int64_t j = threadIdx.x; j < g.n_red; j += kThreads) {
      int64_t rel = 0, jj = j;
      for (int d = g.nr - 1; d >= 0; --d) {
        int64_t q = jj / g.r_extent[d];
        rel += (jj - q * g.r_extent[d]) * g.r_stride[d];
        jj = q;
      }
      acc = R::step(acc, x[off + rel]);
    }
    acc = block_reduce(acc, typename R::Merge(), R::init(), smem);
    if (threadIdx.x == 0) emit<OP, TO_PART>(acc, y, part, o, 0, g.n_out, g.count);
  }
}

// ---- finishing kernel: combine `splits` double partials per output, in split order ----------------
// LANES = 1: one thread per output; 32: one warp per output; 256: one block per output (many
// splits, few outputs, e.g. a full-tensor reduction).
template <int OP, int LANES, bool TO_PART>
__global__ void __launch_bounds__(kThreads)
red_finish_kernel(const double* __restrict__ in, int64_t splits, int64_t n_out, float* y, double* part,
                  Divisor count, int64_t split_stride) {
  using R = RedOp<OP>;
  using Acc = typename R::Acc;
  __shared__ Acc smem[32];
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t o = gid / LANES;
  const int lane = static_cast<int>(gid % LANES);
  if (o >= n_out) return;   // whole warps (LANES == 32) / whole blocks (256) leave together
  Acc acc = R::init();
  for (int64_t s = lane; s < splits; s += LANES) acc = R::merge(acc, static_cast<Acc>(in[s * split_stride + o]));
  if (LANES == 32) acc = warp_reduce(acc, typename R::Merge());
  if (LANES == 256) acc = block_reduce(acc, typename R::Merge(), R::init(), smem);
  if (lane == 0) emit<OP, TO_PART>(acc, y, part, o, 0, n_out, count);
}

// ---- host planning --------------------------------------------------------------------------------
enum Family { kFamA, kFamB, kFamG };

struct Plan {
  Family family;
  bool vec;
  bool a_warp;        // family A: warp-per-output kernel
  bool a_rows;        // family A: staged short-rows kernel
  int rows_per_block;
  int tx;             // family B
  bool b_colwalk;     // family B on the fixed-column walk
  ColWalk cw;
  int64_t splits;
  int64_t n_out, n_red;
  GeomA a;
  GeomB b;
  GeomG gen;
  int64_t scratch_bytes;
};

int make_plan(const int* in_shape, int num_axes, const int* axes, int n_axes, const void* x, Plan* P) {
  if (in_shape == nullptr || axes == nullptr || num_axes < 1 || num_axes > SB200_MAX_AXES || n_axes < 1 ||
      n_axes > num_axes)
    return SB200_ERR_BAD_ARGUMENT;
  bool red[SB200_MAX_AXES] = {false};
  for (int i = 0; i < n_axes; ++i) {
    if (axes[i] < 0 || axes[i] >= num_axes || red[axes[i]]) return SB200_ERR_BAD_ARGUMENT;
    red[axes[i]] = true;
  }
  int64_t ext[SB200_MAX_AXES];
  bool kind[SB200_MAX_AXES];
  int nd = 0;
  int64_t n_out = 1, n_red = 1;
  for (int n = 0; n < num_axes; ++n) {
    const int d = in_shape[n];
    if (d < 1) return SB200_ERR_BAD_ARGUMENT;
    if (red[n]) n_red *= d; else n_out *= d;
    if (n_out * n_red > (1ll << 40)) return SB200_ERR_UNSUPPORTED;
    if (d == 1) continue;
    if (nd > 0 && kind[nd - 1] == red[n]) ext[nd - 1] *= d;
    else { ext[nd] = d; kind[nd] = red[n]; ++nd; }
  }
  if (nd > kMaxDims) return SB200_ERR_UNSUPPORTED;
  P->n_out = n_out, P->n_red = n_red, P->splits = 1, P->scratch_bytes = 0, P->vec = false;
  P->a_warp = false, P->a_rows = false, P->rows_per_block = 1, P->tx = 32, P->b_colwalk = false;
  const Divisor count(static_cast<double>(n_red));
  const int64_t target_blocks = static_cast<int64_t>(sm_count()) * 8;

  // pattern -> family
  auto is = [&](std::initializer_list<bool> pat) {
    if (static_cast<int>(pat.size()) != nd) return false;
    int i = 0;
    for (bool b : pat) if (kind[i++] != b) return false;
    return true;
  };
  const bool T = true, F = false;
  int64_t R0 = 1, K = 1, R1 = 1, K0 = 1, Rm = 1, K1 = 1;
  Family fam;
  if (nd == 0) { fam = kFamA; }                                   // single element
  else if (is({T})) { fam = kFamA; R1 = ext[0]; }
  else if (is({F})) { fam = kFamA; K = ext[0]; }                  // nothing to reduce: R1 = 1
  else if (is({F, T})) { fam = kFamA; K = ext[0]; R1 = ext[1]; }
  else if (is({T, F, T})) { fam = kFamA; R0 = ext[0]; K = ext[1]; R1 = ext[2]; }
  else if (is({T, F})) { fam = kFamB; Rm = ext[0]; K1 = ext[1]; }
  else if (is({F, T, F})) { fam = kFamB; K0 = ext[0]; Rm = ext[1]; K1 = ext[2]; }
  else fam = kFamG;
  // family A needs R0*R1u < 2^32 when R0 > 1 and K in grid.x; otherwise fall back to generic
  if (fam == kFamA && ((R0 > 1 && R0 * R1 >= (1ll << 32)) || K >= (1ll << 31) || R0 >= (1ll << 32))) fam = kFamG;
  if (fam == kFamB && (K0 * ((K1 + 7) / 8) >= (1ll << 31))) fam = kFamG;
  P->family = fam;

  if (fam == kFamA) {
    GeomA& g = P->a;
    const bool vec = (R1 % 4 == 0) && aligned16(x);
    P->vec = vec;
    g.K = K, g.R0 = static_cast<uint32_t>(R0);
    const int64_t r1u = vec ? R1 / 4 : R1;
    g.row_elems = R1, g.r0_stride = K * R1;
    g.n_units = R0 * r1u;
    g.count = count;
    if (R0 == 1 && r1u <= kRowsMaxUnitsPerRow) {
      P->a_rows = true;
      P->rows_per_block = 0;   // depends on the operation's tile: set at launch
      g.R1u = static_cast<uint32_t>(r1u);
      g.div_r1u = FastDiv32(g.R1u);
      g.chunk_units = g.n_units;
    } else if (g.n_units < 2048 && r1u < (1ll << 32)) {
      P->a_warp = true;
      g.R1u = static_cast<uint32_t>(r1u);
      g.div_r1u = FastDiv32(g.R1u);
      g.chunk_units = g.n_units;
    } else {
      // Many small blocks stream better than few long-running ones (see elementwise.cu), and a
      // grid of only a few waves loses up to a whole block duration in its last, partly filled
      // wave: aim at >= kTargetWaves waves of resident blocks, at least kMinTiles tiles per block.
      int64_t splits = (target_blocks * kTargetWaves + K - 1) / K;
      if (K >= target_blocks * 4) splits = 1;   // already several waves of blocks: no second kernel
      const int64_t max_by_work = (g.n_units + kThreads * kUnroll * kMinTiles - 1) / (kThreads * kUnroll * kMinTiles);
      if (splits > max_by_work) splits = max_by_work;
      if (splits > 65535) splits = 65535;
      if (splits < 1) splits = 1;
      int64_t chunk = (g.n_units + splits - 1) / splits;
      const int64_t tile = kThreads * kUnroll;
      chunk = (chunk + tile - 1) / tile * tile;
      splits = (g.n_units + chunk - 1) / chunk;
      g.chunk_units = chunk;
      g.R1u = static_cast<uint32_t>(r1u < (1ll << 32) ? r1u : 0);   // only used when R0 > 1
      g.div_r1u = FastDiv32(g.R1u ? g.R1u : 1);
      P->splits = splits;
    }
  } else if (fam == kFamB) {
    GeomB& g = P->b;
    const bool vec = (K1 % 4 == 0) && aligned16(x);
    P->vec = vec;
    g.K0 = K0, g.R = Rm, g.K1 = K1, g.K1u = vec ? K1 / 4 : K1;
    g.n_out = n_out, g.count = count;
    int best_tx = 32;
    int64_t best_waste = -1;
    for (int tx : {32, 16, 8}) {
      const int64_t waste = (g.K1u + tx - 1) / tx * tx - g.K1u;
      if (best_waste < 0 || waste < best_waste) best_waste = waste, best_tx = tx;
    }
    P->tx = best_tx;
    g.nbx = (g.K1u + best_tx - 1) / best_tx;
    const int ty = kThreads / best_tx;
    const int64_t blocks = g.nbx * K0;
    int64_t splits = (target_blocks * kTargetWaves + blocks - 1) / blocks;
    if (blocks >= target_blocks * 4) splits = 1;   // already several waves of blocks: no second kernel
    const int64_t max_by_work = (Rm + ty * kUnroll * kMinTiles - 1) / (ty * kUnroll * kMinTiles);
    if (splits > max_by_work) splits = max_by_work;
    if (splits > 65535) splits = 65535;
    if (splits < 1) splits = 1;
    int64_t chunk = (Rm + splits - 1) / splits;
    splits = (Rm + chunk - 1) / chunk;
    g.r_chunk = chunk;
    P->splits = splits;
    // the 128-bit walk when the planes alone fill the machine twice over (no split of R)
    ColWalk cw;
    if (K1 >= 2 && plan_colwalk(x, x, K0, Rm, K1, &cw, kWalkOnePass) && cw.grid >= 2u * static_cast<unsigned>(sm_count())) {
      P->b_colwalk = true, P->cw = cw, P->vec = true, P->splits = 1;
    }
  } else {
    GeomG& g = P->gen;
    g.nk = g.nr = 0;
    int64_t stride = 1;
    int64_t strides[kMaxDims];
    for (int d = nd - 1; d >= 0; --d) { strides[d] = stride; stride *= ext[d]; }
    for (int d = 0; d < nd; ++d) {
      if (kind[d]) { g.r_extent[g.nr] = ext[d]; g.r_stride[g.nr] = strides[d]; ++g.nr; }
      else { g.k_extent[g.nk] = ext[d]; g.k_stride[g.nk] = strides[d]; ++g.nk; }
    }
    g.n_out = n_out, g.n_red = n_red, g.count = count;
  }
  if (P->splits > 1) P->scratch_bytes = P->splits * n_out * static_cast<int64_t>(sizeof(double));
  return SB200_OK;
}

template <int OP, bool TO_PART>
void launch_stage1(const Plan& P, const float* x, float* y, double* part, cudaStream_t s) {
  if (P.family == kFamA) {
    if (P.a_rows) {
      const int r1u = static_cast<int>(P.a.R1u);
      const int rows_per_block = RowsTile<OP>::kUnits / r1u;
      const unsigned grid = tile_grid(P.a.K, rows_per_block);
      constexpr int T = RowsTile<OP>::kT;
      if (P.vec) redA_rows_kernel<OP, true, TO_PART><<<grid, T, 0, s>>>(x, y, part, P.a.K, r1u, rows_per_block, P.a.count);
      else redA_rows_kernel<OP, false, TO_PART><<<grid, T, 0, s>>>(x, y, part, P.a.K, r1u, rows_per_block, P.a.count);
    } else if (P.a_warp) {
      const int64_t blocks = (P.a.K * 32 + kThreads - 1) / kThreads;
      const unsigned grid = stream_grid(blocks, 8);
      if (P.vec) redA_warp_kernel<OP, true, TO_PART><<<grid, kThreads, 0, s>>>(x, y, part, P.a);
      else redA_warp_kernel<OP, false, TO_PART><<<grid, kThreads, 0, s>>>(x, y, part, P.a);
    } else {
      dim3 grid(static_cast<unsigned>(P.a.K), static_cast<unsigned>(P.splits));
      if (P.vec) redA_block_kernel<OP, true, TO_PART><<<grid, kThreads, 0, s>>>(x, y, part, P.a);
      else redA_block_kernel<OP, false, TO_PART><<<grid, kThreads, 0, s>>>(x, y, part, P.a);
    }
  } else if (P.family == kFamB && P.b_colwalk) {
    constexpr int U = 2, NB = 4;
    size_t smem = colwalk_smem(P.cw, sizeof(typename RedOp<OP>::Acc));
    if (smem < colwalk_ring_bytes(P.cw, U, NB)) smem = colwalk_ring_bytes(P.cw, U, NB);
    static unsigned long long attr_done = 0;   // per instantiation, one bit per device
    allow_dynamic_smem(redC_kernel<OP, U, NB, TO_PART>, 512 * U * NB * 16, &attr_done);
    redC_kernel<OP, U, NB, TO_PART><<<P.cw.grid, P.cw.threads, smem, s>>>(x, y, part, P.cw, P.n_out, P.b.count);
  } else if (P.family == kFamB) {
    dim3 grid(static_cast<unsigned>(P.b.nbx * P.b.K0), static_cast<unsigned>(P.splits));
#define SB200_LAUNCH_B(TXV)                                                                          \
  if (P.vec) redB_kernel<OP, TXV, true, TO_PART><<<grid, kThreads, 0, s>>>(x, y, part, P.b);         \
  else redB_kernel<OP, TXV, false, TO_PART><<<grid, kThreads, 0, s>>>(x, y, part, P.b);
    if (P.tx == 32) { SB200_LAUNCH_B(32) }
    else if (P.tx == 16) { SB200_LAUNCH_B(16) }
    else { SB200_LAUNCH_B(8) }
#undef SB200_LAUNCH_B
  } else {
    const unsigned grid = stream_grid(P.n_out, 8);
    redG_kernel<OP, TO_PART><<<grid, kThreads, 0, s>>>(x, y, part, P.gen);
  }
}

// in[s * split_stride + o] is part s of output o (split_stride == n_out for the kernels' own scratch).
template <int OP, bool TO_PART>
void launch_finish(const double* in, int64_t splits, int64_t n_out, float* y, double* part, Divisor count,
                   cudaStream_t s, int64_t split_stride = -1) {
  if (split_stride < 0) split_stride = n_out;
  if (splits > 256) {
    red_finish_kernel<OP, 256, TO_PART><<<static_cast<unsigned>(n_out), kThreads, 0, s>>>(in, splits, n_out, y, part, count, split_stride);
  } else if (splits > 8) {
    const int64_t blocks = (n_out * 32 + kThreads - 1) / kThreads;
    red_finish_kernel<OP, 32, TO_PART><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(in, splits, n_out, y, part, count, split_stride);
  } else {
    const int64_t blocks = (n_out + kThreads - 1) / kThreads;
    red_finish_kernel<OP, 1, TO_PART><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(in, splits, n_out, y, part, count, split_stride);
  }
}

// emit_partial: write double partials to `partial` instead of floats to y.
template <int OP>
int run(const Plan& P, const float* x, float* y, double* partial, void* scratch, bool emit_partial,
        cudaStream_t s) {
  const Divisor count(static_cast<double>(P.n_red));
  if (P.splits > 1) {
    double* tmp = static_cast<double*>(scratch);
    launch_stage1<OP, true>(P, x, nullptr, tmp, s);
    int rc = after_launch("sb200_reduce");
    if (rc != SB200_OK) return rc;
    if (emit_partial) launch_finish<OP, true>(tmp, P.splits, P.n_out, nullptr, partial, count, s);
    else launch_finish<OP, false>(tmp, P.splits, P.n_out, y, nullptr, count, s);
    return after_launch("sb200_reduce(finish)");
  }
  if (emit_partial) launch_stage1<OP, true>(P, x, nullptr, partial, s);
  else launch_stage1<OP, false>(P, x, y, nullptr, s);
  return after_launch("sb200_reduce");
}

int dispatch(const Plan& P, int operation, const float* x, float* y, double* partial, void* scratch,
             bool emit_partial, cudaStream_t s) {
  switch (operation) {
    case SB200_RED_PROD: return run<SB200_RED_PROD>(P, x, y, partial, scratch, emit_partial, s);
    case SB200_RED_SUM: return run<SB200_RED_SUM>(P, x, y, partial, scratch, emit_partial, s);
    case SB200_RED_MAX: return run<SB200_RED_MAX>(P, x, y, partial, scratch, emit_partial, s);
    case SB200_RED_MIN: return run<SB200_RED_MIN>(P, x, y, partial, scratch, emit_partial, s);
    case SB200_RED_AVG: return run<SB200_RED_AVG>(P, x, y, partial, scratch, emit_partial, s);
    case SB200_RED_L1: return run<SB200_RED_L1>(P, x, y, partial, scratch, emit_partial, s);
    case SB200_RED_L2: return run<SB200_RED_L2>(P, x, y, partial, scratch, emit_partial, s);
    default: return SB200_ERR_BAD_ARGUMENT;
  }
}

int reduce_common(const float* x, const int* in_shape, int num_axes, const int* axes, int n_axes,
                  int operation, float* y, double* partial, void* scratch, int64_t scratch_bytes,
                  bool emit_partial, void* stream) {
  if (x == nullptr || (emit_partial ? partial == nullptr : y == nullptr)) return SB200_ERR_BAD_ARGUMENT;
  if (operation < SB200_RED_PROD || operation > SB200_RED_L2) return SB200_ERR_BAD_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(x) & 3u) return SB200_ERR_BAD_ARGUMENT;
  Plan P;
  int rc = make_plan(in_shape, num_axes, axes, n_axes, x, &P);
  if (rc != SB200_OK) return rc;
  if (P.scratch_bytes > 0) {
    if (scratch == nullptr || scratch_bytes < P.scratch_bytes || (reinterpret_cast<uintptr_t>(scratch) & 7u))
      return SB200_ERR_SCRATCH;
  }
  return dispatch(P, operation, x, y, partial, scratch, emit_partial, static_cast<cudaStream_t>(stream));
}

// ---- built-in scratch for sb200_reduce_static ------------------------------------------------------
// One fixed array per GPU that loads this library (it lives in the module's global data until the
// process exits).  Host code may not use the name below as a pointer: on the host it is only a
// stand-in for the device symbol.  The device address is asked for once per device, with that
// device current, through cudaGetSymbolAddress, and that address is what the kernels receive.
constexpr int64_t kStaticScratchBytes = SB200_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_static_scratch_mutex;

// Device address of the built-in scratch on the CURRENT device, or an error status.
int static_scratch_address(void** out) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return cuda_failure(err, "sb200_reduce_static(cudaGetDevice)");
  if (dev < 0 || dev >= kMaxDevices) {
    set_error_text("sb200_reduce_static: device ordinal outside 0..63");
    return SB200_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess) return cuda_failure(err, "sb200_reduce_static(cudaGetSymbolAddress)");
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return SB200_OK;
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" {

int64_t sb200_reduce_scratch_bytes(const int* in_shape, int num_axes, const int* axes, int n_axes,
                                   int operation) {
  (void)operation;
  Plan P;
  // The plan depends on 16-byte alignment of x only through the vector/scalar choice, which does
  // not change the number of splits' upper bound by more than 4x; size for the scalar layout.
  if (make_plan(in_shape, num_axes, axes, n_axes, reinterpret_cast<const void*>(4), &P) != SB200_OK) return -1;
  int64_t scalar_bytes = P.scratch_bytes;
  if (make_plan(in_shape, num_axes, axes, n_axes, nullptr, &P) != SB200_OK) return -1;
  return scalar_bytes > P.scratch_bytes ? scalar_bytes : P.scratch_bytes;
}

int sb200_reduce(const float* x, const int* in_shape, int num_axes, const int* axes, int n_axes,
                 int operation, float* y, void* scratch, int64_t scratch_bytes, void* stream) {
  return reduce_common(x, in_shape, num_axes, axes, n_axes, operation, y, nullptr, scratch, scratch_bytes,
                       false, stream);
}

int sb200_reduce_static(const float* x, const int* in_shape, int num_axes, const int* axes, int n_axes,
                        int operation, float* y, void* stream) {
  // the plan's own status (bad argument, or a geometry the kernels do not cover) is what the caller sees
  Plan probe;
  const int plan_rc = make_plan(in_shape, num_axes, axes, n_axes, x, &probe);
  if (plan_rc != SB200_OK) return plan_rc;
  const int64_t need = sb200_reduce_scratch_bytes(in_shape, num_axes, axes, n_axes, operation);
  if (need < 0) return SB200_ERR_BAD_ARGUMENT;
  if (need > kStaticScratchBytes) {
    char msg[200];
    std::snprintf(msg, sizeof(msg),
                  "sb200_reduce_static: this reduction needs %lld bytes of scratch, the built-in buffer holds %lld; "
                  "use sb200_reduce with caller scratch", static_cast<long long>(need),
                  static_cast<long long>(kStaticScratchBytes));
    set_error_text(msg);
    return SB200_ERR_SCRATCH;
  }
  void* scratch = nullptr;
  if (need > 0) {
    int rc = static_scratch_address(&scratch);
    if (rc != SB200_OK) return rc;
  }
  return reduce_common(x, in_shape, num_axes, axes, n_axes, operation, y, nullptr, scratch, kStaticScratchBytes,
                       false, stream);
}

int sb200_reduce_partial(const float* x, const int* in_shape, int num_axes, const int* axes, int n_axes,
                         int operation, double* partial, void* scratch, int64_t scratch_bytes, void* stream) {
  return reduce_common(x, in_shape, num_axes, axes, n_axes, operation, nullptr, partial, scratch,
                       scratch_bytes, true, stream);
}

int sb200_reduce_combine(const double* parts, int64_t n_parts, int64_t part_stride, float* y, int64_t count,
                         int operation, int64_t total_reduced_count, void* stream) {
  if (count < 0 || n_parts < 1 || part_stride < count || total_reduced_count < 1 ||
      (count > 0 && (parts == nullptr || y == nullptr)))
    return SB200_ERR_BAD_ARGUMENT;
  if (count == 0) return SB200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const Divisor c(static_cast<double>(total_reduced_count));
  switch (operation) {
    case SB200_RED_PROD: launch_finish<SB200_RED_PROD, false>(parts, n_parts, count, y, nullptr, c, s, part_stride); break;
    case SB200_RED_SUM: launch_finish<SB200_RED_SUM, false>(parts, n_parts, count, y, nullptr, c, s, part_stride); break;
    case SB200_RED_MAX: launch_finish<SB200_RED_MAX, false>(parts, n_parts, count, y, nullptr, c, s, part_stride); break;
    case SB200_RED_MIN: launch_finish<SB200_RED_MIN, false>(parts, n_parts, count, y, nullptr, c, s, part_stride); break;
    case SB200_RED_AVG: launch_finish<SB200_RED_AVG, false>(parts, n_parts, count, y, nullptr, c, s, part_stride); break;
    case SB200_RED_L1: launch_finish<SB200_RED_L1, false>(parts, n_parts, count, y, nullptr, c, s, part_stride); break;
    case SB200_RED_L2: launch_finish<SB200_RED_L2, false>(parts, n_parts, count, y, nullptr, c, s, part_stride); break;
    default: return SB200_ERR_BAD_ARGUMENT;
  }
  return after_launch("sb200_reduce_combine");
}

int sb200_reduce_finalize(const double* partial, float* y, int64_t count, int operation,
                          int64_t total_reduced_count, void* stream) {
  return sb200_reduce_combine(partial, 1, count, y, count, operation, total_reduced_count, stream);
}

}  // extern "C"
