// Fixed-column 128-bit walk over x viewed as [outer, dim, inner] (inner > 1), shared by the strided
// Softmax and the Normalize family.
//
// A [dim, inner] plane is a flat run of dim*inner floats.  Read as float4, a thread that advances by
// a multiple of p = inner / gcd(inner, 4) float4 per step keeps each of its four lanes on ONE column
// of the plane for the whole walk (inner = 49: p = 49 float4 = 4 rows; inner = 1444: p = 361 float4
// = 1 row).  So every access is 128-bit and coalesced for any `inner`, and no per-element division
// or address arithmetic is left: one pointer bump per float4.  Two block layouts:
//   flat:  `tact` = k*p consecutive threads own consecutive float4 of a plane and step by `tact`;
//          a block holds P = blockDim / tact planes.  Needs p <= 1024 and dim*inner % 4 == 0.
//   tiled: inner % 4 == 0 and rows longer than a block: the block owns a tile of W4 float4 columns
//          and G row groups; thread (g, w) steps by G rows.
// Either way a thread's lane e accumulates one partial per column; the block combines the partials
// of a column through shared memory laid out as [R][ncols] per plane (R partial rows), where lane e
// of thread t sits at slot 4*t + e.
#pragma once

#include "common.cuh"

namespace sb200 {

struct ColWalk {
  int64_t outer;      // planes
  int64_t plane4;     // float4 per plane
  int64_t row4;       // tiled: float4 per row (inner / 4)
  int64_t ntile;      // tiled: column tiles per plane (1 when flat)
  int dim;
  int tiled;          // 0 flat, 1 tiled
  int tact;           // flat: active threads per plane
  int P;              // flat: planes per block (1 when tiled)
  int W4, G;          // tiled: tile width in float4, row groups
  int ncols;          // columns whose partials a plane of the block holds (flat: inner; tiled: 4*W4)
  int R;              // partial rows per column (flat: 4*tact/inner; tiled: G)
  int rows_per_step;  // rows a thread advances per step (flat: 4*tact/inner; tiled: G)
  int threads;        // block size
  unsigned grid;
  FastDiv32 div_tact, div_ncols, div_inner;
};

// Host: choose the layout.  Every candidate (block size x layout) gets a score: the share of
// threads that do useful work, times a factor for the threads an SM can keep resident (two-pass
// kernels are compiled for at most 64 registers: 1024 threads per SM), times a factor for whether the
// patches of all resident blocks fit the L2 (the kernels read their patch twice; the second read
// should not reach DRAM), times small factors against very narrow tiles and very short walks.
// Returns false when the walk does not apply (the caller falls back to its scalar kernel):
// misaligned base, plane size not a multiple of 4 floats, or a ragged inner above 4096.
// `two_pass`: the kernel reads its patch twice (Softmax, Normalize) and is compiled for 64 registers;
// single-pass kernels (Reduce) have no patch to keep, are compiled for blocks of up to 640 threads
// and fit 1280 threads per SM.
inline bool plan_colwalk(const void* x, const void* y, int64_t outer, int64_t dim, int64_t inner, ColWalk* q,
                         bool two_pass = true) {
  if (inner < 2 || dim >= (1ll << 31) || inner >= (1ll << 31)) return false;
  if (!aligned16(x) || !aligned16(y) || (dim * inner) % 4 != 0) return false;
  const int64_t plane4 = dim * inner / 4;
  const int64_t g4 = (inner % 4 == 0) ? 4 : ((inner % 2 == 0) ? 2 : 1);
  const int64_t p = inner / g4;              // period in float4
  const int rp = static_cast<int>(4 / g4);   // rows per period
  const int sms = sm_count();
  auto rate = [&](int T, double eff, int64_t patch_bytes, int64_t blocks, double cnt) {
    const int budget = two_pass ? 1024 : 1280;
    const int per_sm = budget / T > 0 ? budget / T : 1;
    const double occ = static_cast<double>(per_sm * T) / budget;
    int64_t resident = static_cast<int64_t>(sms) * per_sm;
    if (resident > blocks) resident = blocks;
    const double footprint = static_cast<double>(resident) * static_cast<double>(patch_bytes);
    const double l2 = (!two_pass || footprint <= 64e6) ? 1.0 : (footprint <= 100e6 ? 0.9 : 0.75);
    const double work = cnt >= 8 ? 1.0 : (cnt >= 4 ? 0.97 : 0.85);
    return eff * (0.5 + 0.5 * occ) * l2 * work;
  };
  double best = -1.0;
  ColWalk b{};
  if (p <= 1024) {
    // flat: k periods per plane share; partial rows per column R = k*rp kept at 64 or fewer
    int64_t k_cap = 64 / rp;
    const int64_t by_work = plane4 / (4 * p);
    if (by_work < k_cap) k_cap = by_work;
    if (k_cap < 1) k_cap = 1;
    for (int T = 128; T <= (two_pass ? 1024 : 640); T += 32) {
      int64_t k = T / p;
      if (k < 1) continue;
      if (k > k_cap) k = k_cap;
      const int64_t tact = k * p;
      int64_t P = T / tact;
      if (P > outer) P = outer;
      const int64_t blocks = (outer + P - 1) / P;
      if (blocks >= (1ll << 31)) continue;
      const double score = rate(T, static_cast<double>(P * tact) / T, P * plane4 * 16, blocks,
                                static_cast<double>(plane4) / static_cast<double>(tact));
      if (score > best + 1e-9) {
        best = score;
        b.tiled = 0, b.threads = T, b.tact = static_cast<int>(tact), b.P = static_cast<int>(P);
        b.ncols = static_cast<int>(inner), b.R = static_cast<int>(k) * rp, b.rows_per_step = b.R;
        b.W4 = 0, b.G = 0, b.ntile = 1, b.grid = static_cast<unsigned>(blocks);
      }
    }
  }
  if (inner % 4 == 0) {
    const int64_t row4 = inner / 4;
    for (int T = 256; T <= 512; T += 256) {
      for (int W4 = 8; W4 <= T; W4 *= 2) {
        const int G = T / W4;
        if (G > 1 && G * 2 > dim) continue;
        if (W4 > 8 && W4 / 2 >= row4) continue;   // tile wider than twice the row
        const int64_t ntile = (row4 + W4 - 1) / W4;
        const int64_t blocks = outer * ntile;
        if (blocks >= (1ll << 31)) continue;
        const double seg = W4 >= 32 ? 1.0 : (W4 == 16 ? 0.97 : 0.9);
        const double score = seg * rate(T, static_cast<double>(row4) / static_cast<double>(ntile * W4), dim * W4 * 16,
                                        blocks, static_cast<double>(dim) / G);
        if (score > best + 1e-9) {
          best = score;
          b.tiled = 1, b.threads = T, b.tact = T, b.P = 1, b.W4 = W4, b.G = G, b.ntile = ntile;
          b.ncols = 4 * W4, b.R = G, b.rows_per_step = G, b.grid = static_cast<unsigned>(blocks);
        }
      }
    }
  }
  if (best < 0.0) return false;
  *q = b;
  q->outer = outer, q->plane4 = plane4, q->dim = static_cast<int>(dim), q->row4 = inner / 4;
  q->div_inner = FastDiv32(static_cast<uint32_t>(inner));
  q->div_tact = FastDiv32(static_cast<uint32_t>(q->tact));
  q->div_ncols = FastDiv32(static_cast<uint32_t>(q->ncols));
  return true;
}

// What one thread of the walk owns.
struct ColLane {
  int64_t first4;   // index of its first float4 in the tensor
  int64_t step4;    // float4 between consecutive steps
  int cnt;          // steps (0 for an idle thread)
  int slot;         // shared-memory slot of lane 0 (lane e at slot + e); -1 for threads outside the layout
  int col0;         // offset of lane 0's column inside its plane's [R][ncols] partial array
  int plane_base;   // first slot of the thread's plane in shared memory
  int row0;         // row (index along dim) of lane 0's first element; flat layouts: lane e may be on the next row
  int rem0;         // flat: position of lane 0's first element inside its row (column index)
};

// `t` = thread index in the block, `block` = block index (host-callable so that tests can replay the
// layout thread by thread).
__host__ __device__ __forceinline__ ColLane colwalk_thread(const ColWalk& q, uint32_t t, int64_t block) {
  ColLane L;
  if (!q.tiled) {
    const uint32_t pl = q.div_tact.div(t);
    const uint32_t tt = t - pl * q.tact;
    const int64_t n = block * q.P + pl;
    const bool in_layout = pl < static_cast<uint32_t>(q.P);
    const bool live = in_layout && n < q.outer && static_cast<int64_t>(tt) < q.plane4;
    L.first4 = live ? n * q.plane4 + tt : 0;
    L.step4 = q.tact;
    L.cnt = live ? static_cast<int>((q.plane4 - tt + q.tact - 1) / q.tact) : 0;
    L.plane_base = static_cast<int>(pl) * 4 * q.tact;
    L.slot = in_layout ? static_cast<int>(t) * 4 : -1;
    uint32_t row, rem;
    q.div_inner.divmod(4 * tt, row, rem);
    L.col0 = static_cast<int>(rem);
    L.row0 = static_cast<int>(row);
    L.rem0 = static_cast<int>(rem);
  } else {
    const uint32_t w = t % static_cast<uint32_t>(q.W4), g = t / static_cast<uint32_t>(q.W4);
    const int64_t n = block / q.ntile, tile = block - n * q.ntile;
    const int64_t col4 = tile * q.W4 + w;
    const bool live = col4 < q.row4 && static_cast<int>(g) < q.dim;
    L.first4 = live ? n * q.plane4 + g * q.row4 + col4 : 0;
    L.step4 = static_cast<int64_t>(q.G) * q.row4;
    L.cnt = live ? (q.dim - static_cast<int>(g) + q.G - 1) / q.G : 0;
    L.plane_base = 0;
    L.slot = static_cast<int>(t) * 4;
    L.col0 = static_cast<int>(w) * 4;
    L.row0 = static_cast<int>(g);
    L.rem0 = 0;
  }
  return L;
}

// Column of lane e inside the plane's partial array (flat layouts wrap at the end of a row).
__host__ __device__ __forceinline__ int colwalk_col(const ColWalk& q, const ColLane& L, int e) {
  int c = L.col0 + e;
  if (!q.tiled && c >= q.ncols) c -= q.ncols;
  return c;
}

// Dynamic shared memory the walk needs per block for one array of `elem` bytes per lane.
inline size_t colwalk_smem(const ColWalk& q, size_t elem) { return static_cast<size_t>(q.threads) * 4 * elem; }

}  // namespace sb200
