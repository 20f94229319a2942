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
  int period4;        // flat: float4 per period (inner / gcd(inner, 4))
  int rows_per_period;
  int lpc_shift;      // log2 of the lanes that share a column in colwalk_merge (1, 2, 4 or 8 lanes)
  unsigned grid;
  FastDiv32 div_tact, div_ncols, div_inner;
};

// How the kernel that asks for a layout uses it.
enum ColWalkUse {
  kWalkTwoPass = 0,    // reads its patch twice (second time from L2); compiled for 64 registers
  kWalkOnePass = 1,    // single pass (Reduce); blocks of up to 512 threads, 1536 threads per SM
  kWalkResident = 2,   // keeps its patch in registers: a thread may own at most `max_cnt` float4; blocks of
                       // 512 threads or fewer, so that an SM always holds two or more
};

// Host: choose the layout.  Every candidate (block size x layout) gets a score: the share of
// threads that do useful work, times a factor for the threads an SM can keep resident, times a
// factor for whether the patches of all resident blocks fit the L2 (two-pass kernels: the second
// read should not reach DRAM), times a factor for the last, partly filled wave of blocks (long
// blocks in few waves leave SMs idle at the end), times small factors against very narrow tiles
// and very short walks.  Returns false when the walk does not apply (the caller falls back to
// another kernel): misaligned base, plane size not a multiple of 4 floats, a ragged inner above
// 4096, or (kWalkResident) no layout whose threads own `max_cnt` float4 or fewer.
inline bool plan_colwalk(const void* x, const void* y, int64_t outer, int64_t dim, int64_t inner, ColWalk* q,
                         ColWalkUse use = kWalkTwoPass, int max_cnt = 0) {
  if (inner < 2 || dim >= (1ll << 31) || inner >= (1ll << 31)) return false;
  if (!aligned16(x) || !aligned16(y) || (dim * inner) % 4 != 0) return false;
  const int64_t plane4 = dim * inner / 4;
  const int64_t g4 = (inner % 4 == 0) ? 4 : ((inner % 2 == 0) ? 2 : 1);
  const int64_t p = inner / g4;              // period in float4
  const int rp = static_cast<int>(4 / g4);   // rows per period
  const int sms = sm_count();
  const int budget = use == kWalkOnePass ? 1536 : 1024;
  const int max_t = use == kWalkTwoPass ? 1024 : 512;
  auto rate = [&](int T, double eff, int64_t patch_bytes, int64_t blocks, double cnt) {
    const int per_sm = budget / T > 0 ? budget / T : 1;
    const double occ = static_cast<double>(per_sm * T) / budget;
    int64_t resident = static_cast<int64_t>(sms) * per_sm;
    const double waves = static_cast<double>(blocks) / static_cast<double>(resident);
    // single-pass walks stream whole planes: a short last wave costs them nothing measurable (its few
    // blocks get the bandwidth of the idle SMs), while the kernels that hold a patch lose the time of
    // their barriers and merges in it
    const double tail = (use == kWalkOnePass || waves >= 8.0) ? 1.0 : waves / static_cast<double>(static_cast<int64_t>(waves + 0.999999));
    if (resident > blocks) resident = blocks;
    const double footprint = static_cast<double>(resident) * static_cast<double>(patch_bytes);
    const double l2 = (use != kWalkTwoPass || footprint <= 64e6) ? 1.0 : (footprint <= 100e6 ? 0.9 : 0.75);
    const double work = cnt >= 8 ? 1.0 : (cnt >= 4 ? 0.97 : 0.85);
    return eff * (0.5 + 0.5 * occ) * l2 * work * (0.7 + 0.3 * tail);
  };
  double best = -1.0;
  ColWalk b{};
  const int64_t periods = plane4 / p;   // whole number: dim * gcd(inner, 4) is a multiple of 4
  {
    if (p <= 1024) {
      // flat: k periods per step; partial rows per column R = k*rp (kept at 64 or fewer unless the patch
      // has to fit the registers), a thread left about four float4 or more
      const int64_t chunk = periods;   // periods per block
      int64_t k_cap = (use == kWalkResident ? 256 : 64) / rp;
      const int64_t by_work = chunk / 4;
      if (by_work < k_cap) k_cap = by_work;
      if (k_cap < 1) k_cap = 1;
      for (int T = 128; T <= max_t; T += 32) {
        int64_t k = T / p;
        if (k < 1) continue;
        if (k > k_cap) k = k_cap;
        const int64_t tact = k * p;
        const int64_t most = (chunk + k - 1) / k;
        if (use == kWalkResident && most > max_cnt) continue;
        int64_t P = T / tact;
        if (P > outer) P = outer;
        const int64_t blocks = (outer + P - 1) / P;
        if (blocks >= (1ll << 31)) continue;
        // single-pass walks: the longer the contiguous run a block reads per step, the better DRAM
        // pages are used (measured on [1024,512,14,14] over axis 1: 7840-byte runs 0.77 of 8 TB/s,
        // 3920-byte runs 0.70)
        const double run = (use != kWalkOnePass || P * tact * 16 >= 6144) ? 1.0 : (P * tact * 16 >= 3072 ? 0.96 : 0.92);
        const double score = run * rate(T, static_cast<double>(P * tact) / T, P * chunk * p * 16, blocks,
                                        static_cast<double>(chunk) / static_cast<double>(k));
        if (score > best + 1e-9) {
          best = score;
          b.tiled = 0, b.threads = T, b.tact = static_cast<int>(tact), b.P = static_cast<int>(P);
          b.ncols = static_cast<int>(inner), b.R = static_cast<int>(k) * rp, b.rows_per_step = b.R;
          b.W4 = 0, b.G = 0, b.ntile = 1, b.grid = static_cast<unsigned>(blocks);
        }
      }
    }
    if (inner % 4 == 0) {
      // tiled: widths are the powers of two and, for rows that fit a block, the widths that cut the
      // row into 1..8 equal tiles (row4 = 49: 49, 25, 17, 13, 10, 9, 7)
      const int64_t row4 = inner / 4;
      const int64_t chunk = dim;   // rows per block
      for (int T = 256; T <= max_t; T *= 2) {
        int widths[24];
        int nw = 0;
        for (int W4 = 4; W4 <= T; W4 *= 2) widths[nw++] = W4;
        for (int parts = 1; parts <= 8; ++parts) {
          const int64_t w = (row4 + parts - 1) / parts;
          if (w >= 4 && w <= T) widths[nw++] = static_cast<int>(w);
        }
        for (int i = 0; i < nw; ++i) {
          const int W4 = widths[i];
          int G = T / W4;
          if (G > 1 && G * 2 > chunk) G = static_cast<int>(chunk / 2 > 0 ? chunk / 2 : 1);
          if ((W4 & (W4 - 1)) == 0 && W4 > 8 && W4 / 2 >= row4) continue;   // tile wider than twice the row
          const int64_t most = (chunk + G - 1) / G;
          if (use == kWalkResident && most > max_cnt) continue;
          const int64_t ntile = (row4 + W4 - 1) / W4;
          const int64_t blocks = outer * ntile;
          if (blocks >= (1ll << 31)) continue;
          const double seg = W4 >= 32 ? 1.0 : (W4 >= 16 ? 0.97 : (W4 >= 7 ? 0.9 : 0.8));
          const double eff = static_cast<double>(row4) / static_cast<double>(ntile * W4) * static_cast<double>(G * W4) / T;
          const double score = seg * rate(T, eff, chunk * W4 * 16, blocks, static_cast<double>(chunk) / G);
          if (score > best + 1e-9) {
            best = score;
            b.tiled = 1, b.threads = T, b.tact = T, b.P = 1, b.W4 = W4, b.G = G, b.ntile = ntile;
            b.ncols = 4 * W4, b.R = G, b.rows_per_step = G, b.grid = static_cast<unsigned>(blocks);
            }
        }
      }
    }
  }
  if (best < 0.0) return false;
  *q = b;
  q->outer = outer, q->plane4 = plane4, q->dim = static_cast<int>(dim), q->row4 = inner / 4;
  q->period4 = static_cast<int>(p), q->rows_per_period = rp;
  q->div_inner = FastDiv32(static_cast<uint32_t>(inner));
  q->div_tact = FastDiv32(static_cast<uint32_t>(q->tact));
  q->div_ncols = FastDiv32(static_cast<uint32_t>(q->ncols));
  q->lpc_shift = q->R >= 8 ? 3 : (q->R >= 4 ? 2 : (q->R >= 2 ? 1 : 0));
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
    const bool live = col4 < q.row4 && static_cast<int>(g) < q.G && static_cast<int>(g) < q.dim;
    L.first4 = live ? n * q.plane4 + static_cast<int64_t>(g) * q.row4 + col4 : 0;
    L.step4 = static_cast<int64_t>(q.G) * q.row4;
    L.cnt = live ? (q.dim - static_cast<int>(g) + q.G - 1) / q.G : 0;
    L.plane_base = 0;
    L.slot = static_cast<int>(g) < q.G ? static_cast<int>(t) * 4 : -1;
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

// Combine the R partial rows of every (plane, column) held by the block: sm[pl*4*tact + r*ncols + c],
// r < R.  1, 2, 4 or 8 consecutive lanes share a column (rows lane, lane+lanes, ... then a shuffle
// tree), so the order of combination is fixed and the serial part is R/lanes long.  The result lands
// in row 0.  The caller puts a barrier before (partials written) and after (results visible).
template <typename T, typename Op>
__device__ __forceinline__ void colwalk_merge(const ColWalk& q, T* sm, Op op, T identity) {
  if (q.R == 1) return;   // a column's only partial already sits in row 0
  const int total = (q.tiled ? 1 : q.P) * q.ncols;
  const int plane_slots = 4 * q.tact;
  const int lanes = 1 << q.lpc_shift;
  const int sub = threadIdx.x & (lanes - 1);
  const int per_iter = blockDim.x >> q.lpc_shift;
  for (int base = 0; base < total; base += per_iter) {
    const int c = base + (threadIdx.x >> q.lpc_shift);
    T acc = identity;
    T* col = sm;
    if (c < total) {
      int pl = 0, cc = c;
      if (!q.tiled && q.P > 1) {
        pl = static_cast<int>(q.div_ncols.div(static_cast<uint32_t>(c)));
        cc = c - pl * q.ncols;
      }
      col = sm + pl * plane_slots + cc;
      if (sub < q.R) acc = col[sub * q.ncols];
      for (int r = sub + lanes; r < q.R; r += lanes) acc = op(acc, col[r * q.ncols]);
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) acc = op(acc, __shfl_xor_sync(0xffffffffu, acc, o));
    if (c < total && sub == 0) col[0] = acc;   // the lanes of a column sit in one warp: all reads are done
  }
}

// ---- streaming a thread's float4 through a private shared-memory ring ---------------------------
// A thread of the walk reads cnt float4 at ptr, ptr + step, ...  With plain loads the bytes a thread
// keeps in flight are bounded by the registers it can spare (4 float4 = 64 B at 1024 threads per SM is
// not enough to cover HBM latency: the profile shows such kernels waiting on loads most of the time).
// Here every thread owns U*NB float4 slots of shared memory and fills them with 16-byte asynchronous
// copies (cp.async.cg: global -> shared without passing through registers), NB batches of U copies
// ahead of the batch it is consuming, so U*NB*16 bytes per thread are in flight whatever the register
// budget.  A thread only ever reads the slots it filled itself, after cp.async.wait_group: no block
// barrier, no mbarrier, nothing to spin on.
// fn(v, k0, valid): v[0..valid) are the float4 of steps k0..k0+valid; v[valid..U) hold stale bytes.
template <int U, int NB, typename F>
__device__ __forceinline__ void colwalk_stream(const float4* ptr, int64_t step, int cnt, float4* ring, F&& fn) {
  // ring: this thread's slot 0; slot i of the thread is ring[i * blockDim.x]
  const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
  const uint32_t stride = blockDim.x * 16u;
  const int nb = (cnt + U - 1) / U;
  auto issue = [&](int b, int group) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = b * U + u;
      if (k < cnt) cp_async16(base + static_cast<uint32_t>(group * U + u) * stride, ptr + k * step);
    }
    cp_async_commit();   // an empty group when the walk has ended: keeps the group count uniform
  };
#pragma unroll
  for (int b = 0; b < NB; ++b) issue(b, b);
  int group = 0;
  for (int b = 0; b < nb; ++b) {
    cp_async_wait<NB - 1>();
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = ring[(group * U + u) * blockDim.x];
    const int left = cnt - b * U;
    fn(v, b * U, left < U ? left : U);
    issue(b + NB, group);
    group = (group + 1 == NB) ? 0 : group + 1;
  }
  cp_async_wait<0>();
}

// Bytes of shared memory the ring of colwalk_stream<U, NB> takes per block.
inline size_t colwalk_ring_bytes(const ColWalk& q, int U, int NB) { return static_cast<size_t>(q.threads) * U * NB * 16; }

// Dynamic shared memory the walk needs per block for one array of `elem` bytes per lane.
inline size_t colwalk_smem(const ColWalk& q, size_t elem) { return static_cast<size_t>(q.threads) * 4 * elem; }

}  // namespace sb200
