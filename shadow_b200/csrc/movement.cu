// Data-movement operators: Concat / Stack (several tensors -> one), Slice (one -> several),
// Permute, Gather, Pad.  Pure byte movement, HBM-bound: 8 algorithmic bytes per element (one
// read, one write), except Pad whose border is write-only.
//
// Concat, Stack and Slice are one geometry: a "wide" tensor [outer, total] whose rows are the
// concatenation of the rows of N "parts" [outer, width_k].  The reference launches one strided
// copy per part; here one launch moves all parts (up to 16 per launch, longer lists chained).
// Permute collapses dimensions that stay adjacent, then transposes tiles through shared memory
// whenever the innermost dim changes (batched over the other dims; 64x64 tiles moved as float4 on
// both sides when extents and steps are multiples of 4, else 32x32 tiles of floats) and uses an
// index-arithmetic gather when the innermost dim stays (reads and writes both contiguous); no index
// tables are uploaded (the reference copies three int arrays to the device per call).
#include "common.cuh"

namespace sb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxParts = 16;
constexpr int kMaxDims = SB200_MAX_AXES;

struct Parts {
  float* ptr[kMaxParts];        // part base pointers (const-cast for sources)
  int64_t width[kMaxParts];     // elements per row of the part
  int64_t offset[kMaxParts];    // column of the wide row where the part starts
  int64_t first_block[kMaxParts + 1];   // wide kernel: prefix sum of blocks per part
  int64_t tiles_per_row[kMaxParts];
  int n;
};

// Wide parts: a block moves one tile of kTile units of one row of one part.  TO_WIDE: parts ->
// wide tensor (Concat, Stack); else wide tensor -> parts (Slice).
constexpr int kTileUnits = kThreads * 4;

template <bool TO_WIDE, bool VEC>
__global__ void __launch_bounds__(kThreads)
parts_tile_kernel(const __grid_constant__ Parts p, float* wide, int64_t total) {
  constexpr int W = VEC ? 4 : 1;
  int k = 0;
#pragma unroll
  for (int i = 1; i < kMaxParts; ++i)
    if (i < p.n && static_cast<int64_t>(blockIdx.x) >= p.first_block[i]) k = i;
  const int64_t local = static_cast<int64_t>(blockIdx.x) - p.first_block[k];
  const int64_t row = local / p.tiles_per_row[k], tile = local - row * p.tiles_per_row[k];
  const int64_t width_u = p.width[k] / W;
  float* part_row = p.ptr[k] + row * p.width[k];
  float* wide_row = wide + row * total + p.offset[k];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int64_t c = tile * kTileUnits + u * kThreads + threadIdx.x;
    if (c >= width_u) continue;
    if (VEC) {
      if (TO_WIDE) st_stream(reinterpret_cast<float4*>(wide_row) + c, ld_stream(reinterpret_cast<const float4*>(part_row) + c));
      else st_stream(reinterpret_cast<float4*>(part_row) + c, ld_stream(reinterpret_cast<const float4*>(wide_row) + c));
    } else {
      if (TO_WIDE) st_stream(wide_row + c, ld_stream(part_row + c));
      else st_stream(part_row + c, ld_stream(wide_row + c));
    }
  }
}

// Narrow parts (rows of a few elements, e.g. a Stack on the last axis): one thread per element of
// the wide tensor, the part found by a search over the (at most 16) offsets.
template <bool TO_WIDE>
__global__ void __launch_bounds__(kThreads)
parts_elem_kernel(const __grid_constant__ Parts p, float* wide, int64_t total, int64_t count, FastDiv32 div_total) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (i >= count) return;
  // one high multiply instead of a 64-bit division whenever the indices fit 32 bits
  const int64_t row = count < (1ll << 32) ? static_cast<int64_t>(div_total.div(static_cast<uint32_t>(i))) : i / total;
  const int64_t c = i - row * total;
  int k = 0;
#pragma unroll
  for (int j = 1; j < kMaxParts; ++j)
    if (j < p.n && c >= p.offset[j]) k = j;
  if (c < p.offset[0] || c >= p.offset[k] + p.width[k]) return;   // a column owned by a part of another launch
  float* q = p.ptr[k] + row * p.width[k] + (c - p.offset[k]);
  if (TO_WIDE) wide[i] = *q;
  else *q = wide[i];
}

template <bool TO_WIDE>
int run_parts(float* const* parts, const int64_t* widths, int n_parts, float* wide, int64_t outer, cudaStream_t s,
              const char* what) {
  int64_t total = 0;
  for (int k = 0; k < n_parts; ++k) {
    if (parts[k] == nullptr || widths[k] < 1 || (reinterpret_cast<uintptr_t>(parts[k]) & 3u)) return SB200_ERR_BAD_ARGUMENT;
    total += widths[k];
  }
  if (outer > 0 && total > (1ll << 40) / outer) return SB200_ERR_UNSUPPORTED;
  int64_t offset = 0;
  for (int first = 0; first < n_parts; first += kMaxParts) {
    Parts p;
    p.n = (n_parts - first < kMaxParts) ? n_parts - first : kMaxParts;
    bool vec = aligned16(wide) && (total % 4 == 0);
    int64_t max_width = 0, blocks = 0;
    for (int k = 0; k < kMaxParts; ++k) {
      const bool live = k < p.n;
      p.ptr[k] = live ? parts[first + k] : nullptr;
      p.width[k] = live ? widths[first + k] : 0;
      p.offset[k] = offset;
      if (live) {
        vec = vec && aligned16(p.ptr[k]) && (p.width[k] % 4 == 0) && (offset % 4 == 0);
        if (p.width[k] > max_width) max_width = p.width[k];
        offset += p.width[k];
      }
    }
    if (max_width >= 512) {
      const int w = vec ? 4 : 1;
      for (int k = 0; k < kMaxParts; ++k) {
        p.first_block[k] = blocks;
        p.tiles_per_row[k] = k < p.n ? (p.width[k] / w + kTileUnits - 1) / kTileUnits : 1;
        if (k < p.n) blocks += p.tiles_per_row[k] * outer;
      }
      p.first_block[kMaxParts] = blocks;
      if (blocks >= (1ll << 31)) return SB200_ERR_UNSUPPORTED;
      if (vec) parts_tile_kernel<TO_WIDE, true><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(p, wide, total);
      else parts_tile_kernel<TO_WIDE, false><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(p, wide, total);
    } else {
      const int64_t count = outer * total;
      blocks = (count + kThreads - 1) / kThreads;
      if (blocks >= (1ll << 31)) return SB200_ERR_UNSUPPORTED;
      const FastDiv32 div_total(static_cast<uint32_t>(total < (1ll << 32) ? total : 1));
      parts_elem_kernel<TO_WIDE><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(p, wide, total, count, div_total);
    }
    const int rc = after_launch(what);
    if (rc != SB200_OK) return rc;
  }
  return SB200_OK;
}

// ---- Permute ------------------------------------------------------------------------------------
struct PermGeom {
  int nd;
  FastDiv32 out_div[kMaxDims];   // divisor = output step of dim j (elements)
  uint32_t out_step[kMaxDims];
  int64_t in_step[kMaxDims];     // input step of the dim that output dim j comes from
};

// out[i] = in[sum_j (i / out_step_j % ...) * in_step_j]: consecutive threads write consecutive
// outputs; reads are as scattered as the permutation makes them.
__global__ void __launch_bounds__(kThreads)
permute_gather_kernel(const float* __restrict__ x, float* y, int64_t count, const __grid_constant__ PermGeom g) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (i >= count) return;
  uint32_t rem = static_cast<uint32_t>(i);
  int64_t src = 0;
#pragma unroll
  for (int j = 0; j < kMaxDims; ++j) {
    if (j < g.nd) {
      const uint32_t q = g.out_div[j].div(rem);
      rem -= q * g.out_step[j];
      src += static_cast<int64_t>(q) * g.in_step[j];
    }
  }
  y[i] = __ldg(x + src);
}

// Tile transpose for every permutation whose innermost output dim (a) is not the innermost input
// dim (b): a block moves kTilesB tiles of 32 (along a) x 32 (along b) through shared memory, reading
// 128-byte segments along b (contiguous in x) and writing 128-byte segments along a (contiguous in
// y); all 4 * kTilesB loads of a thread are issued before the barrier.  The remaining dims are the
// batch, decoded once per block.  NCHW <-> NHWC is the case with one batch dim.
constexpr int kTilesB = 4;
struct TileGeom {
  int64_t A, Bn;               // extents of a and b
  int64_t a_in_step, b_out_step;   // step of a in x, of b in y (a has step 1 in y, b step 1 in x)
  int64_t tiles_a, tiles_b;    // tiles along a, groups of kTilesB tiles along b
  int nbatch;
  int64_t batch_ext[kMaxDims], batch_in_step[kMaxDims], batch_out_step[kMaxDims];
  FastDiv32 div_tiles_b, div_tiles_a, div_batch[kMaxDims];   // the grid has fewer than 2^31 blocks: every factor fits 32 bits
};

// TB = tiles along b per block: kTilesB, or fewer when b is short (b = 57: two tiles instead of four half-empty ones)
template <int TB>
__global__ void __launch_bounds__(256)
permute_tile_kernel(const float* __restrict__ x, float* y, const __grid_constant__ TileGeom g) {
  __shared__ float tile[TB][32][33];
  // block index -> (batch indices, tile along a, tile along b) by multiply-high divisions (a 64-bit division
  // costs about a hundred instructions, and a thread's useful work here is 32 loads and stores)
  uint32_t rest = blockIdx.x, tb, ta;
  g.div_tiles_b.divmod(rest, rest, tb);
  g.div_tiles_a.divmod(rest, rest, ta);
  int64_t in_base = 0, out_base = 0;
  for (int d = g.nbatch - 1; d >= 0; --d) {
    uint32_t idx;
    g.div_batch[d].divmod(rest, rest, idx);
    in_base += idx * g.batch_in_step[d], out_base += idx * g.batch_out_step[d];
  }
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t a0 = static_cast<int64_t>(ta) * 32, b0 = static_cast<int64_t>(tb) * 32 * TB;
#pragma unroll
  for (int t = 0; t < TB; ++t)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t a = a0 + ty + k * 8, b = b0 + t * 32 + tx;
      if (a < g.A && b < g.Bn) tile[t][ty + k * 8][tx] = ld_stream(x + in_base + a * g.a_in_step + b);
    }
  __syncthreads();
#pragma unroll
  for (int t = 0; t < TB; ++t)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t b = b0 + t * 32 + ty + k * 8, a = a0 + tx;
      if (a < g.A && b < g.Bn) st_stream(y + out_base + b * g.b_out_step + a, tile[t][tx][ty + k * 8]);
    }
}

// The same transposition with 128-bit accesses on both sides, for extents and steps that are
// multiples of 4 floats (16-byte aligned rows): a block moves a 64 (along a) x 64 (along b) tile.
// Thread (ag, b4) reads four float4 - rows a = 4*ag .. 4*ag+3 at columns 4*b4 .. 4*b4+3, 256
// contiguous bytes per 16 threads - transposes its 4x4 block in registers, and leaves four float4
// (row b = 4*b4+j, columns a = 4*ag .. +3) in shared memory; after the barrier the threads read the
// tile row by row and write 256 contiguous bytes per 16 threads.  The shared tile is [64][16] float4
// with the column XOR-ed by (b >> 2) & 7, so the eight lanes that the hardware serves together hit
// eight different 16-byte bank groups in both phases: no padding, no conflicts.  Batch indices are
// decoded once per block with multiply-high divisions.
struct Tile4Geom {
  int A4, B4;                    // extents of a and b in float4
  int TB4;                       // float4 of b per tile (<= 16; the block has 16 * TB4 threads): chosen to divide B4 when it can
  FastDiv32 div_tb4;
  int64_t a_in_step4, b_out_step4;   // step of a in x and of b in y, in float4
  FastDiv32 div_tiles_b, div_tiles_a;
  int nbatch;
  FastDiv32 div_batch[kMaxDims];
  int64_t batch_in_step4[kMaxDims], batch_out_step4[kMaxDims];
};

__global__ void __launch_bounds__(256)
permute_tile4_kernel(const float4* __restrict__ x, float4* y, const __grid_constant__ Tile4Geom g) {
  __shared__ float4 tile[64][16];
  uint32_t rest = blockIdx.x, tb, ta;
  g.div_tiles_b.divmod(rest, rest, tb);
  g.div_tiles_a.divmod(rest, rest, ta);
  int64_t in_base = 0, out_base = 0;
  for (int d = g.nbatch - 1; d >= 0; --d) {
    uint32_t idx;
    g.div_batch[d].divmod(rest, rest, idx);
    in_base += idx * g.batch_in_step4[d], out_base += idx * g.batch_out_step4[d];
  }
  {
    uint32_t agl_u, b4l_u;                                      // position inside the tile
    g.div_tb4.divmod(threadIdx.x, agl_u, b4l_u);
    const int b4l = static_cast<int>(b4l_u), agl = static_cast<int>(agl_u);
    const int b4 = static_cast<int>(tb) * g.TB4 + b4l, ag = static_cast<int>(ta) * 16 + agl;
    if (b4 < g.B4 && ag < g.A4) {
      const float4* src = x + in_base + static_cast<int64_t>(4 * ag) * g.a_in_step4 + b4;
      const float4 r0 = ld_stream(src), r1 = ld_stream(src + g.a_in_step4), r2 = ld_stream(src + 2 * g.a_in_step4),
                   r3 = ld_stream(src + 3 * g.a_in_step4);
      const int col = agl ^ (b4l & 7);
      tile[4 * b4l + 0][col] = make_float4(r0.x, r1.x, r2.x, r3.x);
      tile[4 * b4l + 1][col] = make_float4(r0.y, r1.y, r2.y, r3.y);
      tile[4 * b4l + 2][col] = make_float4(r0.z, r1.z, r2.z, r3.z);
      tile[4 * b4l + 3][col] = make_float4(r0.w, r1.w, r2.w, r3.w);
    }
  }
  __syncthreads();
  const int agl = threadIdx.x & 15, ag = static_cast<int>(ta) * 16 + agl;
  if (ag >= g.A4) return;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int bl = (threadIdx.x >> 4) + g.TB4 * k;              // threadIdx.x >> 4 runs over 0 .. TB4 - 1
    const int b = static_cast<int>(tb) * (4 * g.TB4) + bl;
    if (b < 4 * g.B4) st_stream(y + out_base + static_cast<int64_t>(b) * g.b_out_step4 + ag, tile[bl][agl ^ ((bl >> 2) & 7)]);
  }
}

// ---- Gather, Pad --------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
gather_kernel(const float* __restrict__ x, const int* __restrict__ indexes, float* y, int64_t count, int64_t num_indexes,
              int64_t gather_dim, int64_t inner, FastDiv32 div_inner, FastDiv32 div_num) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (i >= count) return;
  int64_t r, o;   // r = outer * num_indexes + which index
  if (count < (1ll << 32)) {
    r = div_inner.div(static_cast<uint32_t>(i));
    o = div_num.div(static_cast<uint32_t>(r));
  } else {
    r = i / inner;
    o = r / num_indexes;
  }
  const int64_t col = i - r * inner, which = r - o * num_indexes;
  const int64_t gi = __ldg(indexes + which);
  // an index outside [0, gather_dim) would read outside the tensor: it yields 0 instead
  y[i] = (gi >= 0 && gi < gather_dim) ? __ldg(x + (o * gather_dim + gi) * inner + col) : 0.f;
}

// The same with 128-bit accesses (inner a multiple of 4, 16-byte aligned bases): a thread moves kGatherU
// float4, all loads issued before the first store.  count4 = outer * num_indexes * inner / 4 < 2^32.
constexpr int kGatherU = 4;
__global__ void __launch_bounds__(kThreads)
gather_vec_kernel(const float4* __restrict__ x, const int* __restrict__ indexes, float4* y, uint32_t count4, uint32_t num_indexes,
                  int64_t gather_dim, uint32_t inner4, FastDiv32 div_inner4, FastDiv32 div_num) {
  const int64_t first = static_cast<int64_t>(blockIdx.x) * (kThreads * kGatherU) + threadIdx.x;
  float4 v[kGatherU];
#pragma unroll
  for (int u = 0; u < kGatherU; ++u) {
    const int64_t i = first + u * kThreads;
    if (i < count4) {
      uint32_t r, col, o, which;
      div_inner4.divmod(static_cast<uint32_t>(i), r, col);
      div_num.divmod(r, o, which);
      const int64_t gi = __ldg(indexes + which);
      v[u] = make_float4(0.f, 0.f, 0.f, 0.f);   // an index outside [0, gather_dim) yields 0, as in the scalar kernel
      if (gi >= 0 && gi < gather_dim) v[u] = ld_stream(x + (static_cast<int64_t>(o) * gather_dim + gi) * inner4 + col);
    }
  }
#pragma unroll
  for (int u = 0; u < kGatherU; ++u) {
    const int64_t i = first + u * kThreads;
    if (i < count4) st_stream(y + i, v[u]);
  }
}

// A thread owns up to kPadRun consecutive columns of one output row: one index decode per thread
// (by high multiplies: rows < 2^32 is checked by the caller), then plain coalesced 4-byte accesses.
constexpr int kPadRun = 4;
__global__ void __launch_bounds__(kThreads)
pad_kernel(const float* __restrict__ x, float* y, int64_t rows, int in_h, int in_w, int out_h, int out_w, int top,
           int left, float value, int runs_per_row, FastDiv32 div_runs, FastDiv32 div_out_h) {
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (t >= rows * runs_per_row) return;
  uint32_t row, run, plane, oh;
  div_runs.divmod(static_cast<uint32_t>(t), row, run);
  div_out_h.divmod(row, plane, oh);
  const int h = static_cast<int>(oh) - top;
  const bool row_inside = h >= 0 && h < in_h;
  const float* xr = x + (static_cast<int64_t>(plane) * in_h + (row_inside ? h : 0)) * in_w;
  float* yr = y + static_cast<int64_t>(row) * out_w;
  // lane-interleaved columns: consecutive threads of a row write consecutive addresses
#pragma unroll
  for (int k = 0; k < kPadRun; ++k) {
    const int ow = static_cast<int>(run) + k * runs_per_row;
    if (ow >= out_w) break;
    const int w = ow - left;
    float v = value;
    if (row_inside && w >= 0 && w < in_w) v = ld_stream(xr + w);
    st_stream(yr + ow, v);
  }
}

// The same operator with 128-bit stores: the output is one flat run of floats, a thread writes one
// aligned float4 of it and finds the (plane, row, column) of its first element with two
// multiply-high divisions; the following three elements are reached by incrementing.  The sources
// are read as floats (a padded row starts at an arbitrary 4-byte offset of its source row), through
// the L1: the four loads of a warp cover the same sectors.
__global__ void __launch_bounds__(kThreads)
pad_vec_kernel(const float* __restrict__ x, float* y, int64_t total, int in_h, int in_w, int out_h, int out_w, int top,
               int left, float value, FastDiv32 div_out_w, FastDiv32 div_out_h) {
  const int64_t i4 = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t flat = 4 * i4;
  if (flat >= total) return;
  uint32_t row, ow, plane, oh;
  div_out_w.divmod(static_cast<uint32_t>(flat), row, ow);
  div_out_h.divmod(row, plane, oh);
  float v[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int h = static_cast<int>(oh) - top, w = static_cast<int>(ow) - left;
    const bool inside = h >= 0 && h < in_h && w >= 0 && w < in_w && flat + k < total;
    v[k] = inside ? __ldg(x + (static_cast<int64_t>(plane) * in_h + h) * in_w + w) : value;
    if (++ow == static_cast<uint32_t>(out_w)) {
      ow = 0;
      if (++oh == static_cast<uint32_t>(out_h)) oh = 0, ++plane;
    }
  }
  if (flat + 4 <= total) {
    st_stream(reinterpret_cast<float4*>(y) + i4, make_float4(v[0], v[1], v[2], v[3]));
  } else {
    for (int k = 0; flat + k < total; ++k) y[flat + k] = v[k];
  }
}

// Pad with non-negative paddings and an input width that is a multiple of 4: a block builds a band of
// consecutive output rows (planes follow each other, so a band may span planes) in shared memory - filled with
// the value, then overwritten by the input rows that fall into it, which are ONE contiguous range of x read as
// aligned float4 - and writes it out as aligned float4 of the flat output.  No per-element index arithmetic:
// two multiply-high divisions per input float4, none per output float4.
struct PadBand {
  int rows_per_block;
  uint32_t total_rows;        // planes * out_h
  FastDiv32 div_w4, div_in_h, div_out_h;
};

__global__ void __launch_bounds__(kThreads)
pad_smem_kernel(const float* __restrict__ x, float* y, int in_h, int in_w, int out_h, int out_w, int top, int left,
                float value, const __grid_constant__ PadBand q) {
  extern __shared__ __align__(16) float pad_tile[];
  const int t = threadIdx.x;
  const uint32_t r0 = blockIdx.x * static_cast<uint32_t>(q.rows_per_block);
  const int rows = static_cast<int>(min(static_cast<uint32_t>(q.rows_per_block), q.total_rows - r0));
  const int64_t o_start = static_cast<int64_t>(r0) * out_w;
  const int64_t a0 = o_start & ~static_cast<int64_t>(3);
  const int lead = static_cast<int>(o_start - a0);
  const int n_tile = lead + rows * out_w;
  float4* tile4 = reinterpret_cast<float4*>(pad_tile);
  // input rows (flattened over planes) that lie before output row r: whole planes, plus the rows of r's plane above it
  auto input_rows_before = [&](uint32_t r) {
    uint32_t plane, oh;
    q.div_out_h.divmod(r, plane, oh);
    return plane * static_cast<uint32_t>(in_h) + static_cast<uint32_t>(min(max(static_cast<int>(oh) - top, 0), in_h));
  };
  const uint32_t i0 = input_rows_before(r0), i1 = input_rows_before(r0 + rows);
  const int w4 = in_w >> 2, n4 = static_cast<int>(i1 - i0) * w4;
  const float4* src = reinterpret_cast<const float4*>(x) + static_cast<int64_t>(i0) * w4;
  // The band's input (at most kPadU float4 per thread for the usual 24 KB band) is requested first, so that
  // its way from DRAM overlaps the fill of the band; wider bands take further rounds.
  constexpr int kPadU = 6;
  for (int j0 = 0; j0 < n4 || j0 == 0; j0 += kPadU * kThreads) {
    float4 v[kPadU];
#pragma unroll
    for (int u = 0; u < kPadU; ++u) {
      const int j = j0 + u * kThreads + t;
      if (j < n4) v[u] = ld_stream(src + j);
    }
    if (j0 == 0) {
      const float4 fill = make_float4(value, value, value, value);
      for (int j = t; j < (n_tile + 3) >> 2; j += kThreads) tile4[j] = fill;
      __syncthreads();
    }
#pragma unroll
    for (int u = 0; u < kPadU; ++u) {
      const int j = j0 + u * kThreads + t;
      if (j < n4) {
        uint32_t irow, c4, plane, h;
        q.div_w4.divmod(static_cast<uint32_t>(j), irow, c4);
        q.div_in_h.divmod(i0 + irow, plane, h);
        const int64_t out_row = static_cast<int64_t>(plane) * out_h + h + top;
        float* dst = pad_tile + (static_cast<int>(out_row - r0) * out_w + lead + left + 4 * static_cast<int>(c4));
        dst[0] = v[u].x, dst[1] = v[u].y, dst[2] = v[u].z, dst[3] = v[u].w;
      }
    }
  }
  __syncthreads();
  // the band's floats are tile[lead, n_tile): aligned float4 in the middle, single floats where the first or
  // the last float4 is shared with a neighbouring band
  float4* y4 = reinterpret_cast<float4*>(y + a0);
  const int head_end = min((lead + 3) & ~3, n_tile);
  const int body_end = max(n_tile & ~3, head_end);
  for (int j = (head_end >> 2) + t; j < (body_end >> 2); j += kThreads) st_stream(y4 + j, tile4[j]);
  if (t < head_end - lead) y[a0 + lead + t] = pad_tile[lead + t];
  if (t < n_tile - body_end) y[a0 + body_end + t] = pad_tile[body_end + t];
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" {

int sb200_concat(const float* const* inputs, const int64_t* widths, int n_inputs, float* y, int64_t outer,
                 void* stream) {
  if (inputs == nullptr || widths == nullptr || n_inputs < 1 || n_inputs > 4096 || outer < 0) return SB200_ERR_BAD_ARGUMENT;
  if (outer == 0) return SB200_OK;
  if (y == nullptr || (reinterpret_cast<uintptr_t>(y) & 3u)) return SB200_ERR_BAD_ARGUMENT;
  return run_parts<true>(const_cast<float* const*>(inputs), widths, n_inputs, y, outer, static_cast<cudaStream_t>(stream),
                         "sb200_concat");
}

int sb200_slice(const float* x, float* const* outputs, const int64_t* widths, int n_outputs, int64_t outer,
                void* stream) {
  if (outputs == nullptr || widths == nullptr || n_outputs < 1 || n_outputs > 4096 || outer < 0) return SB200_ERR_BAD_ARGUMENT;
  if (outer == 0) return SB200_OK;
  if (x == nullptr || (reinterpret_cast<uintptr_t>(x) & 3u)) return SB200_ERR_BAD_ARGUMENT;
  return run_parts<false>(outputs, widths, n_outputs, const_cast<float*>(x), outer, static_cast<cudaStream_t>(stream),
                          "sb200_slice");
}

int sb200_permute(const float* x, float* y, const int* in_shape, const int* order, int num_axes, void* stream) {
  if (in_shape == nullptr || order == nullptr || num_axes < 1 || num_axes > kMaxDims) return SB200_ERR_BAD_ARGUMENT;
  bool seen[kMaxDims] = {false};
  int64_t count = 1;
  for (int d = 0; d < num_axes; ++d) {
    if (order[d] < 0 || order[d] >= num_axes || seen[order[d]] || in_shape[d] < 0) return SB200_ERR_BAD_ARGUMENT;
    seen[order[d]] = true;
    count *= in_shape[d];
    if (count >= (1ll << 32)) return SB200_ERR_UNSUPPORTED;   // 32-bit index arithmetic in the kernels
  }
  if (count == 0) return SB200_OK;
  if (x == nullptr || y == nullptr || x == y) return SB200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 3u) return SB200_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // input steps; then the output dims in order, dropping extent-1 dims and merging output dims
  // whose input dims are adjacent and in order
  int64_t in_step[kMaxDims];
  int64_t step = 1;
  for (int d = num_axes - 1; d >= 0; --d) { in_step[d] = step; step *= in_shape[d]; }
  int64_t ext[kMaxDims], src_step[kMaxDims];
  int nd = 0;
  for (int j = 0; j < num_axes; ++j) {
    const int d = order[j];
    if (in_shape[d] == 1) continue;
    if (nd > 0 && src_step[nd - 1] == in_step[d] * in_shape[d]) {   // previous output dim is the input dim just outside d
      ext[nd - 1] *= in_shape[d];
      src_step[nd - 1] = in_step[d];
    } else {
      ext[nd] = in_shape[d], src_step[nd] = in_step[d], ++nd;
    }
  }
  if (nd <= 1) {   // the permutation keeps the memory order
    cudaError_t e = cudaMemcpyAsync(y, x, static_cast<size_t>(count) * 4, cudaMemcpyDeviceToDevice, s);
    if (e != cudaSuccess) return cuda_failure(e, "sb200_permute(copy)");
    return SB200_OK;
  }
  // output steps of the collapsed dims
  int64_t out_step[kMaxDims];
  {
    int64_t st = 1;
    for (int j = nd - 1; j >= 0; --j) { out_step[j] = st; st *= ext[j]; }
  }
  // innermost output dim a = nd - 1; if it is not the innermost input dim, transpose tiles of
  // (a, b) with b the dim that has step 1 in x (one exists: the last input dim of extent > 1)
  if (src_step[nd - 1] != 1) {
    int jb = -1;
    for (int j = 0; j < nd - 1; ++j)
      if (src_step[j] == 1) jb = j;
    if (jb >= 0) {
      // 128-bit variant when every extent and step involved is a multiple of 4 floats
      bool vec = aligned16(x) && aligned16(y) && ext[nd - 1] % 4 == 0 && ext[jb] % 4 == 0 && src_step[nd - 1] % 4 == 0 &&
                 out_step[jb] % 4 == 0 && ext[nd - 1] / 4 < (1ll << 30) && ext[jb] / 4 < (1ll << 30);
      for (int j = 0; j < nd - 1 && vec; ++j)
        if (j != jb) vec = src_step[j] % 4 == 0 && out_step[j] % 4 == 0 && ext[j] < (1ll << 31);
      int order[kMaxDims], n_order = 0;
      for (int j = 0; j < nd - 1; ++j)
        if (j != jb) order[n_order++] = j;
      // batch dims by falling input step: over consecutive blocks the one with the SMALLEST input step varies
      // fastest, so the blocks in flight together read neighbouring row segments of x (order 2,0,3,1 of
      // [128,256,56,56]: 224-byte segments that are adjacent in memory; 0.75 -> 0.80 of 8 TB/s against the
      // output's order) - writes stay whole 256-byte segments either way
      for (int a1 = 0; a1 < n_order; ++a1)
        for (int b1 = a1 + 1; b1 < n_order; ++b1)
          if (src_step[order[b1]] > src_step[order[a1]]) { const int tmp = order[a1]; order[a1] = order[b1]; order[b1] = tmp; }
      if (vec) {
        Tile4Geom g;
        g.A4 = static_cast<int>(ext[nd - 1] / 4), g.B4 = static_cast<int>(ext[jb] / 4);
        g.a_in_step4 = src_step[nd - 1] / 4, g.b_out_step4 = out_step[jb] / 4;
        // tiles along b: as few as 16 float4 per tile allow, then of equal width (b = 56 floats: one tile of 14
        // float4 and 224 threads instead of a 16-wide tile with two idle columns)
        const int n_tiles_b = (g.B4 + 15) / 16;
        g.TB4 = (g.B4 + n_tiles_b - 1) / n_tiles_b;
        g.div_tb4 = FastDiv32(static_cast<uint32_t>(g.TB4));
        const int64_t tiles_a = (g.A4 + 15) / 16, tiles_b = n_tiles_b;
        g.div_tiles_a = FastDiv32(static_cast<uint32_t>(tiles_a)), g.div_tiles_b = FastDiv32(static_cast<uint32_t>(tiles_b));
        g.nbatch = 0;
        int64_t blocks = tiles_a * tiles_b;
        for (int o = 0; o < n_order; ++o) {
          const int j = order[o];
          g.div_batch[g.nbatch] = FastDiv32(static_cast<uint32_t>(ext[j]));
          g.batch_in_step4[g.nbatch] = src_step[j] / 4, g.batch_out_step4[g.nbatch] = out_step[j] / 4;
          ++g.nbatch;
          blocks *= ext[j];
        }
        for (int d = g.nbatch; d < kMaxDims; ++d) g.div_batch[d] = FastDiv32(1), g.batch_in_step4[d] = 0, g.batch_out_step4[d] = 0;
        if (blocks < (1ll << 31)) {
          permute_tile4_kernel<<<static_cast<unsigned>(blocks), 16 * g.TB4, 0, s>>>(reinterpret_cast<const float4*>(x),
                                                                             reinterpret_cast<float4*>(y), g);
          return after_launch("sb200_permute");
        }
      }
      TileGeom g;
      g.A = ext[nd - 1], g.Bn = ext[jb];
      g.a_in_step = src_step[nd - 1], g.b_out_step = out_step[jb];
      const int tiles_per_block = g.Bn > 64 ? kTilesB : (g.Bn > 32 ? 2 : 1);
      g.tiles_a = (g.A + 31) / 32, g.tiles_b = (g.Bn + 32 * tiles_per_block - 1) / (32 * tiles_per_block);
      g.nbatch = 0;
      int64_t blocks = g.tiles_a * g.tiles_b;
      for (int o = 0; o < n_order; ++o) {
        const int j = order[o];
        g.batch_ext[g.nbatch] = ext[j], g.batch_in_step[g.nbatch] = src_step[j], g.batch_out_step[g.nbatch] = out_step[j];
        g.div_batch[g.nbatch] = FastDiv32(static_cast<uint32_t>(ext[j] < (1ll << 32) ? ext[j] : 1));
        ++g.nbatch;
        blocks *= ext[j];
      }
      for (int d = g.nbatch; d < kMaxDims; ++d) g.batch_ext[d] = 1, g.batch_in_step[d] = 0, g.batch_out_step[d] = 0, g.div_batch[d] = FastDiv32(1);
      g.div_tiles_a = FastDiv32(static_cast<uint32_t>(g.tiles_a < (1ll << 32) ? g.tiles_a : 1));
      g.div_tiles_b = FastDiv32(static_cast<uint32_t>(g.tiles_b < (1ll << 32) ? g.tiles_b : 1));
      if (blocks < (1ll << 31)) {
        if (tiles_per_block == kTilesB) permute_tile_kernel<kTilesB><<<static_cast<unsigned>(blocks), 256, 0, s>>>(x, y, g);
        else if (tiles_per_block == 2) permute_tile_kernel<2><<<static_cast<unsigned>(blocks), 256, 0, s>>>(x, y, g);
        else permute_tile_kernel<1><<<static_cast<unsigned>(blocks), 256, 0, s>>>(x, y, g);
        return after_launch("sb200_permute");
      }
    }
  }
  PermGeom g;
  g.nd = nd;
  for (int j = nd - 1; j >= 0; --j) {
    g.out_step[j] = static_cast<uint32_t>(out_step[j]);
    g.out_div[j] = FastDiv32(static_cast<uint32_t>(out_step[j]));
    g.in_step[j] = src_step[j];
  }
  for (int j = nd; j < kMaxDims; ++j) { g.out_step[j] = 1; g.out_div[j] = FastDiv32(1); g.in_step[j] = 0; }
  const int64_t blocks = (count + kThreads - 1) / kThreads;
  permute_gather_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(x, y, count, g);
  return after_launch("sb200_permute");
}

int sb200_gather(const float* x, const int* indexes, int64_t num_indexes, int64_t outer, int64_t gather_dim,
                 int64_t inner, float* y, void* stream) {
  if (num_indexes < 1 || outer < 0 || gather_dim < 1 || inner < 1) return SB200_ERR_BAD_ARGUMENT;
  if (outer == 0) return SB200_OK;
  if (x == nullptr || y == nullptr || indexes == nullptr || x == y) return SB200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(indexes)) & 3u)
    return SB200_ERR_BAD_ARGUMENT;
  if (outer * num_indexes > (1ll << 40) / inner || outer * gather_dim > (1ll << 40) / inner) return SB200_ERR_UNSUPPORTED;
  const int64_t count = outer * num_indexes * inner;
  if ((inner & 3) == 0 && aligned16(x) && aligned16(y) && count / 4 < (1ll << 32) && num_indexes < (1ll << 32)) {
    const int64_t count4 = count / 4, per_block = kThreads * kGatherU;
    gather_vec_kernel<<<static_cast<unsigned>((count4 + per_block - 1) / per_block), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(x), indexes, reinterpret_cast<float4*>(y), static_cast<uint32_t>(count4),
        static_cast<uint32_t>(num_indexes), gather_dim, static_cast<uint32_t>(inner / 4),
        FastDiv32(static_cast<uint32_t>(inner / 4)), FastDiv32(static_cast<uint32_t>(num_indexes)));
    return after_launch("sb200_gather");
  }
  const int64_t blocks = (count + kThreads - 1) / kThreads;
  if (blocks >= (1ll << 31)) return SB200_ERR_UNSUPPORTED;
  const FastDiv32 div_inner(static_cast<uint32_t>(inner < (1ll << 32) ? inner : 1));
  const FastDiv32 div_num(static_cast<uint32_t>(num_indexes < (1ll << 32) ? num_indexes : 1));
  gather_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      x, indexes, y, count, num_indexes, gather_dim, inner, div_inner, div_num);
  return after_launch("sb200_gather");
}

int sb200_pad(const float* x, float* y, int64_t planes, int in_h, int in_w, const int* paddings, float value,
              void* stream) {
  if (paddings == nullptr || planes < 0 || in_h < 1 || in_w < 1) return SB200_ERR_BAD_ARGUMENT;
  const int64_t out_h = static_cast<int64_t>(in_h) + paddings[0] + paddings[1];
  const int64_t out_w = static_cast<int64_t>(in_w) + paddings[2] + paddings[3];
  if (out_h < 1 || out_w < 1 || out_h >= (1ll << 31) || out_w >= (1ll << 31)) return SB200_ERR_BAD_ARGUMENT;
  if (planes == 0) return SB200_OK;
  if (x == nullptr || y == nullptr || x == y) return SB200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 3u) return SB200_ERR_BAD_ARGUMENT;
  if (planes > (1ll << 40) / (out_h * out_w)) return SB200_ERR_UNSUPPORTED;
  const int64_t total = planes * out_h * out_w;
  const int64_t rows_all = planes * out_h;
  const int64_t band_rows = (24 * 1024) / (out_w * 4) > 0 ? (24 * 1024) / (out_w * 4) : 1;
  if (paddings[0] >= 0 && paddings[1] >= 0 && paddings[2] >= 0 && paddings[3] >= 0 && (in_w & 3) == 0 && aligned16(x) &&
      aligned16(y) && rows_all < (1ll << 31) && (band_rows * out_w + 8) * 4 <= 47 * 1024 && band_rows * out_w < (1ll << 24)) {
    PadBand q;
    q.rows_per_block = static_cast<int>(band_rows);
    q.total_rows = static_cast<uint32_t>(rows_all);
    q.div_w4 = FastDiv32(static_cast<uint32_t>(in_w / 4));
    q.div_in_h = FastDiv32(static_cast<uint32_t>(in_h));
    q.div_out_h = FastDiv32(static_cast<uint32_t>(out_h));
    const int64_t blocks = (rows_all + band_rows - 1) / band_rows;
    const int smem = static_cast<int>((band_rows * out_w + 8) * 4);
    pad_smem_kernel<<<static_cast<unsigned>(blocks), kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        x, y, in_h, in_w, static_cast<int>(out_h), static_cast<int>(out_w), paddings[0], paddings[2], value, q);
    return after_launch("sb200_pad");
  }
  if (aligned16(y) && total < (1ll << 32)) {
    const int64_t blocks4 = ((total + 3) / 4 + kThreads - 1) / kThreads;
    pad_vec_kernel<<<static_cast<unsigned>(blocks4), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        x, y, total, in_h, in_w, static_cast<int>(out_h), static_cast<int>(out_w), paddings[0], paddings[2], value,
        FastDiv32(static_cast<uint32_t>(out_w)), FastDiv32(static_cast<uint32_t>(out_h)));
    return after_launch("sb200_pad");
  }
  const int64_t rows = planes * out_h;
  const int runs_per_row = static_cast<int>((out_w + kPadRun - 1) / kPadRun);
  const int64_t threads = rows * runs_per_row;
  if (threads >= (1ll << 32)) return SB200_ERR_UNSUPPORTED;   // 32-bit index decode in the kernel
  const int64_t blocks = (threads + kThreads - 1) / kThreads;
  pad_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      x, y, rows, in_h, in_w, static_cast<int>(out_h), static_cast<int>(out_w), paddings[0], paddings[2], value, runs_per_row,
      FastDiv32(static_cast<uint32_t>(runs_per_row)), FastDiv32(static_cast<uint32_t>(out_h)));
  return after_launch("sb200_pad");
}

}  // extern "C"
