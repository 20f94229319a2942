// N-d broadcast binary: y = a (op) b where each input dim equals the output dim or is 1.
//
// Host side: drop output dims of size 1, merge neighbouring dims whose broadcast state is the same
// for both inputs, and turn what is left (at most 8 dims) into per-dim extents, input strides (0 on
// a broadcast dim) and exact fast-division constants, all passed to the kernel BY VALUE: no shape
// tables in device memory, no upload, no scratch.
//
// Device side, three kernels, all with one block per tile of the output (see elementwise.cu):
//  * row-vector kernel (innermost collapsed extent L % 4 == 0, 16-byte aligned pointers): a
//    thread owns a float4 of the output; the outer coordinates are decoded once per float4 with
//    mul-hi divisions; an input that is contiguous along the innermost dim is read as float4, an
//    input that is broadcast along it is read once as a scalar.  An input that is broadcast
//    anywhere is re-read many times, so it is loaded through the normal (L2-retaining) path while
//    the output and a never-repeated input use streaming accesses that do not displace it.
//  * reuse kernel: same, but when a LARGE input is broadcast along some outer dim j (for example
//    A[8,1,2048,2048] against an output [8,16,2048,2048]) the thread keeps that input's float4 in
//    registers and walks dim j itself, so the input crosses L2 once instead of extent_j times.
//  * element kernel: one element per thread slot, any geometry (ragged inner extents, unaligned
//    pointers, more than 2^32 elements through 64-bit division).
// Algorithmic bytes: 4*(|a| + |b| + |y|).
#include "common.cuh"
#include "math.cuh"

namespace sb200 {
namespace {

constexpr int kMaxDims = 8;
constexpr int kThreads = 256;
constexpr int kUnroll = 4;

struct BcastGeom {
  int ndim;                    // collapsed dims, outermost first
  uint32_t extent[kMaxDims];   // output extent per dim
  int64_t a_stride[kMaxDims];  // element strides, 0 where the input is broadcast
  int64_t b_stride[kMaxDims];
  FastDiv32 div[kMaxDims];     // division by extent[k]
  FastDiv32 div_inner4;        // division by extent[ndim-1]/4 (row-vector kernel)
  int64_t total;               // output elements
  bool a_repeats, b_repeats;   // input has a broadcast dim (is read more than once)
  // reuse kernel: dim `loop_dim` of the ORIGINAL collapsed geometry is walked inside the thread;
  // extent/strides above then describe the remaining dims and y_stride their output strides.
  int64_t y_stride[kMaxDims];
  uint32_t loop_extent;
  int64_t loop_y_stride, loop_a_stride, loop_b_stride;
};

template <bool REPEATS>
__device__ __forceinline__ float4 load4(const float* p) {
  return REPEATS ? __ldg(reinterpret_cast<const float4*>(p)) : __ldcs(reinterpret_cast<const float4*>(p));
}
template <bool REPEATS>
__device__ __forceinline__ float load1(const float* p) {
  return REPEATS ? __ldg(p) : __ldcs(p);
}

// A_INNER / B_INNER: the input is contiguous (stride 1) along the innermost collapsed dim; otherwise
// it is broadcast along it (stride 0).
template <typename F, bool A_INNER, bool B_INNER, bool A_REP, bool B_REP>
__global__ void __launch_bounds__(kThreads)
bcast_rowvec_kernel(const float* a, const float* b, float* y, const __grid_constant__ BcastGeom g, F f) {
  const uint32_t nvec = static_cast<uint32_t>(g.total >> 2);
  const int last = g.ndim - 1;
  constexpr uint32_t kTile = kThreads * kUnroll;
  float4* y4 = reinterpret_cast<float4*>(y);
  const uint64_t base = static_cast<uint64_t>(blockIdx.x) * kTile;
  float4 va[kUnroll], vb[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const uint64_t v64 = base + threadIdx.x + u * kThreads;
    if (v64 < nvec) {
      const uint32_t v = static_cast<uint32_t>(v64);
      uint32_t row, p4;
      g.div_inner4.divmod(v, row, p4);
      int64_t ao = A_INNER ? static_cast<int64_t>(p4) << 2 : 0;
      int64_t bo = B_INNER ? static_cast<int64_t>(p4) << 2 : 0;
#pragma unroll
      for (int k = kMaxDims - 2; k >= 0; --k) {
        if (k < last) {
          uint32_t q, c;
          g.div[k].divmod(row, q, c);
          row = q;
          ao += static_cast<int64_t>(c) * g.a_stride[k];
          bo += static_cast<int64_t>(c) * g.b_stride[k];
        }
      }
      if (A_INNER) va[u] = load4<A_REP>(a + ao);
      else { float s = load1<A_REP>(a + ao); va[u] = make_float4(s, s, s, s); }
      if (B_INNER) vb[u] = load4<B_REP>(b + bo);
      else { float s = load1<B_REP>(b + bo); vb[u] = make_float4(s, s, s, s); }
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const uint64_t v64 = base + threadIdx.x + u * kThreads;
    if (v64 < nvec) {
      float4 r = make_float4(f(va[u].x, vb[u].x), f(va[u].y, vb[u].y), f(va[u].z, vb[u].z),
                             f(va[u].w, vb[u].w));
      st_stream(y4 + v64, r);
    }
  }
}

// Reuse kernel.  The thread space is the output with dim `loop` removed (total/loop_extent/4
// float4 slots); each thread walks the removed dim.  A_LOOP / B_LOOP: the input varies along the
// walked dim (it is re-loaded every step) or not (loaded once, kept in registers).
template <typename F, bool A_INNER, bool B_INNER, bool A_LOOP, bool B_LOOP>
__global__ void __launch_bounds__(kThreads)
bcast_reuse_kernel(const float* a, const float* b, float* y, const __grid_constant__ BcastGeom g, F f) {
  const uint32_t nvec = static_cast<uint32_t>((g.total / g.loop_extent) >> 2);
  const int last = g.ndim - 1;
  const uint64_t v64 = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (v64 >= nvec) return;
  uint32_t row, p4;
  g.div_inner4.divmod(static_cast<uint32_t>(v64), row, p4);
  int64_t ao = A_INNER ? static_cast<int64_t>(p4) << 2 : 0;
  int64_t bo = B_INNER ? static_cast<int64_t>(p4) << 2 : 0;
  int64_t yo = static_cast<int64_t>(p4) << 2;
#pragma unroll
  for (int k = kMaxDims - 2; k >= 0; --k) {
    if (k < last) {
      uint32_t q, c;
      g.div[k].divmod(row, q, c);
      row = q;
      ao += static_cast<int64_t>(c) * g.a_stride[k];
      bo += static_cast<int64_t>(c) * g.b_stride[k];
      yo += static_cast<int64_t>(c) * g.y_stride[k];
    }
  }
  // the walked input: cached read-only path if it repeats elsewhere (then it cannot alias y),
  // streaming load if every element is used once
  auto fetch = [](const float* p, bool inner, bool repeats) {
    if (inner) return repeats ? __ldg(reinterpret_cast<const float4*>(p)) : ld_stream(reinterpret_cast<const float4*>(p));
    float s = repeats ? __ldg(p) : ld_stream(p);
    return make_float4(s, s, s, s);
  };
  float4 ka = make_float4(0.f, 0.f, 0.f, 0.f), kb = ka;
  if (!A_LOOP) ka = ld_stream(reinterpret_cast<const float4*>(a + ao));   // the reused input: read exactly once
  if (!B_LOOP) kb = ld_stream(reinterpret_cast<const float4*>(b + bo));
  constexpr int kStep = 4;
  for (uint32_t e0 = 0; e0 < g.loop_extent; e0 += kStep) {
    float4 xa[kStep], xb[kStep];
#pragma unroll
    for (int j = 0; j < kStep; ++j) {
      const uint32_t e = e0 + j;
      if (e < g.loop_extent) {
        xa[j] = A_LOOP ? fetch(a + ao + static_cast<int64_t>(e) * g.loop_a_stride, A_INNER, g.a_repeats) : ka;
        xb[j] = B_LOOP ? fetch(b + bo + static_cast<int64_t>(e) * g.loop_b_stride, B_INNER, g.b_repeats) : kb;
      }
    }
#pragma unroll
    for (int j = 0; j < kStep; ++j) {
      const uint32_t e = e0 + j;
      if (e < g.loop_extent) {
        float4 r = make_float4(f(xa[j].x, xb[j].x), f(xa[j].y, xb[j].y), f(xa[j].z, xb[j].z), f(xa[j].w, xb[j].w));
        st_stream(reinterpret_cast<float4*>(y + yo + static_cast<int64_t>(e) * g.loop_y_stride), r);
      }
    }
  }
}

// Generic: any geometry.  WIDE selects 64-bit index arithmetic (more than 2^32-1 output elements).
template <typename F, bool WIDE>
__global__ void __launch_bounds__(kThreads)
bcast_elem_kernel(const float* a, const float* b, float* y, const __grid_constant__ BcastGeom g, F f) {
  constexpr int64_t kTile = static_cast<int64_t>(kThreads) * kUnroll;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
  float va[kUnroll], vb[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + threadIdx.x + u * kThreads;
    if (i < g.total) {
      int64_t ao = 0, bo = 0;
      if (WIDE) {
        int64_t cc = i;
        for (int k = g.ndim - 1; k >= 0; --k) {
          int64_t q = cc / g.extent[k];
          int64_t c = cc - q * g.extent[k];
          cc = q;
          ao += c * g.a_stride[k];
          bo += c * g.b_stride[k];
        }
      } else {
        uint32_t cc = static_cast<uint32_t>(i);
#pragma unroll
        for (int k = kMaxDims - 1; k >= 0; --k) {
          if (k < g.ndim) {
            uint32_t q, c;
            g.div[k].divmod(cc, q, c);
            cc = q;
            ao += static_cast<int64_t>(c) * g.a_stride[k];
            bo += static_cast<int64_t>(c) * g.b_stride[k];
          }
        }
      }
      va[u] = a[ao];   // plain loads: an input may alias y (in-place)
      vb[u] = b[bo];
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + threadIdx.x + u * kThreads;
    if (i < g.total) y[i] = f(va[u], vb[u]);
  }
}

// Returns SB200_OK and fills g, or an error.
int collapse(const int* a_shape, const int* b_shape, const int* out_shape, int num_axes, BcastGeom* g) {
  if (num_axes < 1 || num_axes > SB200_MAX_AXES) return SB200_ERR_BAD_ARGUMENT;
  int64_t ext[SB200_MAX_AXES];
  bool ab[SB200_MAX_AXES], bb[SB200_MAX_AXES];  // input is broadcast on this dim
  int nd = 0;
  int64_t total = 1;
  for (int n = 0; n < num_axes; ++n) {
    const int o = out_shape[n], da = a_shape[n], db = b_shape[n];
    if (o < 1 || !(da == o || da == 1) || !(db == o || db == 1)) return SB200_ERR_BAD_ARGUMENT;
    if (o != (da > db ? da : db)) return SB200_ERR_BAD_ARGUMENT;
    total *= o;
    if (total > (1ll << 40)) return SB200_ERR_UNSUPPORTED;
    if (o == 1) continue;  // contributes nothing to any index
    const bool a_b = (da == 1), b_b = (db == 1);
    if (nd > 0 && ab[nd - 1] == a_b && bb[nd - 1] == b_b) {
      ext[nd - 1] *= o;
    } else {
      ext[nd] = o, ab[nd] = a_b, bb[nd] = b_b;
      ++nd;
    }
  }
  if (nd == 0) {  // every dim is 1: a single element
    ext[0] = 1, ab[0] = bb[0] = false;
    nd = 1;
  }
  if (nd > kMaxDims) return SB200_ERR_UNSUPPORTED;
  g->ndim = nd;
  g->total = total;
  g->a_repeats = g->b_repeats = false;
  int64_t as = 1, bs = 1;
  for (int k = nd - 1; k >= 0; --k) {
    g->extent[k] = static_cast<uint32_t>(ext[k]);
    if (ext[k] > 0xffffffffll) return SB200_ERR_UNSUPPORTED;
    g->div[k] = FastDiv32(static_cast<uint32_t>(ext[k]));
    g->a_stride[k] = ab[k] ? 0 : as;
    g->b_stride[k] = bb[k] ? 0 : bs;
    if (ab[k]) g->a_repeats = true; else as *= ext[k];
    if (bb[k]) g->b_repeats = true; else bs *= ext[k];
  }
  for (int k = nd; k < kMaxDims; ++k) {
    g->extent[k] = 1, g->a_stride[k] = g->b_stride[k] = 0;
    g->div[k] = FastDiv32(1);
  }
  for (int k = 0; k < kMaxDims; ++k) g->y_stride[k] = 0;
  g->loop_extent = 1, g->loop_y_stride = g->loop_a_stride = g->loop_b_stride = 0;
  const uint32_t inner = g->extent[nd - 1];
  g->div_inner4 = FastDiv32(inner >= 4 ? inner / 4 : 1);
  return SB200_OK;
}

template <typename F, bool AI, bool BI>
void launch_rowvec(const float* a, const float* b, float* y, const BcastGeom& g, F f, unsigned grid,
                   cudaStream_t s) {
  if (g.a_repeats && g.b_repeats) bcast_rowvec_kernel<F, AI, BI, true, true><<<grid, kThreads, 0, s>>>(a, b, y, g, f);
  else if (g.a_repeats) bcast_rowvec_kernel<F, AI, BI, true, false><<<grid, kThreads, 0, s>>>(a, b, y, g, f);
  else if (g.b_repeats) bcast_rowvec_kernel<F, AI, BI, false, true><<<grid, kThreads, 0, s>>>(a, b, y, g, f);
  else bcast_rowvec_kernel<F, AI, BI, false, false><<<grid, kThreads, 0, s>>>(a, b, y, g, f);
}

// Picks the dim the reuse kernel walks: an outer dim along which exactly one input is broadcast,
// where that input is large enough (>= 1 MB) for the saved L2 traffic to matter.  Returns -1 if
// there is none.  `*reuse_a` tells which input stays in registers.
int pick_loop_dim(const BcastGeom& g, int64_t a_elems, int64_t b_elems, bool* reuse_a) {
  int best = -1;
  int64_t best_gain = 0;
  for (int k = 0; k < g.ndim - 1; ++k) {
    const bool ab = g.a_stride[k] == 0, bb = g.b_stride[k] == 0;
    if (ab == bb || g.extent[k] < 2) continue;
    const int64_t reused = ab ? a_elems : b_elems;
    if (reused < (1 << 18)) continue;
    const int64_t gain = reused * (g.extent[k] - 1);
    if (gain > best_gain) best_gain = gain, best = k, *reuse_a = ab;
  }
  return best;
}

template <typename F, bool AI, bool BI>
void launch_reuse(const float* a, const float* b, float* y, const BcastGeom& g, bool reuse_a, F f,
                  unsigned grid, cudaStream_t s) {
  if (reuse_a) bcast_reuse_kernel<F, AI, BI, false, true><<<grid, kThreads, 0, s>>>(a, b, y, g, f);
  else bcast_reuse_kernel<F, AI, BI, true, false><<<grid, kThreads, 0, s>>>(a, b, y, g, f);
}

template <int OP>
int run(const float* a, const float* b, float* y, const BcastGeom& g, cudaStream_t s) {
  using F = BinaryFn<OP>;
  const int last = g.ndim - 1;
  const bool a_inner = g.a_stride[last] == 1, b_inner = g.b_stride[last] == 1;
  const bool vec_ok = (g.extent[last] % 4 == 0) && aligned16(y) && aligned16(a) && aligned16(b) &&
                      (g.total >> 2) < 0xffffffffll && (a_inner || b_inner);
  if (vec_ok) {
    int64_t a_elems = 1, b_elems = 1;
    for (int k = 0; k < g.ndim; ++k) {
      if (g.a_stride[k] != 0) a_elems *= g.extent[k];
      if (g.b_stride[k] != 0) b_elems *= g.extent[k];
    }
    bool reuse_a = false;
    const int loop = pick_loop_dim(g, a_elems, b_elems, &reuse_a);
    // the reused input must be contiguous along the innermost dim (it is kept as a float4)
    if (loop >= 0 && (reuse_a ? a_inner : b_inner)) {
      BcastGeom r = g;   // geometry with dim `loop` taken out
      int64_t ys[kMaxDims], stride = 1;
      for (int k = g.ndim - 1; k >= 0; --k) { ys[k] = stride; stride *= g.extent[k]; }
      r.loop_extent = g.extent[loop];
      r.loop_y_stride = ys[loop], r.loop_a_stride = g.a_stride[loop], r.loop_b_stride = g.b_stride[loop];
      int n = 0;
      for (int k = 0; k < g.ndim; ++k) {
        if (k == loop) continue;
        r.extent[n] = g.extent[k], r.a_stride[n] = g.a_stride[k], r.b_stride[n] = g.b_stride[k];
        r.div[n] = g.div[k], r.y_stride[n] = ys[k];
        ++n;
      }
      for (int k = n; k < kMaxDims; ++k) {
        r.extent[k] = 1, r.a_stride[k] = r.b_stride[k] = r.y_stride[k] = 0, r.div[k] = FastDiv32(1);
      }
      r.ndim = n;
      const int64_t nvec = (g.total / r.loop_extent) >> 2;
      const unsigned grid = tile_grid(nvec, kThreads);
      if (a_inner && b_inner) launch_reuse<F, true, true>(a, b, y, r, reuse_a, F(), grid, s);
      else if (a_inner) launch_reuse<F, true, false>(a, b, y, r, reuse_a, F(), grid, s);
      else launch_reuse<F, false, true>(a, b, y, r, reuse_a, F(), grid, s);
    } else {
      const unsigned grid = tile_grid(g.total >> 2, kThreads * kUnroll);
      if (a_inner && b_inner) launch_rowvec<F, true, true>(a, b, y, g, F(), grid, s);
      else if (a_inner) launch_rowvec<F, true, false>(a, b, y, g, F(), grid, s);
      else launch_rowvec<F, false, true>(a, b, y, g, F(), grid, s);
    }
  } else {
    const unsigned grid = tile_grid(g.total, kThreads * kUnroll);
    if (g.total < 0xffffffffll) bcast_elem_kernel<F, false><<<grid, kThreads, 0, s>>>(a, b, y, g, F());
    else bcast_elem_kernel<F, true><<<grid, kThreads, 0, s>>>(a, b, y, g, F());
  }
  return after_launch("sb200_binary_broadcast");
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" int sb200_binary_broadcast(const float* a, const int* a_shape, const float* b,
                                      const int* b_shape, const int* out_shape, int num_axes, float* y,
                                      int operation, void* stream) {
  if (a == nullptr || b == nullptr || y == nullptr || a_shape == nullptr || b_shape == nullptr ||
      out_shape == nullptr)
    return SB200_ERR_BAD_ARGUMENT;
  if (operation < SB200_ADD || operation > SB200_MIN) return SB200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(y)) & 3u)
    return SB200_ERR_BAD_ARGUMENT;
  BcastGeom g;
  int rc = collapse(a_shape, b_shape, out_shape, num_axes, &g);
  if (rc != SB200_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (operation) {
    case SB200_ADD: return run<SB200_ADD>(a, b, y, g, s);
    case SB200_SUB: return run<SB200_SUB>(a, b, y, g, s);
    case SB200_MUL: return run<SB200_MUL>(a, b, y, g, s);
    case SB200_DIV: return run<SB200_DIV>(a, b, y, g, s);
    case SB200_POW: return run<SB200_POW>(a, b, y, g, s);
    case SB200_MAX: return run<SB200_MAX>(a, b, y, g, s);
    default: return run<SB200_MIN>(a, b, y, g, s);
  }
}
