// N-d broadcast binary: y = a (op) b where each input dim equals the output dim or is 1.
//
// Host side: drop output dims of size 1, merge neighbouring dims whose broadcast state is the same
// for both inputs, and turn what is left (at most 8 dims) into per-dim extents, input strides (0 on
// a broadcast dim) and exact fast-division constants, all passed to the kernel BY VALUE: no shape
// tables in device memory, no upload, no scratch.
//
// Device side, two kernels:
//  * row-vector kernel (innermost collapsed extent L % 4 == 0, 16-byte aligned pointers): a
//    thread owns a float4 of the output; the outer coordinates are decoded once per float4 with
//    mul-hi divisions; an input that is contiguous along the innermost dim is read as float4, an
//    input that is broadcast along it is read once as a scalar.  An input that is broadcast
//    anywhere is re-read many times, so it is loaded through the normal (L2-retaining) path while
//    the output and a never-repeated input use streaming accesses that do not displace it.
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
constexpr int kBlocksPerSm = 8;

struct BcastGeom {
  int ndim;                    // collapsed dims, outermost first
  uint32_t extent[kMaxDims];   // output extent per dim
  int64_t a_stride[kMaxDims];  // element strides, 0 where the input is broadcast
  int64_t b_stride[kMaxDims];
  FastDiv32 div[kMaxDims];     // division by extent[k]
  FastDiv32 div_inner4;        // division by extent[ndim-1]/4 (row-vector kernel)
  int64_t total;               // output elements
  bool a_repeats, b_repeats;   // input has a broadcast dim (is read more than once)
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
  for (uint64_t base = static_cast<uint64_t>(blockIdx.x) * kTile; base < nvec;
       base += static_cast<uint64_t>(gridDim.x) * kTile) {
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
}

// Generic: any geometry.  WIDE selects 64-bit index arithmetic (more than 2^32-1 output elements).
template <typename F, bool WIDE>
__global__ void __launch_bounds__(kThreads)
bcast_elem_kernel(const float* a, const float* b, float* y, const __grid_constant__ BcastGeom g, F f) {
  constexpr int64_t kTile = static_cast<int64_t>(kThreads) * kUnroll;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * kTile; base < g.total;
       base += static_cast<int64_t>(gridDim.x) * kTile) {
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
        va[u] = __ldg(a + ao);
        vb[u] = __ldg(b + bo);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + threadIdx.x + u * kThreads;
      if (i < g.total) y[i] = f(va[u], vb[u]);
    }
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

template <int OP>
int run(const float* a, const float* b, float* y, const BcastGeom& g, cudaStream_t s) {
  using F = BinaryFn<OP>;
  const int last = g.ndim - 1;
  const bool a_inner = g.a_stride[last] == 1, b_inner = g.b_stride[last] == 1;
  const bool vec_ok = (g.extent[last] % 4 == 0) && aligned16(y) && aligned16(a) && aligned16(b) &&
                      (g.total >> 2) < 0xffffffffll && (a_inner || b_inner);
  if (vec_ok) {
    const int64_t nvec = g.total >> 2;
    const unsigned grid = stream_grid((nvec + kThreads * kUnroll - 1) / (kThreads * kUnroll), kBlocksPerSm);
    if (a_inner && b_inner) launch_rowvec<F, true, true>(a, b, y, g, F(), grid, s);
    else if (a_inner) launch_rowvec<F, true, false>(a, b, y, g, F(), grid, s);
    else launch_rowvec<F, false, true>(a, b, y, g, F(), grid, s);
  } else {
    const unsigned grid = stream_grid((g.total + kThreads * kUnroll - 1) / (kThreads * kUnroll), kBlocksPerSm);
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
