// Shared device/host helpers of the sb200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "sb200.h"

namespace sb200 {

// ---- status / launch bookkeeping (host) -------------------------------------------------------

// Records the text of a failed CUDA call for sb200_last_cuda_error() and returns SB200_ERR_CUDA.
int cuda_failure(cudaError_t err, const char* where);

// Stores a message for sb200_last_cuda_error() for failures that are not CUDA errors.
void set_error_text(const char* text);

// Number of kernels this library has launched in the calling process (read by sb200_launch_count()).
void count_launch(int n = 1);

// cudaGetLastError after a launch; SB200_OK or SB200_ERR_CUDA.
inline int after_launch(const char* where) {
  count_launch();
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? SB200_OK : cuda_failure(err, where);
}

// Cached multiprocessor count of the current device (148 on B200).
int sm_count();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Grid with one block per tile of `tile` units (at least one block so that edge work still runs).
inline unsigned tile_grid(int64_t units, int64_t tile) {
  int64_t blocks = (units + tile - 1) / tile;
  if (blocks < 1) blocks = 1;
  return static_cast<unsigned>(blocks);   // callers bound sizes at 2^40 elements: < 2^31 blocks
}

// Grid for a block-stride streaming kernel: as many blocks as there are tiles, capped at
// `waves` resident blocks per SM times the SM count so the grid is a whole multiple of the SMs.
inline unsigned stream_grid(int64_t tiles, int blocks_per_sm) {
  int64_t cap = static_cast<int64_t>(sm_count()) * blocks_per_sm;
  if (tiles < 1) tiles = 1;
  return static_cast<unsigned>(tiles < cap ? tiles : cap);
}

// ---- exact unsigned division by a runtime constant --------------------------------------------
// q = n / d for 0 <= n < 2^32 (or 2^63 for the 64-bit form) using one high multiply.  The magic is
// computed on the host; the device applies it.  Round-up method: m = ceil(2^(32+s) / d) with
// s = ceil(log2 d); q = (mulhi(n, m - 2^32) + n) >> s computed in 64 bits to avoid overflow.
struct FastDiv32 {
  uint32_t d, mul, shift;
  FastDiv32() : d(1), mul(0), shift(0) {}
  explicit FastDiv32(uint32_t divisor) {
    d = divisor ? divisor : 1;
    shift = 0;
    while ((1ull << shift) < d) ++shift;
    uint64_t m = ((1ull << 32) * ((1ull << shift) - d)) / d + 1;
    mul = static_cast<uint32_t>(m);
  }
  __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const {
#ifdef __CUDA_ARCH__
    uint32_t t = __umulhi(n, mul);
#else
    uint32_t t = static_cast<uint32_t>((static_cast<uint64_t>(n) * mul) >> 32);
#endif
    return static_cast<uint32_t>((static_cast<uint64_t>(t) + n) >> shift);
  }
  __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
    q = div(n);
    r = n - q * d;
  }
};

// ---- vector memory access ---------------------------------------------------------------------
// Streaming (evict-first) 128-bit accesses: every tensor here is touched once, so lines should
// not displace anything useful in L2.  Plain (not .nc) loads so that in-place calls stay legal.
__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }
__device__ __forceinline__ float ld_stream(const float* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float* p, float v) { __stcs(p, v); }

// ---- warp / block reductions ------------------------------------------------------------------
template <typename T, typename Op>
__device__ __forceinline__ T warp_reduce(T v, Op op) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// All threads of the block get the result.  `smem` holds at least 32 T.  blockDim.x must be a
// multiple of 32.  Combination order is fixed (lane tree, then warp index order), so results are
// reproducible run to run.
template <typename T, typename Op>
__device__ __forceinline__ T block_reduce(T v, Op op, T identity, T* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  v = warp_reduce(v, op);
  __syncthreads();  // protect smem reuse between consecutive calls
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  T r = (lane < nwarp) ? smem[lane] : identity;
  r = warp_reduce(r, op);
  return r;
}

struct OpAddF { __device__ __forceinline__ float operator()(float a, float b) const { return a + b; } };
struct OpAddD { __device__ __forceinline__ double operator()(double a, double b) const { return a + b; } };
struct OpMulD { __device__ __forceinline__ double operator()(double a, double b) const { return a * b; } };
// std::max(a, b) == (a < b) ? b : a; std::min(a, b) == (b < a) ? b : a  (first argument wins ties/NaN)
struct OpMaxF { __device__ __forceinline__ float operator()(float a, float b) const { return (a < b) ? b : a; } };
struct OpMinF { __device__ __forceinline__ float operator()(float a, float b) const { return (b < a) ? b : a; } };

// ---- opting a kernel into more than 48 KB of dynamic shared memory -----------------------------------
// The attribute belongs to the (kernel, device) pair, and a process may drive several devices (one
// Network per device): `done` is one bit per device ordinal, kept by the caller per kernel
// instantiation.  Racing first calls set the same value.
template <typename Kernel>
inline void allow_dynamic_smem(Kernel kernel, int bytes, unsigned long long* done) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 63;   // ordinals past 63 share a bit: set every time
  const unsigned long long bit = 1ull << dev;
  if ((*done & bit) && dev != 63) return;
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  *done |= bit;
}

// ---- asynchronous 16-byte copies global -> shared (no register staging) ---------------------------
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

}  // namespace sb200
