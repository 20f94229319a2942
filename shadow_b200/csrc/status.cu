// Status strings, CUDA error capture, device queries and the launch counter.
#include <atomic>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace sb200 {
namespace {
thread_local char g_cuda_error[256] = "";
std::atomic<long long> g_launches{0};
}  // namespace

int cuda_failure(cudaError_t err, const char* where) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorString(err),
                cudaGetErrorName(err));
  return SB200_ERR_CUDA;
}

void set_error_text(const char* text) { std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s", text); }

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count() {
  // one entry per device ordinal; filled on first use with that device current
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace sb200

extern "C" {

const char* sb200_status_string(int status) {
  switch (status) {
    case SB200_OK: return "ok";
    case SB200_ERR_BAD_ARGUMENT: return "bad argument";
    case SB200_ERR_UNSUPPORTED: return "unsupported geometry";
    case SB200_ERR_CUDA: return "CUDA error";
    case SB200_ERR_SCRATCH: return "scratch buffer missing, misaligned or too small";
    default: return "unknown status";
  }
}

const char* sb200_last_cuda_error(void) { return sb200::g_cuda_error; }

int sb200_device_sm_count(void) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}

long long sb200_launch_count(void) { return sb200::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
