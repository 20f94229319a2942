// A C++ host with one thread per device (the reference's multi-device model: one Network per device_id,
// shadow/core/context.cu:10-15) shards a tensor on dim 0 over N devices and reduces it over all axes
// through the C entry points alone: sb200_reduce_partial on every device, then ONE call of
// sb200_sharded_reduce_finish (all-gather of the records + fold in rank order).  Every rank must get the
// bits that sb200_reduce gives for the whole tensor on one device (Max) or the same sum within the
// reduction bar (Sum).  No Python, no torch: links libsb200_nccl.so, libsb200.so and the CUDA runtime.
//
//   comm_two_threads <n_devices>      exit 0 = ok, 2 = not enough devices (skipped), 1 = failure
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

#include "sb200_nccl.h"

namespace {

std::atomic<int> g_failures{0};
std::atomic<int> g_ready{0};

#define CHECK_CUDA(call)                                                                 \
  do {                                                                                   \
    cudaError_t e_ = (call);                                                             \
    if (e_ != cudaSuccess) {                                                             \
      std::fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_));                   \
      return false;                                                                      \
    }                                                                                    \
  } while (0)
#define CHECK_SB(call)                                                                   \
  do {                                                                                   \
    int s_ = (call);                                                                     \
    if (s_ != SB200_OK) {                                                                \
      std::fprintf(stderr, "%s: status %d %s %s\n", #call, s_, sb200_last_cuda_error(), sb200_comm_last_error()); \
      return false;                                                                      \
    }                                                                                    \
  } while (0)

constexpr int kBatch = 6, kC = 40, kW = 1000;   // tensor [6, 40, 1000], split on dim 0

float value_at(long long i) { return static_cast<float>(((i * 2654435761ll) % 2001) - 1000) * 1e-3f; }

// Everything a rank does BEFORE the collective; a rank that fails here must not let the others wait.
bool prepare(int rank, int n, float** x, double** record, double** gathered, float** out_sum, float** out_max, int* rows) {
  CHECK_CUDA(cudaSetDevice(rank));
  const int base = kBatch / n, extra = kBatch % n;
  const int lo = rank * base + (rank < extra ? rank : extra);
  *rows = base + (rank < extra ? 1 : 0);
  const long long count = static_cast<long long>(*rows) * kC * kW;
  std::vector<float> host(static_cast<size_t>(count));
  for (long long i = 0; i < count; ++i) host[static_cast<size_t>(i)] = value_at(static_cast<long long>(lo) * kC * kW + i);
  CHECK_CUDA(cudaMalloc(x, sizeof(float) * (count > 0 ? count : 1)));
  CHECK_CUDA(cudaMemcpy(*x, host.data(), sizeof(float) * count, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMalloc(record, sizeof(double) * 2));
  CHECK_CUDA(cudaMalloc(gathered, sizeof(double) * 2 * n));
  CHECK_CUDA(cudaMalloc(out_sum, sizeof(float)));
  CHECK_CUDA(cudaMalloc(out_max, sizeof(float)));
  return true;
}

bool partials(float* x, int rows, double* record) {
  const int shape[3] = {rows, kC, kW}, axes[3] = {0, 1, 2};
  for (int which = 0; which < 2; ++which) {
    const int op = which == 0 ? SB200_RED_SUM : SB200_RED_MAX;
    const long long need = sb200_reduce_scratch_bytes(shape, 3, axes, 3, op);
    if (need < 0) return false;
    void* scratch = nullptr;
    if (need > 0) CHECK_CUDA(cudaMalloc(&scratch, static_cast<size_t>(need)));
    CHECK_SB(sb200_reduce_partial(x, shape, 3, axes, 3, op, record + which, scratch, need, nullptr));
    CHECK_CUDA(cudaDeviceSynchronize());
    if (scratch != nullptr) CHECK_CUDA(cudaFree(scratch));
  }
  return true;
}

void rank_main(int rank, int n, const unsigned char* id, float* result) {
  float *x = nullptr, *out_sum = nullptr, *out_max = nullptr;
  double *record = nullptr, *gathered = nullptr;
  int rows = 0;
  bool ok = prepare(rank, n, &x, &record, &gathered, &out_sum, &out_max, &rows) && partials(x, rows, record);
  if (!ok) g_failures.fetch_add(1);
  // rendezvous on the host first: nobody enters a collective unless every rank got this far
  g_ready.fetch_add(1);
  while (g_ready.load() < n) std::this_thread::yield();
  if (g_failures.load() != 0) return;
  void* comm = nullptr;
  if (sb200_comm_create(id, n, rank, &comm) != SB200_OK) {
    std::fprintf(stderr, "rank %d: sb200_comm_create: %s\n", rank, sb200_comm_last_error());
    g_failures.fetch_add(1);
    return;
  }
  const int ops[2] = {SB200_RED_SUM, SB200_RED_MAX};
  float* outs[2] = {out_sum, out_max};
  int st = sb200_sharded_reduce_finish(comm, record, gathered, 2, 2, ops, 1, static_cast<long long>(kBatch) * kC * kW, outs, nullptr);
  if (st == SB200_OK && cudaDeviceSynchronize() == cudaSuccess) {
    cudaMemcpy(result, out_sum, sizeof(float), cudaMemcpyDeviceToHost);
    cudaMemcpy(result + 1, out_max, sizeof(float), cudaMemcpyDeviceToHost);
  } else {
    std::fprintf(stderr, "rank %d: sharded_reduce_finish status %d %s\n", rank, st, sb200_comm_last_error());
    g_failures.fetch_add(1);
  }
  sb200_comm_destroy(comm);
}

}  // namespace

int main(int argc, char** argv) {
  const int n = argc > 1 ? std::atoi(argv[1]) : 2;
  int devices = 0;
  if (cudaGetDeviceCount(&devices) != cudaSuccess || devices < n || n < 1) {
    std::printf("skip: %d device(s), %d wanted\n", devices, n);
    return 2;
  }
  unsigned char id[SB200_COMM_ID_BYTES];
  if (sb200_comm_new_id(id) != SB200_OK) return 1;
  std::vector<float> results(static_cast<size_t>(2 * n), 0.f);
  std::vector<std::thread> threads;
  for (int r = 0; r < n; ++r) threads.emplace_back(rank_main, r, n, id, results.data() + 2 * r);
  for (auto& t : threads) t.join();
  if (g_failures.load() != 0) return 1;
  // the whole tensor on device 0
  const long long count = static_cast<long long>(kBatch) * kC * kW;
  std::vector<float> host(static_cast<size_t>(count));
  double ref_sum = 0.0;
  float ref_max = -3.4e38f;
  for (long long i = 0; i < count; ++i) {
    host[static_cast<size_t>(i)] = value_at(i);
    ref_sum += host[static_cast<size_t>(i)];
    ref_max = host[static_cast<size_t>(i)] > ref_max ? host[static_cast<size_t>(i)] : ref_max;
  }
  int bad = 0;
  for (int r = 0; r < n; ++r) {
    const float s = results[static_cast<size_t>(2 * r)], m = results[static_cast<size_t>(2 * r + 1)];
    if (s != results[0] || m != results[1]) { std::printf("rank %d differs from rank 0: %.9g %.9g\n", r, s, m); ++bad; }
    if (m != ref_max) { std::printf("rank %d: max %.9g, expected %.9g\n", r, m, ref_max); ++bad; }
    if (std::fabs(static_cast<double>(s) - ref_sum) > 1e-5 * 18.0 * std::fabs(ref_sum) + 1e-3) { std::printf("rank %d: sum %.9g, expected %.9g\n", r, s, ref_sum); ++bad; }
  }
  std::printf("%s: %d ranks, sum %.9g (host double %.9g), max %.9g\n", bad ? "FAIL" : "ok", n, results[0], ref_sum, results[1]);
  return bad ? 1 : 0;
}
