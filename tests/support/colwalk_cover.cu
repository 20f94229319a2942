// Host replay of the fixed-column float4 walk (shadow_b200/csrc/colwalk.cuh): for each geometry on
// the command line (the kind of kernel that uses the layout, 0 = two passes, 1 = one pass, 2 = patch in registers, then "outer dim inner" triples) every thread of every block is replayed and the
// program checks that each float4 of the tensor is visited exactly once, that each of a thread's
// four lanes stays on one column and one (plane, column) partial, that the row arithmetic the
// kernels use for per-row scales holds, and that the shared-memory slots of a block are distinct
// and lie inside the plane's [R][ncols] array.  Prints "ok <layout>" per geometry, or the first
// violation and exits 1.  Host code only: built with nvcc because the header is a CUDA header.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "colwalk.cuh"

namespace sb200 {
int sm_count() { return 148; }
int cuda_failure(cudaError_t, const char*) { return SB200_ERR_CUDA; }
void set_error_text(const char*) {}
void count_launch(int) {}
}  // namespace sb200

using namespace sb200;

static int check(int64_t outer, int64_t dim, int64_t inner, int use) {
  ColWalk q;
  if (!plan_colwalk(reinterpret_cast<void*>(256), reinterpret_cast<void*>(512), outer, dim, inner, &q, static_cast<ColWalkUse>(use), 13)) {
    std::printf("skip %lld %lld %lld (walk does not apply)\n", (long long)outer, (long long)dim, (long long)inner);
    return 0;
  }
  const int64_t total4 = outer * dim * inner / 4;
  std::vector<unsigned char> seen(static_cast<size_t>(total4), 0);
  const int planes = q.tiled ? 1 : q.P;
  if (static_cast<int64_t>(planes) * 4 * q.tact > static_cast<int64_t>(q.threads) * 4) {
    std::printf("FAIL smem: planes %d tact %d threads %d\n", planes, q.tact, q.threads);
    return 1;
  }
  if (static_cast<int64_t>(q.R) * q.ncols > 4ll * q.tact) {
    std::printf("FAIL partial array: R %d ncols %d tact %d\n", q.R, q.ncols, q.tact);
    return 1;
  }
  for (int64_t b = 0; b < q.grid; ++b) {
    std::vector<unsigned char> slot_used(static_cast<size_t>(q.threads) * 4, 0);
    for (int t = 0; t < q.threads; ++t) {
      const ColLane L = colwalk_thread(q, static_cast<uint32_t>(t), b);
      if (L.slot >= 0) {
        for (int e = 0; e < 4; ++e) {
          const int s = L.slot + e;
          if (s < 0 || s >= q.threads * 4 || slot_used[s]) { std::printf("FAIL slot %d (block %lld thread %d)\n", s, (long long)b, t); return 1; }
          slot_used[s] = 1;
          const int c = colwalk_col(q, L, e);
          const int rel = s - L.plane_base - c;
          if (c < 0 || c >= q.ncols || rel < 0 || rel % q.ncols != 0 || rel / q.ncols >= q.R) {
            std::printf("FAIL slot layout: block %lld thread %d lane %d slot %d base %d col %d\n", (long long)b, t, e, s, L.plane_base, c);
            return 1;
          }
        }
      } else if (L.cnt != 0) { std::printf("FAIL: working thread without slot\n"); return 1; }
      if (use == 2 && L.cnt > 13) { std::printf("FAIL: thread owns %d float4, limit 13\n", L.cnt); return 1; }
      for (int j = 0; j < L.cnt; ++j) {
        const int64_t i4 = L.first4 + j * L.step4;
        if (i4 < 0 || i4 >= total4 || seen[i4]) { std::printf("FAIL cover: float4 %lld (block %lld thread %d step %d)\n", (long long)i4, (long long)b, t, j); return 1; }
        seen[i4] = 1;
        for (int e = 0; e < 4; ++e) {
          const int64_t el = i4 * 4 + e;
          const int64_t n = el / (dim * inner), in_plane = el % (dim * inner);
          const int64_t row = in_plane / inner, col = in_plane % inner;
          const int c = colwalk_col(q, L, e);
          const int64_t want_col = q.tiled ? ((b % q.ntile) * q.W4 * 4 + c) : c;
          const int64_t want_n = q.tiled ? b / q.ntile : b * q.P + (L.plane_base / (4 * q.tact));
          const int64_t want_row = L.row0 + ((!q.tiled && L.rem0 + e >= inner) ? 1 : 0) + static_cast<int64_t>(j) * q.rows_per_step;
          if (col != want_col || n != want_n || row != want_row) {
            std::printf("FAIL lane: block %lld thread %d step %d lane %d: (n,row,col) = (%lld,%lld,%lld), layout says (%lld,%lld,%lld)\n",
                        (long long)b, t, j, e, (long long)n, (long long)row, (long long)col, (long long)want_n, (long long)want_row, (long long)want_col);
            return 1;
          }
        }
      }
    }
  }
  for (int64_t i = 0; i < total4; ++i)
    if (!seen[i]) { std::printf("FAIL cover: float4 %lld never visited\n", (long long)i); return 1; }
  std::printf("ok %lld %lld %lld: %s threads %d tact %d P %d W4 %d G %d R %d grid %u\n", (long long)outer, (long long)dim, (long long)inner,
              q.tiled ? "tiled" : "flat", q.threads, q.tact, q.P, q.W4, q.G, q.R, q.grid);
  return 0;
}

int main(int argc, char** argv) {
  int bad = 0;
  if (argc < 2) return 2;
  const int use = std::atoi(argv[1]);   // first argument: how the kernel uses the layout (ColWalkUse: 0, 1 or 2)
  for (int i = 2; i + 2 < argc; i += 3) bad |= check(std::atoll(argv[i]), std::atoll(argv[i + 1]), std::atoll(argv[i + 2]), use);
  return bad;
}
