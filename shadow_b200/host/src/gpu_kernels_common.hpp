// Shared by the kernel-binding translation units (gpu_kernels*.cpp): status check, stream and
// element count helpers.  Uses only members that the reference's Blob / Workspace / Context have too.
#pragma once

#include <cstdint>
#include <memory>
#include <string>

#include "core/kernel.hpp"

#include "sb200.h"

namespace Shadow {

namespace {

using BlobPtr = std::shared_ptr<Blob>;

// Element count as 64 bits: the host library of this repository offers Blob::count64(), the
// reference's Blob only the int count().
template <typename B>
auto count_of(const B& blob, int) -> decltype(static_cast<int64_t>(blob->count64())) {
  return static_cast<int64_t>(blob->count64());
}
template <typename B>
int64_t count_of(const B& blob, long) {
  return static_cast<int64_t>(blob->count());
}
inline int64_t count64(const BlobPtr& blob) { return count_of(blob, 0); }

inline void expect_ok(int status, const char* what) {
  if (status != SB200_OK) {
    LOG(FATAL) << what << " failed: " << sb200_status_string(status)
               << (status == SB200_ERR_CUDA ? std::string(" - ") + sb200_last_cuda_error() : std::string());
  }
}

inline void* stream_of(Workspace* ws) { return ws->Ctx()->stream(); }

}  // namespace

}  // namespace Shadow
