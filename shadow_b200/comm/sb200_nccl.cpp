// The cross-GPU combine step (include/sb200_nccl.h) over NCCL: communicator set-up from a
// caller-supplied identifier, all-reduce / all-gather of double partials on the caller's stream, and
// the gather-then-fold form that finishes several reductions with one collective.  Host code only:
// the folding kernel is sb200_reduce_combine of libsb200.so.
#include "sb200_nccl.h"

#include <cstdio>
#include <cstring>

#include <cuda_runtime.h>
#include <nccl.h>

namespace {

thread_local char g_comm_error[256] = "";

int comm_failure(ncclResult_t rc, const char* where) {
  std::snprintf(g_comm_error, sizeof(g_comm_error), "%s: %s", where, ncclGetErrorString(rc));
  return SB200_ERR_COMM;
}

struct Comm {
  ncclComm_t nccl;
  int n_ranks, rank;
};

static_assert(sizeof(ncclUniqueId) == SB200_COMM_ID_BYTES, "identifier size");

// NCCL's reduction for the partials of a SB200_RED_* reduction; false for an unknown code.
bool nccl_op_for(int operation, ncclRedOp_t* op) {
  switch (operation) {
    case SB200_RED_SUM: case SB200_RED_AVG: case SB200_RED_L1: case SB200_RED_L2: *op = ncclSum; return true;
    case SB200_RED_PROD: *op = ncclProd; return true;
    case SB200_RED_MAX: *op = ncclMax; return true;
    case SB200_RED_MIN: *op = ncclMin; return true;
    default: return false;
  }
}

}  // namespace

extern "C" {

const char* sb200_comm_last_error(void) { return g_comm_error; }

int sb200_comm_new_id(void* id_out) {
  if (id_out == nullptr) return SB200_ERR_BAD_ARGUMENT;
  ncclUniqueId id;
  const ncclResult_t rc = ncclGetUniqueId(&id);
  if (rc != ncclSuccess) return comm_failure(rc, "ncclGetUniqueId");
  std::memcpy(id_out, &id, sizeof(id));
  return SB200_OK;
}

int sb200_comm_create(const void* id, int n_ranks, int rank, void** comm_out) {
  if (id == nullptr || comm_out == nullptr || n_ranks < 1 || rank < 0 || rank >= n_ranks) return SB200_ERR_BAD_ARGUMENT;
  *comm_out = nullptr;
  ncclUniqueId uid;
  std::memcpy(&uid, id, sizeof(uid));
  ncclComm_t nccl = nullptr;
  const ncclResult_t rc = ncclCommInitRank(&nccl, n_ranks, uid, rank);
  if (rc != ncclSuccess) return comm_failure(rc, "ncclCommInitRank");
  *comm_out = new Comm{nccl, n_ranks, rank};
  return SB200_OK;
}

int sb200_comm_destroy(void* comm) {
  if (comm == nullptr) return SB200_ERR_BAD_ARGUMENT;
  Comm* c = static_cast<Comm*>(comm);
  const ncclResult_t rc = ncclCommDestroy(c->nccl);
  delete c;
  return rc == ncclSuccess ? SB200_OK : comm_failure(rc, "ncclCommDestroy");
}

int sb200_comm_query(void* comm, int* n_ranks_out, int* rank_out) {
  if (comm == nullptr) return SB200_ERR_BAD_ARGUMENT;
  const Comm* c = static_cast<const Comm*>(comm);
  if (n_ranks_out != nullptr) *n_ranks_out = c->n_ranks;
  if (rank_out != nullptr) *rank_out = c->rank;
  return SB200_OK;
}

int sb200_allreduce_partials(void* comm, double* partial, int64_t count, int operation, void* stream) {
  ncclRedOp_t op;
  if (comm == nullptr || count < 0 || !nccl_op_for(operation, &op)) return SB200_ERR_BAD_ARGUMENT;
  if (count == 0) return SB200_OK;
  if (partial == nullptr) return SB200_ERR_BAD_ARGUMENT;
  const Comm* c = static_cast<const Comm*>(comm);
  const ncclResult_t rc = ncclAllReduce(partial, partial, static_cast<size_t>(count), ncclDouble, op, c->nccl,
                                        static_cast<cudaStream_t>(stream));
  return rc == ncclSuccess ? SB200_OK : comm_failure(rc, "ncclAllReduce");
}

int sb200_allreduce_scalar(void* comm, double* partial, int operation, void* stream) {
  return sb200_allreduce_partials(comm, partial, 1, operation, stream);
}

int sb200_allgather_records(void* comm, const double* record, double* gathered, int64_t record_doubles, void* stream) {
  if (comm == nullptr || record_doubles < 0) return SB200_ERR_BAD_ARGUMENT;
  if (record_doubles == 0) return SB200_OK;
  if (record == nullptr || gathered == nullptr) return SB200_ERR_BAD_ARGUMENT;
  const Comm* c = static_cast<const Comm*>(comm);
  const ncclResult_t rc = ncclAllGather(record, gathered, static_cast<size_t>(record_doubles), ncclDouble, c->nccl,
                                        static_cast<cudaStream_t>(stream));
  return rc == ncclSuccess ? SB200_OK : comm_failure(rc, "ncclAllGather");
}

int sb200_sharded_reduce_finish(void* comm, const double* record, double* gathered, int64_t record_doubles,
                                int n_reductions, const int* operations, int64_t count, int64_t total_reduced_count,
                                float* const* y, void* stream) {
  if (comm == nullptr || n_reductions < 1 || operations == nullptr || y == nullptr || count < 1 ||
      total_reduced_count < 1 || record_doubles < static_cast<int64_t>(n_reductions) * count)
    return SB200_ERR_BAD_ARGUMENT;
  for (int i = 0; i < n_reductions; ++i) {
    ncclRedOp_t unused;
    if (y[i] == nullptr || !nccl_op_for(operations[i], &unused)) return SB200_ERR_BAD_ARGUMENT;
  }
  const int rc = sb200_allgather_records(comm, record, gathered, record_doubles, stream);
  if (rc != SB200_OK) return rc;
  const Comm* c = static_cast<const Comm*>(comm);
  for (int i = 0; i < n_reductions; ++i) {
    const int st = sb200_reduce_combine(gathered + static_cast<int64_t>(i) * count, c->n_ranks, record_doubles, y[i], count,
                                        operations[i], total_reduced_count, stream);
    if (st != SB200_OK) return st;
  }
  return SB200_OK;
}

}  // extern "C"
