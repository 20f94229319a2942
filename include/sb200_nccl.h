/*
 * sb200_nccl - C ABI of the cross-GPU combine step for tensors sharded on their outermost dimension
 * (`libsb200_nccl.so`; links `libsb200.so` and NCCL, so that `libsb200.so` itself keeps depending on
 * nothing but the CUDA runtime).
 *
 * The reference is single-device: its multi-device model is one Network per device_id
 * (shadow/core/context.cu:10-15, shadow/core/network_impl.hpp:16-25), each driven by its own host
 * thread or process, with no exchange between them.  A host that shards a tensor over such
 * Networks needs exactly one exchange on this path: the partial results of a reduction that runs
 * over the sharded dimension.  These entry points provide it to a C or C++ host; none of them has a
 * counterpart in the reference.
 *
 * One communicator per (process, device).  Every rank makes the same sequence of calls; a call
 * enqueues on `stream` (cudaStream_t as void*) and returns without synchronising, like the rest of
 * the ABI.  Status codes are those of sb200.h plus SB200_ERR_COMM.
 */
#ifndef SB200_NCCL_H_
#define SB200_NCCL_H_

#include <stdint.h>

#include "sb200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define SB200_ERR_COMM 5          /* an NCCL call failed; see sb200_comm_last_error */
#define SB200_COMM_ID_BYTES 128   /* size of the opaque identifier that rank 0 hands to the others */

/* Text of the calling thread's last SB200_ERR_COMM ("" if none). */
const char* sb200_comm_last_error(void);

/* Rank 0 creates the identifier (ncclGetUniqueId) and ships its SB200_COMM_ID_BYTES bytes to the
 * other ranks by any means the host has (a file, a socket, MPI, a torch store). */
int sb200_comm_new_id(void* id_out);
/* Collective over all ranks: creates this rank's communicator on the CURRENT device
 * (ncclCommInitRank).  `*comm_out` is an opaque handle. */
int sb200_comm_create(const void* id, int n_ranks, int rank, void** comm_out);
int sb200_comm_destroy(void* comm);
int sb200_comm_query(void* comm, int* n_ranks_out, int* rank_out);

/* All-reduce of double partials in place (sum / product / max / min chosen by the REDUCTION's
 * operation code SB200_RED_*: Sum, Avg, L1 and L2 partials add, Prod multiplies, Max and Min
 * take the extremum).  partial: `count` doubles written by sb200_reduce_partial.  The order in
 * which NCCL combines ranks is its own; use the gather form below where the bits must not depend
 * on it.  sb200_allreduce_scalar is the count == 1 case (a full-tensor reduction). */
int sb200_allreduce_partials(void* comm, double* partial, int64_t count, int operation, void* stream);
int sb200_allreduce_scalar(void* comm, double* partial, int operation, void* stream);

/* All-gather of one record per rank: gathered[r * record_doubles + i] = rank r's record[i].
 * A record may carry the partials of several reductions back to back. */
int sb200_allgather_records(void* comm, const double* record, double* gathered, int64_t record_doubles, void* stream);

/* Gather and finish in one call: all-gathers the records, then for reduction i (operation
 * operations[i], partials at record[i * count .. (i + 1) * count)) folds the n_ranks partials of every
 * output in rank order (sb200_reduce_combine) into y[i][0 .. count).  Deterministic: every rank
 * computes the same bits whatever the communicator's topology.
 *   record_doubles >= n_reductions * count;  total_reduced_count = elements reduced per output
 *   over ALL ranks (used by Avg);  operations and y are HOST arrays. */
int sb200_sharded_reduce_finish(void* comm, const double* record, double* gathered, int64_t record_doubles,
                                int n_reductions, const int* operations, int64_t count, int64_t total_reduced_count,
                                float* const* y, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* SB200_NCCL_H_ */
