/*
 * raft_b200_mg - row-sharded forms of the dense reductions over the GPUs of one node, driven by ONE
 * host process (libraft_b200_mg.so; needs libraft_b200.so and NCCL).
 *
 * The reference has no multi-GPU form of these primitives. What it has is the single-process handle
 * that owns one NCCL communicator per device (core/device_resources_snmg.hpp:36-120, communicators
 * created with ncclCommInitAll in core/resource/nccl_comm.hpp:22-30); b2r_mg_comm is the
 * counterpart of that handle for this library, and b2r_mg_comm_adopt takes the communicators such a
 * handle already holds.
 *
 * The matrix is sharded by contiguous row blocks, shard d on device d:
 *   - one output per ROW (row norms, row sums, row argmin): every device writes the outputs of its
 *     own rows; nothing is exchanged;
 *   - one output per COLUMN, and keyed row sums: every device reduces its shard without final_op,
 *     the partials are all-reduced with NCCL (sum / min / max), final_op runs on every device; all
 *     devices end up with the full result.
 * Everything is asynchronous: the work of device d is enqueued on streams[d] (or on the
 * communicator's own stream of that device when `streams` is NULL); b2r_mg_sync waits for the own
 * streams. Calls on one communicator must not overlap in time (NCCL's rule for one host thread
 * driving several devices).
 */
#ifndef RAFT_B200_MG_H
#define RAFT_B200_MG_H

#include "raft_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b2r_mg_comm b2r_mg_comm;

/* Communicator over `n_devices` CUDA devices (ordinals in `devices`, all different): creates the
 * NCCL communicators (ncclCommInitAll) and one non-blocking stream per device. */
B2R_API int b2r_mg_comm_create(b2r_mg_comm** comm, const int* devices, int n_devices);

/* Same, on NCCL communicators the caller owns (`nccl_comms[d]` is the ncclComm_t of devices[d], e.g.
 * raft::resource::get_nccl_comms(handle)[d] of a device_resources_snmg, core/resource/nccl_comm.hpp:70-95);
 * they are not destroyed by b2r_mg_comm_destroy. */
B2R_API int b2r_mg_comm_adopt(b2r_mg_comm** comm, const int* devices, int n_devices, void* const* nccl_comms);

B2R_API int b2r_mg_comm_destroy(b2r_mg_comm* comm);
B2R_API int b2r_mg_comm_size(const b2r_mg_comm* comm);

/* Waits for the communicator's own streams (not for caller streams). */
B2R_API int b2r_mg_sync(b2r_mg_comm* comm);

/*
 * Sharded raft::linalg::reduce (linalg/reduce.cuh:55-76). `desc` describes ONE shard except for
 * n_rows, which is taken from shard_rows[d]; ins[d] / outs[d] are device pointers on device d.
 * ALONG_ROWS: outs[d] receives shard_rows[d] outputs. ALONG_COLUMNS: every outs[d] receives all
 * n_cols outputs; reduce_op must be add, min or max; `inplace` is refused (B2R_ERR_UNSUPPORTED).
 */
B2R_API int b2r_mg_reduce(b2r_mg_comm* comm,
                          const b2r_reduce_desc* desc,
                          void* const* outs,
                          const void* const* ins,
                          const int64_t* shard_rows,
                          const b2r_stream_t* streams);

/*
 * Sharded raft::linalg::reduce_rows_by_key (linalg/reduce_rows_by_key.cuh:52-116): keys and weights
 * are sharded with the rows. Every sums[d] ([nkeys x ncols]) and counts[d] (int64 [nkeys]; `counts`
 * may be NULL, single entries may not) receives the result over ALL shards. `reset` zero adds the
 * result to the table DEVICE 0 held before the call (what an earlier call left is the same on
 * every device).
 */
B2R_API int b2r_mg_reduce_rows_by_key(b2r_mg_comm* comm,
                                      void* const* sums,
                                      int64_t* const* counts,
                                      const void* const* A,
                                      int64_t lda,
                                      const void* const* keys,
                                      const void* const* weights,
                                      int32_t data_dtype,
                                      int32_t key_dtype,
                                      const int64_t* shard_rows,
                                      int64_t ncols,
                                      int64_t nkeys,
                                      int32_t reset,
                                      const b2r_stream_t* streams);

#ifdef __cplusplus
}
#endif
#endif /* RAFT_B200_MG_H */
