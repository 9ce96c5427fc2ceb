/*
 * candle_b200_nccl -- the vocabulary-sharded lookup as one C call (separate library, so that the
 * core one carries no NCCL dependency): libcandle_b200_nccl.so, linked against libcandle_b200.so
 * and libnccl.  Same conventions as candle_b200.h.
 *
 * The collective is the one candle has: `Comm::all_reduce(.., &ReduceOp::Sum)` wrapped as
 * `AllReduce: CustomOp1` (candle-examples/examples/llama_multiprocess/model.rs:31-90), one
 * process per GPU, the NCCL unique id passed between processes by the host
 * (llama_multiprocess/main.rs:146-173).  `comm` is an `ncclComm_t`; a Rust caller hands over the
 * handle cudarc already holds.
 */
#ifndef CANDLE_B200_NCCL_H_
#define CANDLE_B200_NCCL_H_

#include "candle_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CB200_NCCL_UNIQUE_ID_BYTES 128

/* Thin wrappers for hosts that have no NCCL binding of their own (the Python tests):
 * ncclGetUniqueId, ncclCommInitRank, ncclCommDestroy. */
CB200_API int cb200_nccl_unique_id(void* id_out /* CB200_NCCL_UNIQUE_ID_BYTES */);
CB200_API int cb200_nccl_comm_init(void** comm_out, int nranks, const void* id, int rank);
CB200_API int cb200_nccl_comm_destroy(void* comm);

/*
 * Vocabulary-sharded cb200_qembedding -> sum over ranks -> rms_norm, enqueued on `stream`:
 *   scratch = masked lookup of ALL ids in this rank's rows [vocab_begin, vocab_end) (-0.0 elsewhere)
 *   scratch = ncclAllReduce(scratch, sum)            (exact: one non-zero contributor per element)
 *   y       = rms_norm(scratch, alpha, eps)
 * `scratch` is caller-provided device memory of at least n_ids * hidden * sizeof(out_dtype)
 * bytes, 16-byte aligned; its contents after the call are the gathered rows.  The reference has
 * no such entry point: its embedding is replicated under tensor parallelism
 * (llama_multiprocess/model.rs:181-184).
 */
CB200_API int cb200_sharded_qembedding_rms_norm(void* comm, const void* qtable, int qtype, const void* ids,
                                                const void* alpha, void* y, void* scratch, size_t scratch_bytes,
                                                int64_t vocab, int32_t hidden, int64_t n_ids, float eps,
                                                int out_dtype, int id_dtype, int64_t vocab_begin,
                                                int64_t vocab_end, int flags, cb200_status* status,
                                                cb200_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* CANDLE_B200_NCCL_H_ */
