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
 * ncclCommInitRank with a deadline.  The reference's set-up blocks for as long as a peer is missing
 * (its ranks poll for the id file forever, llama_multiprocess/main.rs:156-158, and
 * `Comm::from_rank` then waits inside NCCL); here the communicator is created in NCCL's
 * non-blocking mode and polled on the host: if the ranks have not all joined within `timeout_ms`
 * the half-built communicator is aborted, *comm_out stays NULL and CB200_E_TIMEOUT is returned --
 * the caller can report the missing peer and retry or leave.  No device work is involved.  A
 * communicator made this way stays non-blocking; the sharded entry points below wait (on the host,
 * with the same kind of deadline) until NCCL has accepted their collective.
 */
CB200_API int cb200_nccl_comm_init_timeout(void** comm_out, int nranks, const void* id, int rank, int timeout_ms);

/*
 * Vocabulary-sharded cb200_qembedding -> sum over ranks -> rms_norm, enqueued on `stream`:
 *   scratch = masked lookup of ALL ids in this rank's rows [vocab_begin, vocab_end) (zero bits elsewhere)
 *   scratch = ncclAllReduce(scratch, sum over the bit patterns taken as unsigned integers)
 *   y       = rms_norm(scratch, alpha, eps)
 * Each element has one non-zero contributor, so the integer sum returns that contributor's bits
 * whatever they encode.  A floating-point sum does not: NCCL's bf16 sum over 8 GPUs returned +0.0
 * where every rank held -0.0 and altered NaN payloads on large buffers, while its 2- and 4-GPU sums
 * (and the 8-GPU sum of a small buffer) kept them.
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

/*
 * The same operation for callers that must not allocate device memory and have no buffer to lend:
 * code that runs after the application's memory pool has claimed the whole device (a cudaMalloc
 * there fails, or fragments what the pool thinks it owns), and latency-critical serving loops,
 * where the device-wide synchronisation a cudaMalloc / cudaFree implies stalls every stream.
 * It has no counterpart in the reference.
 *
 * Instead of a `scratch` argument it uses a fixed array of CB200_STATIC_SCRATCH_BYTES that is part
 * of the library image (each GPU that loads the library holds it until the process exits), so
 * n_ids * hidden * sizeof(out_dtype) must not exceed that size; larger requests are refused with
 * CB200_E_UNSUPPORTED_SHAPE and a message, and should go to the entry point above.  Inputs and
 * outputs are still the caller's.  The call itself performs no cudaMalloc, cudaFree or other
 * allocating call; with a non-NULL `comm` it issues one ncclAllReduce on a communicator the caller
 * created earlier (pass NULL for a single rank: no NCCL call is made).
 *
 * The first call on a device looks the array's device address up (cudaGetSymbolAddress, with
 * that device current) and keeps it.  Under CUDA's default lazy module loading that lookup is also
 * what brings the library's device image, array included, onto the device: the 32 MiB are reserved
 * THEN, not when the host library is loaded.  So make the first call on each device early -- before
 * a memory pool claims the rest of the device (afterwards it can fail with an out-of-memory error),
 * and outside any stream capture -- or run the process with CUDA_MODULE_LOADING=EAGER.  Every later
 * call allocates nothing.  All calls share the one array, which keeps the previous call's rows:
 * nothing in it needs clearing, because for valid ids the lookup rewrites every byte the later steps
 * read (the row of y that belongs to an out-of-range id, which `status` records, is undefined), but
 * two calls whose work overlaps on the GPU (different streams, or threads) race on it -- serialise
 * them.
 */
#define CB200_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)

CB200_API int cb200_sharded_qembedding_rms_norm_static(void* comm, const void* qtable, int qtype, const void* ids,
                                                       const void* alpha, void* y, int64_t vocab, int32_t hidden,
                                                       int64_t n_ids, float eps, int out_dtype, int id_dtype,
                                                       int64_t vocab_begin, int64_t vocab_end, int flags,
                                                       cb200_status* status, cb200_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* CANDLE_B200_NCCL_H_ */
