/*
 * candle_b200 -- C ABI of the B200 (sm_100a) normalisation + embedding kernels.
 *
 * Each entry point replaces one device-side step of candle's CUDA backend for this path and is
 * what a Rust `extern "C"` block (in the style of candle-flash-attn/src/ffi.rs:3-51) binds.
 * Conventions, identical for every function:
 *   - all tensor pointers are DEVICE pointers to contiguous row-major data whose start offset
 *     has already been applied by the caller (candle-nn/src/ops.rs:536-543 does the same
 *     `slice(o1..o2)` before launching); strides are never passed;
 *   - the CALLER allocates every output (candle: `unsafe { dev.alloc::<T>(el) }`,
 *     candle-nn/src/ops.rs:557); the library allocates and frees nothing and writes every
 *     output element of a call that succeeds;
 *   - alignment: the norms and the dense gathers accept any pointer the element type allows and
 *     take slower kernels (same results) for tensors that are not 16-byte aligned; the quantised
 *     entry points require 16-byte aligned outputs (refused with CB200_E_INVALID_ARGUMENT
 *     otherwise) and write them fastest when they are 32-byte aligned, one 256-bit store per
 *     lane; buffers from cudarc's or any other device allocator satisfy all of this;
 *   - work is enqueued on `stream` and the call returns without synchronising;
 *   - the return value is 0 or a negative CB200_E_* code; cb200_last_error() returns a
 *     thread-local message for the last failing call of the calling thread;
 *   - problems only the device can see (an id outside the table, a bounded wait that ran out)
 *     are recorded in a caller-provided `cb200_status` record in device memory, which the caller
 *     zeroes before the call and reads after synchronising the stream; kernels never trap.
 *
 * Numerics: results equal those of candle's CPU backend on the same inputs -- bit-exact for the
 * gathers and the Q4_0/Q8_0 decoders, and for the norms bit-exact as well (NaN payloads aside)
 * unless CB200_FLAG_FAST_SUM is set, because the row sums are accumulated in candle's strictly
 * sequential f32 order (candle-nn/src/ops.rs:484-490, 709-715) and every rounding step of its
 * f32 / f16 / bf16 arithmetic is reproduced.
 */
#ifndef CANDLE_B200_H_
#define CANDLE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CB200_VERSION 100

#if defined(__GNUC__)
#define CB200_API __attribute__((visibility("default")))
#else
#define CB200_API
#endif

/* Element types of tensors (candle DType::F32 / F16 / BF16). */
#define CB200_DTYPE_F32 0
#define CB200_DTYPE_F16 1
#define CB200_DTYPE_BF16 2

/* Index types (candle DType::U8 / U32 / I64, the three IntDType ids index_select accepts,
 * candle-core/src/cuda_backend/mod.rs:366-372). */
#define CB200_ID_U8 0
#define CB200_ID_U32 1
#define CB200_ID_I64 2

/* Block formats: ggml type ids as in candle-core/src/quantized/mod.rs:152-171.  Q4_0 and Q8_0 are
 * accepted everywhere; Q4_1, Q5_0, Q5_1 and the K-quant super-blocks of 256 elements (Q2K .. Q8K,
 * candle-core/src/quantized/k_quants.rs:96-154) by cb200_dequantize, cb200_qembedding and
 * cb200_qembedding_rms_norm (one launch for the usual row lengths, two otherwise).  Q8_1 is refused:
 * candle has no decoder for it (k_quants.rs:693-695).  A row must be a whole number of blocks:
 * hidden % 32 == 0, hidden % 256 == 0 for the K-quants. */
#define CB200_QTYPE_Q4_0 2
#define CB200_QTYPE_Q4_1 3
#define CB200_QTYPE_Q5_0 6
#define CB200_QTYPE_Q5_1 7
#define CB200_QTYPE_Q8_0 8
#define CB200_QTYPE_Q2K 10
#define CB200_QTYPE_Q3K 11
#define CB200_QTYPE_Q4K 12
#define CB200_QTYPE_Q5K 13
#define CB200_QTYPE_Q6K 14
#define CB200_QTYPE_Q8K 15

/* flags */
#define CB200_FLAG_FAST_SUM 1 /* tree-order row sums: faster for some shapes, NOT bit-faithful */
/* Implementation selectors.  Results are identical whichever kernel runs; the tests use these
 * to cross-check the independent kernels against each other at sizes the CPU oracle is slow at. */
#define CB200_FLAG_FORCE_LANEROW 0x100 /* lane-per-row sequential kernel even where the register kernel applies */
#define CB200_FLAG_FORCE_GENERIC 0x200 /* any-shape scalar kernel */
#define CB200_FLAG_FORCE_REPLAY 0x400  /* register kernels: take the exact replay path for every row */

/* return codes */
#define CB200_OK 0
#define CB200_E_INVALID_ARGUMENT -1
#define CB200_E_UNSUPPORTED_DTYPE -2
#define CB200_E_CUDA -3
#define CB200_E_NCCL -4
#define CB200_E_UNSUPPORTED_SHAPE -5
#define CB200_E_TIMEOUT -6 /* a host-side wait with a deadline ran out (communicator setup) */

/* cb200_status.code */
#define CB200_STATUS_OK 0
#define CB200_STATUS_INVALID_INDEX 1 /* candle: Error::InvalidIndex{index,size,op:"index-select"} */
#define CB200_STATUS_WAIT_TIMEOUT 2  /* a bounded device-side wait gave up */

typedef struct cb200_status {
  int32_t code;     /* CB200_STATUS_*; only the first problem of a call is kept */
  int32_t reserved;
  int64_t position; /* which id (flattened position) was bad / which row timed out */
  int64_t index;    /* the offending id value */
  int64_t size;     /* the dimension size it was checked against */
} cb200_status;

typedef struct CUstream_st* cb200_stream_t; /* == cudaStream_t */

CB200_API int cb200_version(void);
CB200_API const char* cb200_last_error(void);

/*
 * RMS norm over the last dimension, optionally fused with the residual add that precedes it.
 *   h = residual ? T(x + residual) : x          (the rounded sum candle's `Tensor::add` yields,
 *                                                candle-core/src/op.rs:330)
 *   y = h / T(sqrt(mean(h^2) + eps)) * alpha     (candle-nn/src/ops.rs:484-495)
 * Replaces the CUDA launch in RmsNorm::cuda_fwd (candle-nn/src/ops.rs:510-580, kernel
 * `rmsnorm_{f32,f16,bf16}` of candle-kernels/src/reduce.cu:135-175) and, when `residual` is
 * given, also the `badd_*` launch before it (candle-kernels/src/binary.cu:5).
 * x, residual, y, sum_out: [rows, cols]; alpha: [cols]; residual and sum_out may be NULL;
 * sum_out, when given, receives h (what the model keeps as the next residual stream).
 * y may alias x or residual; sum_out may alias x or residual.
 */
CB200_API int cb200_rms_norm(const void* x, const void* residual, const void* alpha, void* y, void* sum_out,
                   int64_t rows, int32_t cols, float eps, int dtype, int flags, cb200_stream_t stream);

/*
 * Layer norm with affine weight and bias, optionally fused with the preceding residual add.
 *   y = T((h - mean) * (1/sqrt(var + eps)) * gamma + beta), all in f32 with one final rounding
 * (candle-nn/src/ops.rs:709-726).  Replaces LayerNorm::cuda_fwd (candle-nn/src/ops.rs:743-822,
 * kernel `layernorm_*` of candle-kernels/src/reduce.cu:72-131).
 */
CB200_API int cb200_layer_norm(const void* x, const void* residual, const void* gamma, const void* beta, void* y,
                     void* sum_out, int64_t rows, int32_t cols, float eps, int dtype, int flags,
                     cb200_stream_t stream);

/*
 * cb200_rms_norm / cb200_layer_norm with a status record.  Some of the norm kernels stage rows with
 * the bulk-copy engine and wait for them with a bounded wait; should such a wait ever run out the
 * rows concerned are left unwritten.  These variants record that as CB200_STATUS_WAIT_TIMEOUT in
 * `status` (NULL is allowed and makes them identical to the plain entry points, which have no way
 * to tell).  The reference has no counterpart: its kernels wait for nothing.
 */
CB200_API int cb200_rms_norm_checked(const void* x, const void* residual, const void* alpha, void* y, void* sum_out,
                           int64_t rows, int32_t cols, float eps, int dtype, int flags, cb200_status* status,
                           cb200_stream_t stream);
CB200_API int cb200_layer_norm_checked(const void* x, const void* residual, const void* gamma, const void* beta,
                             void* y, void* sum_out, int64_t rows, int32_t cols, float eps, int dtype, int flags,
                             cb200_status* status, cb200_stream_t stream);

/*
 * candle's composite ("slow") norm in one launch: what LayerNorm::forward computes whenever the
 * fused op does not apply -- no bias (LayerNorm::new_no_bias, layer_norm_no_bias), remove_mean ==
 * false (LayerNorm::rms_norm, RmsNorm::forward_diff / into_inner), or an input that had to be made
 * contiguous first (candle-nn/src/layer_norm.rs:108-136) -- and what ops::rms_norm_slow /
 * layer_norm_slow compute (candle-nn/src/ops.rs:628-639, 876-894):
 *   x = f32(x); if remove_mean: x -= sum(x) / n;  d = sqrt(sum(x*x) / n + eps);
 *   y = T(x / d) * weight (+ bias), the product and the sum evaluated in T
 * Replaces the chain of to_dtype / sum_keepdim / affine / broadcast_{sub,div,mul,add} / sqr / sqrt
 * launches (kernels of candle-kernels/src/{cast,reduce,affine,binary,unary}.cu).  Differs from
 * cb200_rms_norm / cb200_layer_norm in where it rounds, as candle's two paths do.  The row sums
 * follow the order of candle's CPU `vec_sum` in an AVX build (candle-core/src/cpu/mod.rs:113-135,
 * cpu/avx.rs:54-66), which makes the result bit-equal to that build; other builds of candle sum
 * in another order and agree to rounding error.  `bias` may be NULL.
 */
CB200_API int cb200_layer_norm_slow(const void* x, const void* weight, const void* bias, void* y, int64_t rows,
                          int32_t cols, float eps, int dtype, int remove_mean, cb200_stream_t stream);

/*
 * softmax over the last dimension: y[r, :] = exp(x[r, :] - max(x[r, :])) / sum(...), x and y
 * [rows, cols] contiguous, y not aliasing x.  Replaces SoftmaxLastDim::cuda_fwd
 * (candle-nn/src/ops.rs:335-386, kernel `softmax_*` of candle-kernels/src/reduce.cu:177-219) with the
 * arithmetic of its cpu_fwd (:296-333): everything in T, the row sum in candle's CPU order -- the
 * AVX-ordered vec_sum for f32, one T-rounded addition per element for f16 / bf16.  exp follows the
 * correctly rounded value where candle calls the platform's expf; the two agree except in the rare
 * cases where that libm does not round correctly.
 */
CB200_API int cb200_softmax_last_dim(const void* x, void* y, int64_t rows, int32_t cols, int dtype,
                                     cb200_stream_t stream);

/*
 * Rotary embeddings (candle-nn/src/rotary_emb.rs), all three fused forms, computed in T with every
 * product and the final sum / difference rounded separately as on the CPU (rotary_emb.rs:47-60,
 * 288-305, 540-558); replaces the kernels `rope_i_*`, `rope_*`, `rope_thd_*` of
 * candle-kernels/src/reduce.cu:221-278:
 *   CB200_ROPE_INTERLEAVED  rope_i    src [b, h, t, d], pairs (x[2k], x[2k+1])
 *   CB200_ROPE_HALF         rope      src [b, h, t, d], pairs (x[k], x[k + d/2])
 *   CB200_ROPE_THD          rope_thd  src [b, t, h, d], pairs (x[k], x[k + d/2])
 *   y1 = x1 * cos[t, k] - x2 * sin[t, k];  y2 = x1 * sin[t, k] + x2 * cos[t, k]
 * cos and sin are [>= t, d/2] contiguous, of the same dtype as src; dst has the shape of src and does
 * not alias it.
 */
#define CB200_ROPE_INTERLEAVED 0
#define CB200_ROPE_HALF 1
#define CB200_ROPE_THD 2
CB200_API int cb200_rope(const void* src, const void* cos, const void* sin, void* dst, int64_t b, int32_t h, int32_t t,
                         int32_t d, int dtype, int variant, cb200_stream_t stream);

/*
 * Self-test hook, not for production use: with `enable` != 0 every later launch of a kernel that
 * waits for bulk copies polls only a few dozen times and expects 16 bytes more than its copies
 * deliver, so every such wait runs out, the kernel records CB200_STATUS_WAIT_TIMEOUT, lets the
 * copies it issued land and returns -- the give-up path executes although nothing is wrong with the
 * device.  Results of calls made in this mode are undefined.  enable == 0 restores normal waiting.
 * Process-wide.  No counterpart in the reference.
 */
CB200_API int cb200_selftest_wait_expiry(int enable);

/*
 * index_select along one dimension of a contiguous tensor viewed as [left, src_dim, right]:
 *   out[l, i, :] = src[l, ids[i], :]   for i < n_ids
 * Replaces IndexSelect::f + BackendStorage::index_select of the CUDA backend
 * (candle-core/src/cuda_backend/mod.rs:352-410, 1622-1626; kernel `is_{u8,u32,i64}_{T}` of
 * candle-kernels/src/indexing.cu:6-44).  `elem_size` is the element size in bytes (any dtype).
 * Unlike the reference kernel every id is bounds-checked; a bad id is reported through `status`
 * (as the CPU backend does, candle-core/src/cpu_backend/mod.rs:539-546) and its output slice is
 * left unwritten.
 */
CB200_API int cb200_index_select(const void* src, const void* ids, void* out, int64_t left, int64_t src_dim,
                       int64_t right, int64_t n_ids, int32_t elem_size, int id_dtype, cb200_status* status,
                       cb200_stream_t stream);

/*
 * Embedding::forward (candle-nn/src/embedding.rs:29-36): out[i, :] = table[ids[i], :], table
 * [vocab, hidden].  Equivalent to cb200_index_select with left = 1.
 */
CB200_API int cb200_embedding(const void* table, const void* ids, void* out, int64_t vocab, int32_t hidden,
                    int64_t n_ids, int dtype, int id_dtype, cb200_status* status, cb200_stream_t stream);

/*
 * Whole-buffer block decode: k elements (a whole number of blocks) of any supported format -> out_dtype.
 * Replaces QCudaStorage::dequantize / dequantize_f16 (candle-core/src/quantized/cuda.rs:69-124,
 * 391-414; kernels `dequantize_block_q{4,8}_0_{f32,f16}` of candle-kernels/src/quantized.cu:
 * 779-805, 1068-1091) and, for bf16 / f16 output, the cast kernel that follows it
 * (candle-kernels/src/cast.cu:4-25).  Values equal GgmlType::to_float on the CPU
 * (candle-core/src/quantized/k_quants.rs:163-183, 568-584; K-quants :834-871, 1095-1149, 1313-1342,
 * 1528-1563, 1716-1746, 1827-1839; CUDA twins candle-kernels/src/quantized.cu:807-1066) including
 * the sign of zero and, for the formats whose decode rounds more than once, the operation order.
 */
CB200_API int cb200_dequantize(const void* blocks, int qtype, void* out, int64_t k, int out_dtype,
                     cb200_stream_t stream);

/*
 * Row lookup straight out of a block-quantised [vocab, hidden] table (hidden a whole number of blocks):
 *   out[i, :] = T(to_float(qtable[ids[i], :]))
 * i.e. what QTensor::dequantize + to_dtype + Embedding::forward compute
 * (candle-transformers/src/models/quantized_llama.rs:378-379, candle-nn/src/embedding.rs:29-36)
 * without materialising the decoded table.  The reference has no such device entry point.
 * Vocab sharding: `qtable` holds rows [vocab_begin, vocab_end) of the full table; ids inside that
 * range are decoded, ids outside it (but < vocab) produce rows of zero BITS, so that adding the
 * shards' partial rows as unsigned integers (one non-zero contributor per element) assembles the
 * unsharded result bit for bit, -0.0, subnormals and NaN payloads included; pass 0 and `vocab` for
 * an unsharded table.  ids >= vocab are reported through `status`.
 */
CB200_API int cb200_qembedding(const void* qtable, int qtype, const void* ids, void* out, int64_t vocab,
                     int32_t hidden, int64_t n_ids, int out_dtype, int id_dtype, int64_t vocab_begin,
                     int64_t vocab_end, cb200_status* status, cb200_stream_t stream);

/*
 * Fused Embedding::forward -> rms_norm: y[i, :] = rms_norm(table[ids[i], :], alpha, eps); when
 * `gathered` is not NULL it also receives the gathered rows (the residual stream).  Replaces an
 * `is_*` launch followed by a `rmsnorm_*` launch (candle-transformers/src/models/llama.rs:507
 * followed by :446).
 */
CB200_API int cb200_embedding_rms_norm(const void* table, const void* ids, const void* alpha, void* y, void* gathered,
                             int64_t vocab, int32_t hidden, int64_t n_ids, float eps, int dtype,
                             int id_dtype, int flags, cb200_status* status, cb200_stream_t stream);

/* Fused cb200_qembedding -> rms_norm in `out_dtype` (same sharding arguments). */
CB200_API int cb200_qembedding_rms_norm(const void* qtable, int qtype, const void* ids, const void* alpha, void* y,
                              void* gathered, int64_t vocab, int32_t hidden, int64_t n_ids, float eps,
                              int out_dtype, int id_dtype, int64_t vocab_begin, int64_t vocab_end,
                              int flags, cb200_status* status, cb200_stream_t stream);

/*
 * The exchange step of a vocabulary-sharded table fused into the lookup: the rank that owns a row
 * produces it and stores it in every rank's output buffer.  `dsts[0 .. n_dsts)` (a HOST array of
 * 1..8 device pointers) are buffers of the same shape [n_ids, hidden]: this rank's own and the
 * peers' buffers mapped into this process (CUDA IPC / virtual-memory mapping over NVLink).  The
 * call decodes and RMS-normalises only the ids inside [vocab_begin, vocab_end) and writes each
 * finished row to all destinations with plain stores; rows owned by other ranks are not touched.
 * When every rank has made the call and the ranks have synchronised (the caller's barrier, after
 * which the stores are visible), each buffer holds all rows, bit-identical to the unsharded
 * lookup + norm.  Per GPU this moves (N-1)/N of the output over NVLink once and does 1/N of the
 * decode and norm work, where the masked lookup + all-reduce of candle's tensor-parallel example
 * (candle-examples/examples/llama_multiprocess/model.rs:31-90) moves twice that and normalises
 * every row on every rank.  A buffer may be reused only after its readers are done on every rank.
 * Needs the single-launch kernel: f16 / bf16 output and a hidden size it has a split for.
 */
CB200_API int cb200_qembedding_rms_norm_owner(const void* qtable, int qtype, const void* ids, const void* alpha,
                                    void* const* dsts, int n_dsts, int64_t vocab, int32_t hidden,
                                    int64_t n_ids, float eps, int out_dtype, int id_dtype,
                                    int64_t vocab_begin, int64_t vocab_end, int flags, cb200_status* status,
                                    cb200_stream_t stream);

/*
 * The same exchange for callers that continue ROW-SHARDED after the lookup (each rank works on its
 * own block of token rows): a finished row is stored into ONE buffer only, that of the rank whose
 * block contains it.  `dsts[r]` (HOST array, in rank order, 1..8 entries) is rank r's buffer -- this
 * rank's own memory for its own entry, peers' buffers mapped into this process for the others -- of
 * shape [row_bounds[r + 1] - row_bounds[r], hidden]; `row_bounds` (HOST array of n_dsts + 1 entries,
 * from 0 to n_ids, non-decreasing) gives the blocks, e.g. contiguous blocks whose sizes differ by at
 * most one.  Per GPU only about (N-1)/N^2 of the output crosses NVLink, against (N-1)/N for
 * cb200_qembedding_rms_norm_owner and 2(N-1)/N for candle's all-reduce
 * (candle-examples/examples/llama_multiprocess/model.rs:31-90); after the ranks' barrier each buffer
 * holds exactly its block, bit-identical to those rows of the unsharded lookup + norm.
 */
CB200_API int cb200_qembedding_rms_norm_row_owner(const void* qtable, int qtype, const void* ids, const void* alpha,
                                        void* const* dsts, int n_dsts, const int64_t* row_bounds, int64_t vocab,
                                        int32_t hidden, int64_t n_ids, float eps, int out_dtype, int id_dtype,
                                        int64_t vocab_begin, int64_t vocab_end, int flags, cb200_status* status,
                                        cb200_stream_t stream);

/*
 * The cheapest exchange for a vocabulary-sharded table with row-sharded consumers: route the RAW block
 * rows.  For every id inside [vocab_begin, vocab_end) this rank copies the quantised row -- hidden / 32
 * blocks, e.g. 4608 bytes of Q4_0 where the decoded bf16 row has 16384 -- into `dsts[r]`, the staging
 * buffer of the rank r whose block of token rows [row_bounds[r], row_bounds[r + 1]) contains the id's
 * position i, at row i - row_bounds[r] (HOST arrays in rank order as for
 * cb200_qembedding_rms_norm_row_owner; the peers' staging buffers are mapped into this process).  After
 * the ranks' barrier each staging buffer is a dense [rows_r, hidden] table of blocks in token order,
 * and the rank decodes and normalises it locally with cb200_qembedding_rms_norm (ids 0 .. rows_r - 1):
 * bit-identical to the unsharded lookup + norm, with about (N-1)/N^2 of the QUANTISED bytes crossing
 * NVLink per GPU.  Ids of other ranks are skipped; ids >= vocab are reported through `status`.  The
 * reference has no counterpart (its tensor-parallel example replicates the embedding,
 * candle-examples/examples/llama_multiprocess/model.rs:181-184).
 */
CB200_API int cb200_qembedding_route_rows(const void* qtable, int qtype, const void* ids, void* const* dsts, int n_dsts,
                                const int64_t* row_bounds, int64_t vocab, int32_t hidden, int64_t n_ids, int id_dtype,
                                int64_t vocab_begin, int64_t vocab_end, cb200_status* status, cb200_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* CANDLE_B200_H_ */
