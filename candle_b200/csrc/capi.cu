// The extern "C" surface declared in include/candle_b200.h: argument validation, error strings
// and dispatch to the kernel launchers.  No allocation, no synchronisation, no global state
// beyond a thread-local error message.
#include <cstdarg>
#include <cstdio>

#include <nvtx3/nvToolsExt.h>

#include "launch.h"
#include "qblocks.cuh"
#include "rms_rowreg.cuh"

namespace {

// An NVTX range around every entry point that enqueues work, named after it: what candle's
// `tracing` spans around `forward` show in a Chrome trace, these show on a profiler's timeline.
// Without a profiler attached a range is two calls through a null function table.
struct TraceRange {
  explicit TraceRange(const char* name) { nvtxRangePushA(name); }
  ~TraceRange() { nvtxRangePop(); }
  TraceRange(const TraceRange&) = delete;
  TraceRange& operator=(const TraceRange&) = delete;
};

thread_local char g_last_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_result(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return CB200_OK;
  return fail(CB200_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

bool valid_dtype(int d) { return d == CB200_DTYPE_F32 || d == CB200_DTYPE_F16 || d == CB200_DTYPE_BF16; }
bool valid_id_dtype(int d) { return d == CB200_ID_U8 || d == CB200_ID_U32 || d == CB200_ID_I64; }
bool valid_qtype(int q) { return cb200::qblock_bytes(q) != 0; }
// the formats the single-launch lookup + norm kernel decodes
bool fusable_qtype(int q) { return q == CB200_QTYPE_Q4_0 || q == CB200_QTYPE_Q8_0; }
int elem_bytes(int d) { return d == CB200_DTYPE_F32 ? 4 : 2; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename... P>
bool all_aligned16(P... ptrs) {
  return (aligned16(ptrs) && ...);
}

int norm_impl(int op, const void* x, const void* residual, const void* alpha, const void* beta, void* y,
              void* sum_out, int64_t rows, int32_t cols, float eps, int dtype, int flags, cb200_status* status,
              cudaStream_t stream) {
  const char* name = op == cb200::kOpLayerNorm ? "cb200_layer_norm" : "cb200_rms_norm";
  if (!valid_dtype(dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported dtype code %d", name, dtype);
  if (rows < 0 || cols < 0) return fail(CB200_E_INVALID_ARGUMENT, "%s: negative shape [%lld, %d]", name, (long long)rows, cols);
  if (rows == 0) return CB200_OK;
  if (cols == 0) return fail(CB200_E_INVALID_ARGUMENT, "%s: rows of zero columns cannot be normalised", name);
  if (x == nullptr || alpha == nullptr || y == nullptr || (op == cb200::kOpLayerNorm && beta == nullptr))
    return fail(CB200_E_INVALID_ARGUMENT, "%s: null tensor pointer", name);
  if (rows > (int64_t(1) << 40)) return fail(CB200_E_INVALID_ARGUMENT, "%s: too many rows", name);

  const bool vec_ok = all_aligned16(x, residual, alpha, beta, y, sum_out) &&
                      (static_cast<int64_t>(cols) * elem_bytes(dtype)) % 16 == 0;
  const bool force_lane = flags & CB200_FLAG_FORCE_LANEROW;
  const bool force_generic = flags & CB200_FLAG_FORCE_GENERIC;

  if (op == cb200::kOpRmsNorm && vec_ok && !force_lane && !force_generic && residual == nullptr &&
      dtype != CB200_DTYPE_F32 && cols <= 4096 && rows >= 32768 && cb200::qrms_rowreg_supported(dtype, cols)) {
    // no residual: a row brings too few bytes for the register kernel to cover the memory latency;
    // the row-slot kernel stages rows with bulk copies several rows ahead.  Measured better for
    // many rows of up to 4096 columns (0.69 -> 0.76 of the HBM peak), worse at 8192 columns and
    // for few rows.
    cb200::QRmsArgs a{};
    a.qtable = static_cast<const unsigned char*>(x);
    a.alpha = static_cast<const uint4*>(alpha);
    a.y = static_cast<uint4*>(y);
    a.gathered = static_cast<uint4*>(sum_out);
    a.vocab = rows;
    a.vocab_end = rows;
    a.status = status;
    a.rows = rows;
    a.V = cols / 8;
    a.n = cols;
    a.row_bytes = cols * 2;
    a.bulk = 1;
    a.eps = eps;
    a.flags = flags;
    return cuda_result(cb200::launch_qrms_rowreg(cb200::kQTypeDense16, dtype, a, stream), name);
  }
  if (op == cb200::kOpRmsNorm && vec_ok && !force_lane && !force_generic && cb200::rms_rowreg_supported(dtype, cols)) {
    cb200::RmsRowRegArgs a{};
    a.x = static_cast<const uint4*>(x);
    a.res = static_cast<const uint4*>(residual);
    a.alpha = static_cast<const uint4*>(alpha);
    a.y = static_cast<uint4*>(y);
    a.sum_out = static_cast<uint4*>(sum_out);
    a.status = status;
    a.rows = rows;
    a.V = cols / 8;
    a.n = cols;
    a.eps = eps;
    a.flags = flags;
    return cuda_result(cb200::launch_rms_rowreg(dtype, a, stream), name);
  }
  cb200::LaneRowArgs a{};
  a.x = x;
  a.status = status;
  a.res = residual;
  a.alpha = alpha;
  a.beta = beta;
  a.y = y;
  a.sum_out = sum_out;
  a.rows = rows;
  a.n = cols;
  a.eps = eps;
  a.classic = force_lane ? 1 : 0;
  if (vec_ok && !force_generic && cb200::norm_lanerow_supported(dtype, cols))
    return cuda_result(cb200::launch_norm_lanerow(dtype, op, a, stream), name);
  return cuda_result(cb200::launch_norm_generic(dtype, op, a, stream), name);
}

int check_lookup(const char* name, const void* table, const void* ids, const void* out, int64_t vocab,
                 int64_t hidden, int64_t n_ids, int id_dtype) {
  if (!valid_id_dtype(id_dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported ids dtype code %d", name, id_dtype);
  if (vocab < 0 || hidden < 0 || n_ids < 0) return fail(CB200_E_INVALID_ARGUMENT, "%s: negative shape", name);
  if (n_ids > 0 && hidden > 0 && (table == nullptr || ids == nullptr || out == nullptr))
    return fail(CB200_E_INVALID_ARGUMENT, "%s: null tensor pointer", name);
  return CB200_OK;
}

}  // namespace

extern "C" {

int cb200_version(void) { return CB200_VERSION; }

const char* cb200_last_error(void) { return g_last_error; }

int cb200_rms_norm(const void* x, const void* residual, const void* alpha, void* y, void* sum_out, int64_t rows,
                   int32_t cols, float eps, int dtype, int flags, cb200_stream_t stream) {
  const TraceRange trace("cb200_rms_norm");
  return norm_impl(cb200::kOpRmsNorm, x, residual, alpha, nullptr, y, sum_out, rows, cols, eps, dtype, flags, nullptr,
                   stream);
}

int cb200_rms_norm_checked(const void* x, const void* residual, const void* alpha, void* y, void* sum_out,
                           int64_t rows, int32_t cols, float eps, int dtype, int flags, cb200_status* status,
                           cb200_stream_t stream) {
  const TraceRange trace("cb200_rms_norm_checked");
  return norm_impl(cb200::kOpRmsNorm, x, residual, alpha, nullptr, y, sum_out, rows, cols, eps, dtype, flags, status,
                   stream);
}

int cb200_layer_norm(const void* x, const void* residual, const void* gamma, const void* beta, void* y,
                     void* sum_out, int64_t rows, int32_t cols, float eps, int dtype, int flags,
                     cb200_stream_t stream) {
  const TraceRange trace("cb200_layer_norm");
  return norm_impl(cb200::kOpLayerNorm, x, residual, gamma, beta, y, sum_out, rows, cols, eps, dtype, flags, nullptr,
                   stream);
}

int cb200_layer_norm_checked(const void* x, const void* residual, const void* gamma, const void* beta, void* y,
                             void* sum_out, int64_t rows, int32_t cols, float eps, int dtype, int flags,
                             cb200_status* status, cb200_stream_t stream) {
  const TraceRange trace("cb200_layer_norm_checked");
  return norm_impl(cb200::kOpLayerNorm, x, residual, gamma, beta, y, sum_out, rows, cols, eps, dtype, flags, status,
                   stream);
}

int cb200_layer_norm_slow(const void* x, const void* weight, const void* bias, void* y, int64_t rows, int32_t cols,
                          float eps, int dtype, int remove_mean, cb200_stream_t stream) {
  const TraceRange trace("cb200_layer_norm_slow");
  const char* name = "cb200_layer_norm_slow";
  if (!valid_dtype(dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported dtype code %d", name, dtype);
  if (rows < 0 || cols < 0) return fail(CB200_E_INVALID_ARGUMENT, "%s: negative shape [%lld, %d]", name, (long long)rows, cols);
  if (rows == 0) return CB200_OK;
  if (cols == 0) return fail(CB200_E_INVALID_ARGUMENT, "%s: rows of zero columns cannot be normalised", name);
  if (x == nullptr || weight == nullptr || y == nullptr) return fail(CB200_E_INVALID_ARGUMENT, "%s: null tensor pointer", name);
  if (rows > (int64_t(1) << 40)) return fail(CB200_E_INVALID_ARGUMENT, "%s: too many rows", name);
  return cuda_result(cb200::launch_norm_slow(dtype, x, weight, bias, y, rows, cols, eps, remove_mean != 0, stream), name);
}

int cb200_softmax_last_dim(const void* x, void* y, int64_t rows, int32_t cols, int dtype, cb200_stream_t stream) {
  const TraceRange trace("cb200_softmax_last_dim");
  const char* name = "cb200_softmax_last_dim";
  if (!valid_dtype(dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported dtype code %d", name, dtype);
  if (rows < 0 || cols < 0) return fail(CB200_E_INVALID_ARGUMENT, "%s: negative shape [%lld, %d]", name, (long long)rows, cols);
  if (rows == 0 || cols == 0) return CB200_OK;
  if (x == nullptr || y == nullptr) return fail(CB200_E_INVALID_ARGUMENT, "%s: null tensor pointer", name);
  if (x == y) return fail(CB200_E_INVALID_ARGUMENT, "%s: the output must not alias the input", name);
  return cuda_result(cb200::launch_softmax_last_dim(dtype, x, y, rows, cols, stream), name);
}

int cb200_rope(const void* src, const void* cos, const void* sin, void* dst, int64_t b, int32_t h, int32_t t, int32_t d,
               int dtype, int variant, cb200_stream_t stream) {
  const TraceRange trace("cb200_rope");
  const char* name = "cb200_rope";
  if (!valid_dtype(dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported dtype code %d", name, dtype);
  if (variant < CB200_ROPE_INTERLEAVED || variant > CB200_ROPE_THD)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: unknown variant %d", name, variant);
  if (b < 0 || h < 0 || t < 0 || d < 0) return fail(CB200_E_INVALID_ARGUMENT, "%s: negative shape", name);
  if (d % 2 != 0) return fail(CB200_E_INVALID_ARGUMENT, "%s: the last dimension (%d) must be even", name, d);
  if (b == 0 || h == 0 || t == 0 || d == 0) return CB200_OK;
  if (src == nullptr || cos == nullptr || sin == nullptr || dst == nullptr)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: null tensor pointer", name);
  if (src == dst) return fail(CB200_E_INVALID_ARGUMENT, "%s: the output must not alias the input", name);
  return cuda_result(cb200::launch_rope(variant, dtype, src, cos, sin, dst, b, h, t, d, stream), name);
}

int cb200_selftest_wait_expiry(int enable) {
  // 64 polls and 16 bytes that never arrive: every bounded wait of the bulk-copy kernels runs out
  cb200::set_wait_tuning(enable ? cb200::WaitTuning{64u, 16u} : cb200::WaitTuning{cb200::kWaitSpins, 0u});
  return CB200_OK;
}

int cb200_index_select(const void* src, const void* ids, void* out, int64_t left, int64_t src_dim, int64_t right,
                       int64_t n_ids, int32_t elem_size, int id_dtype, cb200_status* status,
                       cb200_stream_t stream) {
  const TraceRange trace("cb200_index_select");
  const char* name = "cb200_index_select";
  if (!valid_id_dtype(id_dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported ids dtype code %d", name, id_dtype);
  if (left < 0 || src_dim < 0 || right < 0 || n_ids < 0 || elem_size <= 0)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: bad shape", name);
  if (left == 0 || right == 0 || n_ids == 0) return CB200_OK;
  if (src == nullptr || ids == nullptr || out == nullptr) return fail(CB200_E_INVALID_ARGUMENT, "%s: null tensor pointer", name);
  cb200::GatherArgs a{};
  a.src = static_cast<const unsigned char*>(src);
  a.ids = ids;
  a.out = static_cast<unsigned char*>(out);
  a.left = left;
  a.src_dim = src_dim;
  a.n_ids = n_ids;
  a.row_bytes = right * elem_size;
  a.id_dtype = id_dtype;
  a.status = status;
  return cuda_result(cb200::launch_gather_rows(a, stream), name);
}

int cb200_embedding(const void* table, const void* ids, void* out, int64_t vocab, int32_t hidden, int64_t n_ids,
                    int dtype, int id_dtype, cb200_status* status, cb200_stream_t stream) {
  const TraceRange trace("cb200_embedding");
  if (!valid_dtype(dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "cb200_embedding: unsupported dtype code %d", dtype);
  int rc = check_lookup("cb200_embedding", table, ids, out, vocab, hidden, n_ids, id_dtype);
  if (rc != CB200_OK) return rc;
  return cb200_index_select(table, ids, out, 1, vocab, hidden, n_ids, elem_bytes(dtype), id_dtype, status, stream);
}

int cb200_dequantize(const void* blocks, int qtype, void* out, int64_t k, int out_dtype, cb200_stream_t stream) {
  const TraceRange trace("cb200_dequantize");
  const char* name = "cb200_dequantize";
  if (!valid_qtype(qtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported block format %d", name, qtype);
  if (!valid_dtype(out_dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported dtype code %d", name, out_dtype);
  const int be = cb200::qblock_elems(qtype);
  if (k < 0 || k % be != 0)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: %lld is not divisible by %d", name, (long long)k, be);
  if (k == 0) return CB200_OK;
  if (blocks == nullptr || out == nullptr) return fail(CB200_E_INVALID_ARGUMENT, "%s: null tensor pointer", name);
  if (!aligned16(out) || (reinterpret_cast<uintptr_t>(blocks) & 1u))
    return fail(CB200_E_INVALID_ARGUMENT, "%s: output must be 16-byte aligned and blocks 2-byte aligned", name);
  return cuda_result(cb200::launch_dequantize_flat(qtype, out_dtype, blocks, out, k / 8, stream), name);
}

int cb200_qembedding(const void* qtable, int qtype, const void* ids, void* out, int64_t vocab, int32_t hidden,
                     int64_t n_ids, int out_dtype, int id_dtype, int64_t vocab_begin, int64_t vocab_end,
                     cb200_status* status, cb200_stream_t stream) {
  const TraceRange trace("cb200_qembedding");
  const char* name = "cb200_qembedding";
  if (!valid_qtype(qtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported block format %d", name, qtype);
  if (!valid_dtype(out_dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported dtype code %d", name, out_dtype);
  int rc = check_lookup(name, qtable, ids, out, vocab, hidden, n_ids, id_dtype);
  if (rc != CB200_OK) return rc;
  if (hidden % cb200::qblock_elems(qtype) != 0)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: hidden size %d is not divisible by %d", name, hidden,
                cb200::qblock_elems(qtype));
  if (vocab_begin < 0 || vocab_end < vocab_begin || vocab_end > vocab)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: bad vocab shard [%lld, %lld) of %lld", name, (long long)vocab_begin,
                (long long)vocab_end, (long long)vocab);
  if (n_ids == 0 || hidden == 0) return CB200_OK;
  if (!aligned16(out) || (reinterpret_cast<uintptr_t>(qtable) & 1u))
    return fail(CB200_E_INVALID_ARGUMENT, "%s: output must be 16-byte aligned and the table 2-byte aligned", name);
  cb200::QGatherArgs a{};
  a.qtable = static_cast<const unsigned char*>(qtable);
  a.ids = ids;
  a.out = out;
  a.id_dtype = id_dtype;
  a.vocab = vocab;
  a.vocab_begin = vocab_begin;
  a.vocab_end = vocab_end;
  a.status = status;
  a.rows = n_ids;
  a.n = hidden;
  a.row_bytes = hidden / cb200::qblock_elems(qtype) * cb200::qblock_bytes(qtype);
  a.bulk = aligned16(qtable) && a.row_bytes % 16 == 0;
  if (2 * ((a.row_bytes + 15) & ~15) + 64 > 227 * 1024)
    return fail(CB200_E_UNSUPPORTED_SHAPE, "%s: hidden size %d exceeds the staged-row limit", name, hidden);
  return cuda_result(cb200::launch_qgather(qtype, out_dtype, a, stream), name);
}

int cb200_embedding_rms_norm(const void* table, const void* ids, const void* alpha, void* y, void* gathered,
                             int64_t vocab, int32_t hidden, int64_t n_ids, float eps, int dtype, int id_dtype,
                             int flags, cb200_status* status, cb200_stream_t stream) {
  const TraceRange trace("cb200_embedding_rms_norm");
  const char* name = "cb200_embedding_rms_norm";
  if (!valid_dtype(dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported dtype code %d", name, dtype);
  int rc = check_lookup(name, table, ids, y, vocab, hidden, n_ids, id_dtype);
  if (rc != CB200_OK) return rc;
  if (n_ids == 0) return CB200_OK;
  if (hidden == 0) return fail(CB200_E_INVALID_ARGUMENT, "%s: rows of zero columns cannot be normalised", name);
  if (alpha == nullptr) return fail(CB200_E_INVALID_ARGUMENT, "%s: null tensor pointer", name);
  const bool vec_ok = all_aligned16(table, alpha, y, gathered) && (static_cast<int64_t>(hidden) * elem_bytes(dtype)) % 16 == 0;
  const bool force_lane = flags & CB200_FLAG_FORCE_LANEROW;
  const bool force_generic = flags & CB200_FLAG_FORCE_GENERIC;
  if (vec_ok && !force_lane && !force_generic && dtype != CB200_DTYPE_F32 &&
      cb200::qrms_rowreg_supported(dtype, hidden)) {
    // 16-bit tables whose rows split over the row-slot kernel: rows staged by bulk copies, several
    // rows ahead, instead of loaded into registers one row ahead (measured 0.59 -> 0.79 of the HBM
    // peak at 4096 columns, 0.69 -> 0.73 at 8192)
    cb200::QRmsArgs a{};
    a.qtable = static_cast<const unsigned char*>(table);
    a.ids = ids;
    a.alpha = static_cast<const uint4*>(alpha);
    a.y = static_cast<uint4*>(y);
    a.gathered = static_cast<uint4*>(gathered);
    a.id_dtype = id_dtype;
    a.vocab = vocab;
    a.vocab_begin = 0;
    a.vocab_end = vocab;
    a.status = status;
    a.rows = n_ids;
    a.V = hidden / 8;
    a.n = hidden;
    a.row_bytes = hidden * 2;
    a.bulk = 1;
    a.eps = eps;
    a.flags = flags;
    return cuda_result(cb200::launch_qrms_rowreg(cb200::kQTypeDense16, dtype, a, stream), name);
  }
  if (vec_ok && !force_lane && !force_generic && cb200::rms_rowreg_supported(dtype, hidden)) {
    cb200::RmsRowRegArgs a{};
    a.x = static_cast<const uint4*>(table);
    a.alpha = static_cast<const uint4*>(alpha);
    a.y = static_cast<uint4*>(y);
    a.sum_out = static_cast<uint4*>(gathered);
    a.ids = ids;
    a.id_dtype = id_dtype;
    a.vocab = vocab;
    a.status = status;
    a.rows = n_ids;
    a.V = hidden / 8;
    a.n = hidden;
    a.eps = eps;
    a.flags = flags;
    return cuda_result(cb200::launch_rms_rowreg(dtype, a, stream), name);
  }
  cb200::LaneRowArgs a{};
  a.x = table;
  a.alpha = alpha;
  a.y = y;
  a.sum_out = gathered;
  a.ids = ids;
  a.id_dtype = id_dtype;
  a.vocab = vocab;
  a.status = status;
  a.rows = n_ids;
  a.n = hidden;
  a.eps = eps;
  a.bulk = 1;
  a.classic = force_lane ? 1 : 0;
  if (vec_ok && !force_generic && cb200::norm_lanerow_supported(dtype, hidden))
    return cuda_result(cb200::launch_norm_lanerow(dtype, cb200::kOpRmsNorm, a, stream), name);
  return cuda_result(cb200::launch_norm_generic(dtype, cb200::kOpRmsNorm, a, stream), name);
}

int cb200_qembedding_rms_norm(const void* qtable, int qtype, const void* ids, const void* alpha, void* y,
                              void* gathered, int64_t vocab, int32_t hidden, int64_t n_ids, float eps, int out_dtype,
                              int id_dtype, int64_t vocab_begin, int64_t vocab_end, int flags, cb200_status* status,
                              cb200_stream_t stream) {
  const TraceRange trace("cb200_qembedding_rms_norm");
  const char* name = "cb200_qembedding_rms_norm";
  if (!valid_qtype(qtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported block format %d", name, qtype);
  if (!valid_dtype(out_dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported dtype code %d", name, out_dtype);
  int rc = check_lookup(name, qtable, ids, y, vocab, hidden, n_ids, id_dtype);
  if (rc != CB200_OK) return rc;
  if (hidden % cb200::qblock_elems(qtype) != 0)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: hidden size %d is not divisible by %d", name, hidden,
                cb200::qblock_elems(qtype));
  if (vocab_begin < 0 || vocab_end < vocab_begin || vocab_end > vocab)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: bad vocab shard [%lld, %lld) of %lld", name, (long long)vocab_begin,
                (long long)vocab_end, (long long)vocab);
  if (n_ids == 0) return CB200_OK;
  if (hidden == 0) return fail(CB200_E_INVALID_ARGUMENT, "%s: rows of zero columns cannot be normalised", name);
  if (alpha == nullptr) return fail(CB200_E_INVALID_ARGUMENT, "%s: null tensor pointer", name);
  if (!all_aligned16(alpha, y, gathered) || (reinterpret_cast<uintptr_t>(qtable) & 1u))
    return fail(CB200_E_INVALID_ARGUMENT, "%s: alpha, y and gathered must be 16-byte aligned, the table 2-byte aligned", name);
  // the single-launch kernel stages rows with bulk copies, which need a 16-byte aligned table
  const bool fused = fusable_qtype(qtype) && out_dtype != CB200_DTYPE_F32 && aligned16(qtable) &&
                     cb200::qrms_rowreg_supported(out_dtype, hidden) &&
                     !(flags & (CB200_FLAG_FORCE_LANEROW | CB200_FLAG_FORCE_GENERIC));
  const bool forced = (flags & (CB200_FLAG_FORCE_LANEROW | CB200_FLAG_FORCE_GENERIC)) != 0;
  if (!fused && !forced && aligned16(qtable) && cb200::kqrms_supported(qtype, out_dtype, hidden)) {
    // K-quant super-blocks and Q4_1 / Q5_0 / Q5_1: the row-register kernel with a decoder in front, one launch
    cb200::QRmsArgs a{};
    a.qtable = static_cast<const unsigned char*>(qtable);
    a.ids = ids;
    a.alpha = static_cast<const uint4*>(alpha);
    a.y = static_cast<uint4*>(y);
    a.gathered = static_cast<uint4*>(gathered);
    a.id_dtype = id_dtype;
    a.vocab = vocab;
    a.vocab_begin = vocab_begin;
    a.vocab_end = vocab_end;
    a.status = status;
    a.rows = n_ids;
    a.V = hidden / 8;
    a.n = hidden;
    a.row_bytes = hidden / cb200::qblock_elems(qtype) * cb200::qblock_bytes(qtype);
    a.bulk = 1;
    a.eps = eps;
    a.flags = flags;
    return cuda_result(cb200::launch_kqrms(qtype, out_dtype, a, stream), name);
  }
  if (!fused) {
    // Two launches (f32 output, a row length the fused kernel has no exact split for, or a forced
    // implementation): decode into `gathered`, or into y itself, then normalise (in place if y).
    // (Running the pair over chunks of rows small enough to stay in L2 between the two launches was
    // measured slower -- 615 us against 456 us for 65536 rows of 4096 columns from a Q4K table: the
    // launches' ramps and tails cost more than the second trip through HBM.)
    void* mid = gathered != nullptr ? gathered : y;
    rc = cb200_qembedding(qtable, qtype, ids, mid, vocab, hidden, n_ids, out_dtype, id_dtype, vocab_begin,
                          vocab_end, status, stream);
    if (rc != CB200_OK) return rc;
    return cb200_rms_norm(mid, nullptr, alpha, y, nullptr, n_ids, hidden, eps, out_dtype, flags, stream);
  }
  cb200::QRmsArgs a{};
  a.qtable = static_cast<const unsigned char*>(qtable);
  a.ids = ids;
  a.alpha = static_cast<const uint4*>(alpha);
  a.y = static_cast<uint4*>(y);
  a.gathered = static_cast<uint4*>(gathered);
  a.id_dtype = id_dtype;
  a.vocab = vocab;
  a.vocab_begin = vocab_begin;
  a.vocab_end = vocab_end;
  a.status = status;
  a.rows = n_ids;
  a.V = hidden / 8;
  a.n = hidden;
  a.row_bytes = hidden / cb200::qblock_elems(qtype) * cb200::qblock_bytes(qtype);
  a.bulk = aligned16(qtable) && a.row_bytes % 16 == 0;
  a.eps = eps;
  a.flags = flags;
  return cuda_result(cb200::launch_qrms_rowreg(qtype, out_dtype, a, stream), name);
}

static int owner_impl(const char* name, const void* qtable, int qtype, const void* ids, const void* alpha,
                      void* const* dsts, int n_dsts, const int64_t* row_bounds, int64_t vocab, int32_t hidden,
                      int64_t n_ids, float eps, int out_dtype, int id_dtype, int64_t vocab_begin, int64_t vocab_end,
                      int flags, cb200_status* status, cb200_stream_t stream) {
  if (!valid_qtype(qtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported block format %d", name, qtype);
  if (!valid_dtype(out_dtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported dtype code %d", name, out_dtype);
  if (dsts == nullptr || n_dsts < 1 || n_dsts > 8)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: between 1 and 8 destinations are supported, got %d", name, n_dsts);
  int rc = check_lookup(name, qtable, ids, dsts[0], vocab, hidden, n_ids, id_dtype);
  if (rc != CB200_OK) return rc;
  if (hidden % cb200::qblock_elems(qtype) != 0)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: hidden size %d is not divisible by %d", name, hidden,
                cb200::qblock_elems(qtype));
  if (vocab_begin < 0 || vocab_end < vocab_begin || vocab_end > vocab)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: bad vocab shard [%lld, %lld) of %lld", name, (long long)vocab_begin,
                (long long)vocab_end, (long long)vocab);
  if (row_bounds != nullptr) {
    if (row_bounds[0] != 0 || row_bounds[n_dsts] != n_ids)
      return fail(CB200_E_INVALID_ARGUMENT, "%s: row bounds must run from 0 to n_ids (%lld), got %lld .. %lld", name,
                  (long long)n_ids, (long long)row_bounds[0], (long long)row_bounds[n_dsts]);
    for (int d = 0; d < n_dsts; ++d)
      if (row_bounds[d + 1] < row_bounds[d])
        return fail(CB200_E_INVALID_ARGUMENT, "%s: row bounds must not decrease (entry %d)", name, d + 1);
  }
  if (n_ids == 0) return CB200_OK;
  if (alpha == nullptr) return fail(CB200_E_INVALID_ARGUMENT, "%s: null tensor pointer", name);
  if (!aligned16(alpha) || !aligned16(qtable))
    return fail(CB200_E_INVALID_ARGUMENT, "%s: alpha and the table must be 16-byte aligned", name);
  for (int d = 0; d < n_dsts; ++d) {
    const bool empty = row_bounds != nullptr && row_bounds[d + 1] == row_bounds[d];
    if ((dsts[d] == nullptr && !empty) || !aligned16(dsts[d]))
      return fail(CB200_E_INVALID_ARGUMENT, "%s: destination %d is null or not 16-byte aligned", name, d);
  }
  if (!fusable_qtype(qtype) || out_dtype == CB200_DTYPE_F32 || !cb200::qrms_rowreg_supported(out_dtype, hidden))
    return fail(CB200_E_INVALID_ARGUMENT,
                "%s: needs the single-launch kernel (Q4_0 / Q8_0 blocks, f16 / bf16 output, hidden a multiple of 32 "
                "that splits over 32, 64 or 128 threads); got format %d, dtype %d, hidden %d", name, qtype,
                out_dtype, hidden);
  cb200::QRmsArgs a{};
  a.qtable = static_cast<const unsigned char*>(qtable);
  a.ids = ids;
  a.alpha = static_cast<const uint4*>(alpha);
  a.y = static_cast<uint4*>(dsts[0]);
  a.id_dtype = id_dtype;
  a.vocab = vocab;
  a.vocab_begin = vocab_begin;
  a.vocab_end = vocab_end;
  a.status = status;
  a.rows = n_ids;
  a.V = hidden / 8;
  a.n = hidden;
  a.row_bytes = hidden / cb200::qblock_elems(qtype) * cb200::qblock_bytes(qtype);
  a.bulk = aligned16(qtable) && a.row_bytes % 16 == 0;
  a.eps = eps;
  a.flags = flags;
  a.owned_only = row_bounds != nullptr ? 2 : 1;
  a.n_more = n_dsts - 1;
  for (int d = 1; d < n_dsts; ++d) a.y_more[d - 1] = static_cast<uint4*>(dsts[d]);
  if (row_bounds != nullptr)
    for (int d = 0; d <= n_dsts; ++d) a.row_bounds[d] = row_bounds[d];
  return cuda_result(cb200::launch_qrms_rowreg(qtype, out_dtype, a, stream), name);
}

int cb200_qembedding_rms_norm_owner(const void* qtable, int qtype, const void* ids, const void* alpha,
                                    void* const* dsts, int n_dsts, int64_t vocab, int32_t hidden, int64_t n_ids,
                                    float eps, int out_dtype, int id_dtype, int64_t vocab_begin, int64_t vocab_end,
                                    int flags, cb200_status* status, cb200_stream_t stream) {
  const TraceRange trace("cb200_qembedding_rms_norm_owner");
  return owner_impl("cb200_qembedding_rms_norm_owner", qtable, qtype, ids, alpha, dsts, n_dsts, nullptr, vocab, hidden,
                    n_ids, eps, out_dtype, id_dtype, vocab_begin, vocab_end, flags, status, stream);
}

int cb200_qembedding_rms_norm_row_owner(const void* qtable, int qtype, const void* ids, const void* alpha,
                                        void* const* dsts, int n_dsts, const int64_t* row_bounds, int64_t vocab,
                                        int32_t hidden, int64_t n_ids, float eps, int out_dtype, int id_dtype,
                                        int64_t vocab_begin, int64_t vocab_end, int flags, cb200_status* status,
                                        cb200_stream_t stream) {
  const TraceRange trace("cb200_qembedding_rms_norm_row_owner");
  const char* name = "cb200_qembedding_rms_norm_row_owner";
  if (row_bounds == nullptr) return fail(CB200_E_INVALID_ARGUMENT, "%s: null row bounds", name);
  return owner_impl(name, qtable, qtype, ids, alpha, dsts, n_dsts, row_bounds, vocab, hidden, n_ids, eps, out_dtype,
                    id_dtype, vocab_begin, vocab_end, flags, status, stream);
}

int cb200_qembedding_route_rows(const void* qtable, int qtype, const void* ids, void* const* dsts, int n_dsts,
                                const int64_t* row_bounds, int64_t vocab, int32_t hidden, int64_t n_ids, int id_dtype,
                                int64_t vocab_begin, int64_t vocab_end, cb200_status* status, cb200_stream_t stream) {
  const TraceRange trace("cb200_qembedding_route_rows");
  const char* name = "cb200_qembedding_route_rows";
  if (!valid_qtype(qtype)) return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported block format %d", name, qtype);
  if (dsts == nullptr || row_bounds == nullptr || n_dsts < 1 || n_dsts > 8)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: between 1 and 8 destinations with their row bounds are needed, got %d", name,
                n_dsts);
  int rc = check_lookup(name, qtable, ids, dsts[0], vocab, hidden, n_ids, id_dtype);
  if (rc != CB200_OK) return rc;
  if (hidden % cb200::qblock_elems(qtype) != 0)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: hidden size %d is not divisible by %d", name, hidden,
                cb200::qblock_elems(qtype));
  if (vocab_begin < 0 || vocab_end < vocab_begin || vocab_end > vocab)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: bad vocab shard [%lld, %lld) of %lld", name, (long long)vocab_begin,
                (long long)vocab_end, (long long)vocab);
  if (row_bounds[0] != 0 || row_bounds[n_dsts] != n_ids)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: row bounds must run from 0 to n_ids (%lld), got %lld .. %lld", name,
                (long long)n_ids, (long long)row_bounds[0], (long long)row_bounds[n_dsts]);
  for (int d = 0; d < n_dsts; ++d) {
    if (row_bounds[d + 1] < row_bounds[d])
      return fail(CB200_E_INVALID_ARGUMENT, "%s: row bounds must not decrease (entry %d)", name, d + 1);
    if (dsts[d] == nullptr && row_bounds[d + 1] != row_bounds[d])
      return fail(CB200_E_INVALID_ARGUMENT, "%s: destination %d is null", name, d);
    if (reinterpret_cast<uintptr_t>(dsts[d]) & 1u)
      return fail(CB200_E_INVALID_ARGUMENT, "%s: destination %d is not 2-byte aligned", name, d);
  }
  if (n_ids == 0 || hidden == 0) return CB200_OK;
  if (reinterpret_cast<uintptr_t>(qtable) & 1u)
    return fail(CB200_E_INVALID_ARGUMENT, "%s: the table must be 2-byte aligned", name);
  const int row_bytes = hidden / cb200::qblock_elems(qtype) * cb200::qblock_bytes(qtype);
  return cuda_result(cb200::launch_qroute_rows(static_cast<const unsigned char*>(qtable), ids, id_dtype, vocab, vocab_begin,
                                               vocab_end, status, n_ids, row_bytes, dsts, n_dsts, row_bounds, stream),
                     name);
}

}  // extern "C"
