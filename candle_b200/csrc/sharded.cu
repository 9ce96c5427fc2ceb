// The vocabulary-sharded lookup behind one C call: masked quantised lookup into scratch, NCCL sum,
// RMS norm.  Built into its own library (libcandle_b200_nccl.so).
#include <cstdarg>
#include <cstdio>

#include <cuda_runtime.h>
#include <nccl.h>

#include "../../include/candle_b200_nccl.h"

namespace {

thread_local char g_nccl_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_nccl_error, sizeof(g_nccl_error), fmt, ap);
  va_end(ap);
  fprintf(stderr, "candle_b200_nccl: %s\n", g_nccl_error);
  return code;
}

int nccl_result(ncclResult_t r, const char* what) {
  if (r == ncclSuccess) return CB200_OK;
  return fail(CB200_E_NCCL, "%s: %s", what, ncclGetErrorString(r));
}

size_t elem_bytes(int dtype) { return dtype == CB200_DTYPE_F32 ? 4 : 2; }

// Steps shared by the entry points: lookup into `scratch`, sum over ranks in place, normalise.
int sharded_steps(void* comm, const void* qtable, int qtype, const void* ids, const void* alpha, void* y,
                  void* scratch, int64_t vocab, int32_t hidden, int64_t n_ids, float eps, int out_dtype, int id_dtype,
                  int64_t vocab_begin, int64_t vocab_end, int flags, cb200_status* status, cb200_stream_t stream) {
  int rc = cb200_qembedding(qtable, qtype, ids, scratch, vocab, hidden, n_ids, out_dtype, id_dtype, vocab_begin,
                            vocab_end, status, stream);
  if (rc != CB200_OK) return fail(rc, "cb200_sharded_qembedding_rms_norm: %s", cb200_last_error());
  if (comm != nullptr) {
    const ncclDataType_t dt = out_dtype == CB200_DTYPE_F32 ? ncclFloat32 : (out_dtype == CB200_DTYPE_F16 ? ncclFloat16 : ncclBfloat16);
    rc = nccl_result(ncclAllReduce(scratch, scratch, static_cast<size_t>(n_ids) * hidden, dt, ncclSum,
                                   static_cast<ncclComm_t>(comm), reinterpret_cast<cudaStream_t>(stream)),
                     "ncclAllReduce");
    if (rc != CB200_OK) return rc;
  }
  rc = cb200_rms_norm(scratch, nullptr, alpha, y, nullptr, n_ids, hidden, eps, out_dtype, flags, stream);
  if (rc != CB200_OK) return fail(rc, "cb200_sharded_qembedding_rms_norm: %s", cb200_last_error());
  return CB200_OK;
}

}  // namespace

extern "C" {

int cb200_nccl_unique_id(void* id_out) {
  static_assert(sizeof(ncclUniqueId) == CB200_NCCL_UNIQUE_ID_BYTES, "unexpected ncclUniqueId size");
  if (id_out == nullptr) return fail(CB200_E_INVALID_ARGUMENT, "cb200_nccl_unique_id: null pointer");
  return nccl_result(ncclGetUniqueId(static_cast<ncclUniqueId*>(id_out)), "ncclGetUniqueId");
}

int cb200_nccl_comm_init(void** comm_out, int nranks, const void* id, int rank) {
  if (comm_out == nullptr || id == nullptr || nranks < 1 || rank < 0 || rank >= nranks)
    return fail(CB200_E_INVALID_ARGUMENT, "cb200_nccl_comm_init: bad arguments");
  ncclComm_t comm = nullptr;
  int rc = nccl_result(ncclCommInitRank(&comm, nranks, *static_cast<const ncclUniqueId*>(id), rank), "ncclCommInitRank");
  *comm_out = comm;
  return rc;
}

int cb200_nccl_comm_destroy(void* comm) {
  if (comm == nullptr) return CB200_OK;
  return nccl_result(ncclCommDestroy(static_cast<ncclComm_t>(comm)), "ncclCommDestroy");
}

int cb200_sharded_qembedding_rms_norm(void* comm, const void* qtable, int qtype, const void* ids, const void* alpha,
                                      void* y, void* scratch, size_t scratch_bytes, int64_t vocab, int32_t hidden,
                                      int64_t n_ids, float eps, int out_dtype, int id_dtype, int64_t vocab_begin,
                                      int64_t vocab_end, int flags, cb200_status* status, cb200_stream_t stream) {
  if (n_ids < 0 || hidden < 0) return fail(CB200_E_INVALID_ARGUMENT, "cb200_sharded_qembedding_rms_norm: negative shape");
  if (out_dtype != CB200_DTYPE_F32 && out_dtype != CB200_DTYPE_F16 && out_dtype != CB200_DTYPE_BF16)
    return fail(CB200_E_UNSUPPORTED_DTYPE, "cb200_sharded_qembedding_rms_norm: unsupported dtype code %d", out_dtype);
  const size_t need = static_cast<size_t>(n_ids) * hidden * elem_bytes(out_dtype);
  if (need == 0) return CB200_OK;
  if (scratch == nullptr || scratch_bytes < need)
    return fail(CB200_E_INVALID_ARGUMENT, "cb200_sharded_qembedding_rms_norm: scratch of %zu bytes needed, %zu given", need,
                scratch_bytes);
  return sharded_steps(comm, qtable, qtype, ids, alpha, y, scratch, vocab, hidden, n_ids, eps, out_dtype, id_dtype,
                       vocab_begin, vocab_end, flags, status, stream);
}

}  // extern "C"
