// The vocabulary-sharded lookup behind one C call: masked quantised lookup into scratch, NCCL sum,
// RMS norm.  Built into its own library (libcandle_b200_nccl.so).
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <thread>

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

// On a non-blocking communicator a call may return ncclInProgress; poll the communicator until it
// has settled or `timeout_ms` is over.  Blocking communicators never take the loop.
constexpr int kCollectiveAcceptMs = 30000;
int nccl_settle(ncclComm_t comm, ncclResult_t r, const char* what, int timeout_ms) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  while (r == ncclInProgress) {
    if (std::chrono::steady_clock::now() > deadline)
      return fail(CB200_E_TIMEOUT, "%s: not completed within %d ms", what, timeout_ms);
    std::this_thread::sleep_for(std::chrono::microseconds(200));
    ncclResult_t q = ncclCommGetAsyncError(comm, &r);
    if (q != ncclSuccess) return nccl_result(q, "ncclCommGetAsyncError");
  }
  return nccl_result(r, what);
}

// Steps shared by the entry points: lookup into `scratch`, sum over ranks in place, normalise.
int sharded_steps(void* comm, const void* qtable, int qtype, const void* ids, const void* alpha, void* y,
                  void* scratch, int64_t vocab, int32_t hidden, int64_t n_ids, float eps, int out_dtype, int id_dtype,
                  int64_t vocab_begin, int64_t vocab_end, int flags, cb200_status* status, cb200_stream_t stream) {
  int rc = cb200_qembedding(qtable, qtype, ids, scratch, vocab, hidden, n_ids, out_dtype, id_dtype, vocab_begin,
                            vocab_end, status, stream);
  if (rc != CB200_OK) return fail(rc, "cb200_sharded_qembedding_rms_norm: %s", cb200_last_error());
  if (comm != nullptr) {
    // The partial rows are summed as unsigned integers over their bit patterns: foreign rows are zero
    // bits, so every word has one non-zero contributor and comes out unchanged, whatever it encodes.
    const size_t bytes = static_cast<size_t>(n_ids) * hidden * elem_bytes(out_dtype);
    const bool words = bytes % 4 == 0;
    rc = nccl_settle(static_cast<ncclComm_t>(comm),
                     ncclAllReduce(scratch, scratch, words ? bytes / 4 : bytes, words ? ncclUint32 : ncclUint8, ncclSum,
                                   static_cast<ncclComm_t>(comm), reinterpret_cast<cudaStream_t>(stream)),
                     "ncclAllReduce", kCollectiveAcceptMs);
    if (rc != CB200_OK) return rc;
  }
  rc = cb200_rms_norm(scratch, nullptr, alpha, y, nullptr, n_ids, hidden, eps, out_dtype, flags, stream);
  if (rc != CB200_OK) return fail(rc, "cb200_sharded_qembedding_rms_norm: %s", cb200_last_error());
  return CB200_OK;
}

// Scratch for the allocation-free entry point.  It lives in the library image: every GPU that loads
// the library's device code carries these bytes until the process exits.  In host code the array's
// name is only a host-side handle, not a device address, so the address is looked up once per device
// (below) and that pointer is what the kernels get.  With CUDA's default lazy module loading the
// device image -- and with it the array's memory -- is brought onto a device by that first lookup,
// not when the host library is loaded; CUDA_MODULE_LOADING=EAGER moves it to context creation.
__device__ __align__(256) unsigned char g_static_scratch[CB200_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
void* g_static_ptr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// Device address of the static scratch on the CURRENT device; resolved on the first call per device.
int static_scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(CB200_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(CB200_E_CUDA, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(CB200_E_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
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

int cb200_nccl_comm_init_timeout(void** comm_out, int nranks, const void* id, int rank, int timeout_ms) {
  if (comm_out == nullptr || id == nullptr || nranks < 1 || rank < 0 || rank >= nranks || timeout_ms < 0)
    return fail(CB200_E_INVALID_ARGUMENT, "cb200_nccl_comm_init_timeout: bad arguments");
  *comm_out = nullptr;
  ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
  config.blocking = 0;
  ncclComm_t comm = nullptr;
  ncclResult_t r = ncclCommInitRankConfig(&comm, nranks, *static_cast<const ncclUniqueId*>(id), rank, &config);
  if (r != ncclSuccess && r != ncclInProgress) return nccl_result(r, "ncclCommInitRankConfig");
  int rc = comm != nullptr ? nccl_settle(comm, ncclInProgress, "ncclCommInitRankConfig", timeout_ms)
                           : fail(CB200_E_NCCL, "ncclCommInitRankConfig returned no communicator");
  if (rc != CB200_OK) {
    // a peer is missing (or NCCL failed): give the half-built communicator back, keep the message
    if (comm != nullptr) ncclCommAbort(comm);
    if (rc == CB200_E_TIMEOUT)
      return fail(rc, "cb200_nccl_comm_init_timeout: rank %d of %d: the ranks did not all join within %d ms", rank,
                  nranks, timeout_ms);
    return rc;
  }
  *comm_out = comm;
  return CB200_OK;
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

int cb200_sharded_qembedding_rms_norm_static(void* comm, const void* qtable, int qtype, const void* ids,
                                             const void* alpha, void* y, int64_t vocab, int32_t hidden, int64_t n_ids,
                                             float eps, int out_dtype, int id_dtype, int64_t vocab_begin,
                                             int64_t vocab_end, int flags, cb200_status* status,
                                             cb200_stream_t stream) {
  const char* name = "cb200_sharded_qembedding_rms_norm_static";
  if (n_ids < 0 || hidden < 0) return fail(CB200_E_INVALID_ARGUMENT, "%s: negative shape", name);
  if (out_dtype != CB200_DTYPE_F32 && out_dtype != CB200_DTYPE_F16 && out_dtype != CB200_DTYPE_BF16)
    return fail(CB200_E_UNSUPPORTED_DTYPE, "%s: unsupported dtype code %d", name, out_dtype);
  const size_t need = static_cast<size_t>(n_ids) * hidden * elem_bytes(out_dtype);
  if (need == 0) return CB200_OK;
  if (need > CB200_STATIC_SCRATCH_BYTES)
    return fail(CB200_E_UNSUPPORTED_SHAPE,
                "%s: %lld rows x %d columns need %zu bytes of scratch, the built-in scratch holds %zu; use "
                "cb200_sharded_qembedding_rms_norm with a buffer of your own",
                name, (long long)n_ids, hidden, need, static_cast<size_t>(CB200_STATIC_SCRATCH_BYTES));
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc != CB200_OK) return rc;
  // Nothing in the scratch has to start at zero: for valid ids the lookup writes every byte the later
  // steps read.  A row whose id is out of range is left unwritten (and recorded in `status`), so the
  // array's old contents are what gets summed and normalised for it: that row of y is undefined.
  return sharded_steps(comm, qtable, qtype, ids, alpha, y, scratch, vocab, hidden, n_ids, eps, out_dtype, id_dtype,
                       vocab_begin, vocab_end, flags, status, stream);
}

}  // extern "C"
