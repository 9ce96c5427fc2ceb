// Host-side launcher declarations shared by the .cu files and the C ABI layer.
#pragma once

#include "common.cuh"

namespace cb200 {

// launch_cache.cu: per-device values and per-kernel attributes, set up once and cached.
// device_sm_count: SMs of the current device.  kernel_launch_config: raises `func`'s dynamic
// shared-memory limit to the architectural maximum (once), applies the shared-memory carve-out
// preference when it changes (pass -1 to leave it alone) and returns how many CTAs of `threads`
// threads and `smem` dynamic bytes fit on an SM (pass NULL to skip the query).
cudaError_t device_sm_count(int* out);
cudaError_t kernel_launch_config(const void* func, int threads, size_t smem, int carveout_percent,
                                 int* ctas_per_sm);

// The wait parameters every launcher copies into its kernel's arguments (launch_cache.cu).
WaitTuning wait_tuning();
void set_wait_tuning(WaitTuning t);

// SMs of the current device for grid sizing; if the query fails the launch that follows reports
// the error, and 148 (B200) stands in meanwhile.
inline int sm_count() {
  int n = 148;
  return device_sm_count(&n) == cudaSuccess ? n : 148;
}

constexpr int kOpRmsNorm = 0;
constexpr int kOpLayerNorm = 1;

// Arguments of the lane-per-row and any-shape norm kernels.
struct LaneRowArgs {
  const void* x;      // [rows, n], or the dense table [vocab, n] when ids != nullptr
  const void* res;    // optional residual (dense source only)
  const void* alpha;  // weight [n]
  const void* beta;   // bias [n] (layer norm)
  void* y;
  void* sum_out;      // optional: h = x + res, or the gathered rows
  const void* ids;
  int id_dtype;
  int64_t vocab;
  cb200_status* status;
  int64_t rows;
  int n;
  float eps;
  int bulk;   // gather source: stage rows with the bulk-copy engine
  int V;      // filled by the launcher: 16-byte vectors per row
  int pitch;  // filled by the launcher: shared-memory row pitch in bytes
  int R;      // filled by the launcher: rows per CTA
  int classic;  // keep to the whole-row kernel where the streaming one would apply (cross-checks)
  WaitTuning wt;  // filled by the launcher
};

struct RmsRowRegArgs;
struct QRmsArgs;

bool rms_rowreg_supported(int dtype, int cols);
bool qrms_rowreg_supported(int dtype, int cols);
cudaError_t launch_rms_rowreg(int dtype, const RmsRowRegArgs& a, cudaStream_t stream);
cudaError_t launch_qrms_rowreg(int qtype, int dtype, const QRmsArgs& a, cudaStream_t stream);
// lookup + RMS norm for the K-quant super-block formats (kqrms.cu)
bool kqrms_supported(int qtype, int dtype, int cols);
cudaError_t launch_kqrms(int qtype, int dtype, const QRmsArgs& a, cudaStream_t stream);

bool norm_lanerow_supported(int dtype, int cols);
cudaError_t launch_norm_lanerow(int dtype, int op, const LaneRowArgs& a, cudaStream_t stream);
cudaError_t launch_norm_generic(int dtype, int op, const LaneRowArgs& a, cudaStream_t stream);

// candle's composite norm (norm_slow.cu); bias may be NULL
cudaError_t launch_norm_slow(int dtype, const void* x, const void* weight, const void* bias, void* y, int64_t rows,
                             int n, float eps, int remove_mean, cudaStream_t stream);

// softmax over the last dimension and rotary embeddings (neighbours.cu).  rope variants: 0 rope_i
// (interleaved pairs, src [b, h, t, d]), 1 rope (half-split pairs, [b, h, t, d]), 2 rope_thd ([b, t, h, d]).
cudaError_t launch_softmax_last_dim(int dtype, const void* x, void* y, int64_t rows, int n, cudaStream_t stream);
cudaError_t launch_rope(int variant, int dtype, const void* src, const void* cos_, const void* sin_, void* dst, int64_t b,
                        int h, int t, int d, cudaStream_t stream);

// Row gathers (embedding.cu)
struct GatherArgs {
  const unsigned char* src;  // [left, src_dim, row_bytes]
  const void* ids;
  unsigned char* out;        // [left, n_ids, row_bytes]
  int64_t left, src_dim, n_ids;
  int64_t row_bytes;
  int id_dtype;
  cb200_status* status;
  WaitTuning wt;  // filled by the launcher
};
cudaError_t launch_gather_rows(const GatherArgs& a, cudaStream_t stream);

struct QGatherArgs {
  const unsigned char* qtable;
  const void* ids;
  void* out;
  int id_dtype;
  int64_t vocab, vocab_begin, vocab_end;
  cb200_status* status;
  int64_t rows;
  int n;          // elements per row (multiple of 32)
  int row_bytes;  // bytes per quantised row
  int bulk;
  WaitTuning wt;  // filled by the launcher
};
cudaError_t launch_qgather(int qtype, int out_dtype, const QGatherArgs& a, cudaStream_t stream);
cudaError_t launch_qroute_rows(const unsigned char* qtable, const void* ids, int id_dtype, int64_t vocab,
                               int64_t vocab_begin, int64_t vocab_end, cb200_status* status, int64_t rows, int row_bytes,
                               void* const* dsts, int n_dsts, const int64_t* row_bounds, cudaStream_t stream);
cudaError_t launch_dequantize_flat(int qtype, int out_dtype, const void* blocks, void* out, int64_t n_vec,
                                   cudaStream_t stream);  // n_vec: groups of 8 elements

}  // namespace cb200
