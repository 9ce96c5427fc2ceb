// Kernels and launchers of the register-resident RMS norm (see rms_rowreg.cuh for the method):
// dense rows (optionally + residual), rows gathered from a dense table, and rows decoded on the
// fly from a Q4_0 / Q8_0 table staged into shared memory by the bulk-copy engine.
#include "launch.h"
#include "qblocks.cuh"
#include "rms_rowreg.cuh"

namespace cb200 {

// Registers are capped so that 1536 threads (1024 for the 8-vector variant) stay resident per SM.
template <int VPT, int BT>
constexpr int rowreg_min_blocks() {
  return (VPT == 8 ? 1024 : 1536) / BT;
}

template <int DT, int VPT, int BT>
__global__ void __launch_bounds__(BT, rowreg_min_blocks<VPT, BT>()) rms_rowreg_kernel(const RmsRowRegArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tx = threadIdx.x, ty = threadIdx.y, tpr = blockDim.x, rpc = blockDim.y;
  RowRegSmem sm(smem_raw, rpc, a.V, ty);

  const int64_t row = static_cast<int64_t>(blockIdx.x) * rpc + ty;
  bool live = row < a.rows;
  const uint4* xr = nullptr;
  if (live) {
    if (a.ids != nullptr) {
      uint64_t id = read_id(a.ids, a.id_dtype, row);
      if (id >= static_cast<uint64_t>(a.vocab)) {
        if (tx == 0) report_status(a.status, CB200_STATUS_INVALID_INDEX, row, static_cast<int64_t>(id), a.vocab);
        live = false;
      } else {
        xr = a.x + id * a.V;
      }
    } else {
      xr = a.x + row * a.V;
    }
  }
  const uint4* rr = (live && a.res != nullptr) ? a.res + row * a.V : nullptr;

  uint4 h[VPT];
  uint4 rv[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    int v = k * tpr + tx;
    h[k] = (live && v < a.V) ? ldg_stream(xr + v) : make_uint4(0, 0, 0, 0);
  }
  if (rr != nullptr) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      int v = k * tpr + tx;
      rv[k] = (v < a.V) ? ldg_stream(rr + v) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) h[k] = add_round_vec<DT>(h[k], rv[k]);
  }
  float lsum = 0.0f, lw = 0.0f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    int v = k * tpr + tx;
    if (v < a.V) accumulate_vec<DT>(h[k], v, a.n, lsum, lw);
  }
  if (live && a.sum_out != nullptr) {
    uint4* so = a.sum_out + row * a.V;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      int v = k * tpr + tx;
      if (v < a.V) stg_stream(so + v, h[k]);
    }
  }
  const float m = resolve_row_m<DT, VPT>(h, lsum, lw, a.V, a.n, a.eps, a.flags, sm);
  if (live) write_rms_row<DT, VPT>(h, m, a.alpha, a.y + row * a.V, a.V);
}

// ---------------------------------------------------------------------------------------------
// Quantised source: each CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ... with a two-stage
// ring of shared-memory row buffers; one thread issues the bulk copy of the next row while the
// CTA decodes and normalises the current one.
// ---------------------------------------------------------------------------------------------

constexpr int kQStages = 2;

template <int QT, int DT, int VPT, int BT>
__global__ void __launch_bounds__(BT, (VPT >= 4 ? 1024 : 1536) / BT) qrms_rowreg_kernel(const QRmsArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tx = threadIdx.x, tpr = blockDim.x;
  RowRegSmem sm(smem_raw, 1, a.V, 0);
  const size_t core_bytes = RowRegSmem::bytes(1, a.V, true);
  const int stage_bytes = (a.row_bytes + 15) & ~15;
  unsigned char* stage0 = smem_raw + core_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage0 + kQStages * stage_bytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kQStages);

  if (tx == 0) {
    for (int s = 0; s < kQStages; ++s) mbar_init(&bars[s], 1);
    mbar_init_fence();
    *abort_flag = 0;
  }
  __syncthreads();

  // Row state for a pipeline slot: 0 = decode from the staged bytes, 1 = masked (-0.0 row),
  // 2 = skip (bad id).  Computed identically by every thread from the id.
  auto classify = [&](int64_t row, uint64_t& id) -> int {
    id = read_id(a.ids, a.id_dtype, row);
    if (id >= static_cast<uint64_t>(a.vocab)) return 2;
    if (id < static_cast<uint64_t>(a.vocab_begin) || id >= static_cast<uint64_t>(a.vocab_end)) return 1;
    return 0;
  };
  auto issue = [&](int64_t row, int stage) {  // thread 0 only
    uint64_t id;
    if (classify(row, id) != 0) return;
    const unsigned char* src = a.qtable + (id - a.vocab_begin) * static_cast<uint64_t>(a.row_bytes);
    mbar_expect_tx(&bars[stage], static_cast<uint32_t>(a.row_bytes));
    bulk_g2s(stage0 + stage * stage_bytes, src, static_cast<uint32_t>(a.row_bytes), &bars[stage]);
  };

  const int64_t first = blockIdx.x, step = gridDim.x;
  if (a.bulk && tx == 0 && first < a.rows) issue(first, 0);
  uint32_t phase = 0;  // one parity bit per stage
  int it = 0;
  for (int64_t row = first; row < a.rows; row += step, ++it) {
    const int stage = it % kQStages;
    unsigned char* buf = stage0 + stage * stage_bytes;
    uint64_t id;
    const int kind = classify(row, id);
    // The other stage is free: its readers finished before the previous row's first barrier.
    if (a.bulk && tx == 0 && row + step < a.rows) issue(row + step, (it + 1) % kQStages);
    if (kind == 0) {
      if (a.bulk) {
        // A wait that runs out is recorded and acted on after the row's barriers, where the
        // whole CTA sees the flag and can leave together.
        if (!mbar_wait(&bars[stage], (phase >> stage) & 1u)) *abort_flag = 1;
        phase ^= 1u << stage;
      } else {
        // rows that are not 16-byte multiples: cooperative 2-byte copies
        const uint16_t* src =
            reinterpret_cast<const uint16_t*>(a.qtable + (id - a.vocab_begin) * static_cast<uint64_t>(a.row_bytes));
        uint16_t* dst = reinterpret_cast<uint16_t*>(buf);
        for (int i = tx; i < a.row_bytes / 2; i += tpr) dst[i] = src[i];
        __syncthreads();
      }
    }
    if (kind == 2 && tx == 0) report_status(a.status, CB200_STATUS_INVALID_INDEX, row, static_cast<int64_t>(id), a.vocab);

    uint4 h[VPT];
    float lsum = 0.0f, lw = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      int v = k * tpr + tx;
      if (v < a.V && kind == 0) {
        h[k] = decode_vec8<QT, DT>(buf, v);
        accumulate_vec<DT>(h[k], v, a.n, lsum, lw);
      } else {
        h[k] = (kind == 1) ? neg_zero_vec<DT>() : make_uint4(0, 0, 0, 0);
      }
    }
    const float m = resolve_row_m<DT, VPT>(h, lsum, lw, a.V, a.n, a.eps, a.flags, sm);
    if (*abort_flag) {
      if (tx == 0) {
        report_status(a.status, CB200_STATUS_WAIT_TIMEOUT, row, static_cast<int64_t>(id), a.vocab);
        // bounded second chance for this row's copy and for the prefetch of the next one, so
        // that no copy lands in shared memory after the CTA has retired
        mbar_wait(&bars[stage], ((phase >> stage) & 1u) ^ 1u);
        uint64_t nid;
        if (row + step < a.rows && classify(row + step, nid) == 0) {
          const int ns = (it + 1) % kQStages;
          mbar_wait(&bars[ns], (phase >> ns) & 1u);
        }
      }
      return;
    }
    if (kind != 2) {
      if (a.gathered != nullptr) {
        uint4* g = a.gathered + row * a.V;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          int v = k * tpr + tx;
          if (v < a.V) stg_stream(g + v, h[k]);
        }
      }
      write_rms_row<DT, VPT>(h, m, a.alpha, a.y + row * a.V, a.V);
    }
    // No barrier here: every thread finished decoding `buf` before the row's first barrier and
    // reads the published m before the next row's first barrier, so the prefetch issued at the
    // top of the next iteration and the next row's scratch writes cannot race with this row.
  }
}

// ---------------------------------------------------------------------------------------------
// Launchers
// ---------------------------------------------------------------------------------------------
static void rowreg_shape(int V, int& tpr, int& vpt, int& rpc) {
  int want = (V + 3) / 4;
  tpr = 32;
  while (tpr < want && tpr < 512) tpr <<= 1;
  vpt = (V + tpr - 1) / tpr;
  rpc = tpr >= 128 ? 1 : 128 / tpr;
}

bool rms_rowreg_supported(int dtype, int cols) {
  return (dtype == kDtBF16 || dtype == kDtF16) && cols % 8 == 0 && cols >= 8 && cols <= 32768;
}

template <int DT, int VPT, int BT>
static cudaError_t launch_dense_t(const RmsRowRegArgs& a, int tpr, int rpc, cudaStream_t stream) {
  const bool with_rows = !(a.flags & CB200_FLAG_FAST_SUM);
  size_t smem = RowRegSmem::bytes(rpc, a.V, with_rows);
  auto kern = rms_rowreg_kernel<DT, VPT, BT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  dim3 block(tpr, rpc);
  dim3 grid(static_cast<unsigned>((a.rows + rpc - 1) / rpc));
  kern<<<grid, block, smem, stream>>>(a);
  return cudaGetLastError();
}

template <int DT, int VPT>
static cudaError_t launch_dense_bt(const RmsRowRegArgs& a, int tpr, int rpc, cudaStream_t stream) {
  const int bt = tpr * rpc;
  if (bt <= 128) return launch_dense_t<DT, VPT, 128>(a, tpr, rpc, stream);
  if (bt <= 256) return launch_dense_t<DT, VPT, 256>(a, tpr, rpc, stream);
  return launch_dense_t<DT, VPT, 512>(a, tpr, rpc, stream);
}

template <int DT>
static cudaError_t launch_dense_dt(const RmsRowRegArgs& a, cudaStream_t stream) {
  int tpr, vpt, rpc;
  rowreg_shape(a.V, tpr, vpt, rpc);
  if (vpt <= 1) return launch_dense_bt<DT, 1>(a, tpr, rpc, stream);
  if (vpt <= 2) return launch_dense_bt<DT, 2>(a, tpr, rpc, stream);
  if (vpt <= 4) return launch_dense_bt<DT, 4>(a, tpr, rpc, stream);
  return launch_dense_bt<DT, 8>(a, tpr, rpc, stream);
}

cudaError_t launch_rms_rowreg(int dtype, const RmsRowRegArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  return dtype == kDtBF16 ? launch_dense_dt<kDtBF16>(a, stream) : launch_dense_dt<kDtF16>(a, stream);
}

template <int QT, int DT, int VPT, int BT>
static cudaError_t launch_q_t(const QRmsArgs& a, int tpr, cudaStream_t stream) {
  const int stage_bytes = (a.row_bytes + 15) & ~15;
  size_t smem = RowRegSmem::bytes(1, a.V, true) + static_cast<size_t>(kQStages) * stage_bytes + kQStages * 8 + 8;
  auto kern = qrms_rowreg_kernel<QT, DT, VPT, BT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  // persistent: exactly as many CTAs as fit on the device, each streaming rows through its ring
  int ctas_per_sm = 1;
  cudaError_t oe = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, kern, tpr, smem);
  if (oe != cudaSuccess) return oe;
  if (ctas_per_sm < 1) ctas_per_sm = 1;
  int64_t grid = static_cast<int64_t>(kSmCount) * ctas_per_sm;
  if (grid > a.rows) grid = a.rows;
  kern<<<static_cast<unsigned>(grid), tpr, smem, stream>>>(a);
  return cudaGetLastError();
}

template <int QT, int DT, int VPT>
static cudaError_t launch_q_bt(const QRmsArgs& a, int tpr, cudaStream_t stream) {
  if (tpr <= 128) return launch_q_t<QT, DT, VPT, 128>(a, tpr, stream);
  if (tpr <= 256) return launch_q_t<QT, DT, VPT, 256>(a, tpr, stream);
  return launch_q_t<QT, DT, VPT, 512>(a, tpr, stream);
}

template <int QT, int DT>
static cudaError_t launch_q_dt(const QRmsArgs& a, cudaStream_t stream) {
  int tpr, vpt, rpc;
  rowreg_shape(a.V, tpr, vpt, rpc);
  if (tpr < 512 && vpt > 2) tpr *= 2;  // the decoder needs registers: two vectors per thread where possible
  if (tpr < 64) tpr = 64;              // one row per CTA here: keep at least two warps busy
  vpt = (a.V + tpr - 1) / tpr;
  if (vpt <= 1) return launch_q_bt<QT, DT, 1>(a, tpr, stream);
  if (vpt <= 2) return launch_q_bt<QT, DT, 2>(a, tpr, stream);
  if (vpt <= 4) return launch_q_bt<QT, DT, 4>(a, tpr, stream);
  return launch_q_bt<QT, DT, 8>(a, tpr, stream);
}

cudaError_t launch_qrms_rowreg(int qtype, int dtype, const QRmsArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  if (qtype == CB200_QTYPE_Q8_0)
    return dtype == kDtBF16 ? launch_q_dt<CB200_QTYPE_Q8_0, kDtBF16>(a, stream)
                            : launch_q_dt<CB200_QTYPE_Q8_0, kDtF16>(a, stream);
  return dtype == kDtBF16 ? launch_q_dt<CB200_QTYPE_Q4_0, kDtBF16>(a, stream)
                          : launch_q_dt<CB200_QTYPE_Q4_0, kDtF16>(a, stream);
}

}  // namespace cb200
