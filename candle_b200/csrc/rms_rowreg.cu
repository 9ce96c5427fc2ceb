// Kernels and launchers of the register-resident RMS norm (see rms_rowreg.cuh for the method):
// dense rows (optionally + residual), rows gathered from a dense table, and rows decoded on the
// fly from a Q4_0 / Q8_0 table staged into shared memory by the bulk-copy engine.
//
// All kernels are persistent: the grid is as many CTAs as fit on the device and each CTA walks
// rows with a stride.  Loaded HBM latency on B200 is about 3 us, so an SM needs on the order of
// 100 KB of reads in flight at all times; the dense kernel gets there by starting the next row's
// 16-byte asynchronous copies before it processes the current row, the quantised kernel by
// keeping a ring of bulk copies in flight.
#include "launch.h"
#include "qblocks.cuh"
#include "rms_rowreg.cuh"

namespace cb200 {

// Dense rows.  Every row slot of a CTA owns a ring of `stages` staging buffers in shared memory.
// Each thread copies its own 16-byte vectors of the rows ahead (and of their residual rows) into
// the ring with asynchronous copies, which need no registers while in flight, and only ever reads
// back the vectors it copied itself, so no barrier guards the ring.  A buffer is refilled once its
// row's T(m) is known; until then it doubles as the place where h is parked if the row needs the
// exact replay.  Three 256-thread CTAs with two 32 KB buffers each keep up to 192 KB of reads in
// flight per SM.
template <int VPT, int BT>
constexpr int rowreg_min_blocks() {
  return (VPT == 8 ? 512 : 768) / BT;
}

template <int DT, int VPT, int BT>
__global__ void __launch_bounds__(BT, rowreg_min_blocks<VPT, BT>()) rms_rowreg_kernel(const RmsRowRegArgs a, int stages) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tx = threadIdx.x, ty = threadIdx.y, tpr = blockDim.x, rpc = blockDim.y;
  RowRegSmem sm(smem_raw, rpc, tpr, a.V, ty);
  const bool has_res = a.res != nullptr;
  const int buf_vecs = has_res ? 2 * a.V : a.V;
  uint4* ring = reinterpret_cast<uint4*>(smem_raw + RowRegSmem::bytes(rpc, tpr, a.V, false)) +
                static_cast<size_t>(ty) * stages * buf_vecs;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * rpc;

  // Starts the copies of row r into ring slot `slot` (one copy group per call, empty if there is
  // nothing to copy); returns whether the row is live (inside the tensor and with a valid id).
  auto issue = [&](int64_t r, int slot) -> bool {
    bool ok = r < a.rows;
    const uint4* xr = nullptr;
    if (ok) {
      if (a.ids != nullptr) {
        const uint64_t id = read_id(a.ids, a.id_dtype, r);
        if (id >= static_cast<uint64_t>(a.vocab)) {
          if (tx == 0) report_status(a.status, CB200_STATUS_INVALID_INDEX, r, static_cast<int64_t>(id), a.vocab);
          ok = false;
        } else {
          xr = a.x + id * a.V;
        }
      } else {
        xr = a.x + r * a.V;
      }
    }
    if (ok) {
      uint4* sx = ring + static_cast<size_t>(slot) * buf_vecs;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = k * tpr + tx;
        if (v < a.V) cp_async16(sx + v, xr + v);
      }
      if (has_res) {
        const uint4* rr = a.res + r * a.V;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = k * tpr + tx;
          if (v < a.V) cp_async16(sx + a.V + v, rr + v);
        }
      }
    }
    cp_async_commit();
    return ok;
  };

  int64_t row = static_cast<int64_t>(blockIdx.x) * rpc + ty;
  uint32_t live_bits = 0;  // bit s: the row in ring slot s is live
  for (int j = 0; j < stages; ++j)
    if (issue(row + j * stride, j)) live_bits |= 1u << j;
  int slot = 0;
  while (row < a.rows) {
    cp_async_wait_pending(stages - 1);
    uint4* sx = ring + static_cast<size_t>(slot) * buf_vecs;
    const bool live = (live_bits >> slot) & 1u;
    uint4 h[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = k * tpr + tx;
      if (v < a.V && live)
        h[k] = has_res ? add_round_vec<DT>(sx[v], sx[a.V + v]) : sx[v];
      else
        h[k] = make_uint4(0, 0, 0, 0);
    }
    float lsum = 0.0f, lw = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = k * tpr + tx;
      if (v < a.V) accumulate_vec<DT>(h[k], v, a.n, lsum, lw);
    }
    const float m = resolve_row_m<DT, VPT>(h, lsum, lw, a.V, a.n, a.eps, a.flags, sm, sx);
    // the slot is free now (a replay, if any, is over): refill it with the row `stages` ahead
    if (issue(row + static_cast<int64_t>(stages) * stride, slot))
      live_bits |= 1u << slot;
    else
      live_bits &= ~(1u << slot);
    if (live) {
      if (a.sum_out != nullptr) {
        uint4* so = a.sum_out + row * a.V;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = k * tpr + tx;
          if (v < a.V) stg_stream(so + v, h[k]);
        }
      }
      write_rms_row<DT, VPT>(h, m, a.alpha, a.y + row * a.V, a.V);
    }
    row += stride;
    slot = slot + 1 == stages ? 0 : slot + 1;
  }
  cp_async_wait_all();
}

// ---------------------------------------------------------------------------------------------
// Quantised source: each CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ... through a ring of
// shared-memory row buffers that thread 0 keeps filled with bulk copies kQStages-1 rows ahead.
// ---------------------------------------------------------------------------------------------
constexpr int kQStages = 8;

template <int QT, int DT, int VPT, int BT>
__global__ void __launch_bounds__(BT, 1024 / BT) qrms_rowreg_kernel(const QRmsArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tx = threadIdx.x, tpr = blockDim.x;
  RowRegSmem sm(smem_raw, 1, tpr, a.V, 0);
  const size_t core_bytes = RowRegSmem::bytes(1, tpr, a.V, true);
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
  if (a.bulk && tx == 0) {
    for (int j = 0; j < kQStages - 1; ++j)
      if (first + j * step < a.rows) issue(first + j * step, j);
  }
  uint32_t phase = 0;  // one parity bit per stage
  int it = 0;
  for (int64_t row = first; row < a.rows; row += step, ++it) {
    const int stage = it % kQStages;
    unsigned char* buf = stage0 + stage * stage_bytes;
    uint64_t id;
    const int kind = classify(row, id);
    // The stage used by the previous row is free: its readers finished before that row's first
    // barrier, which thread 0 has passed.  Refill it with the row kQStages-1 ahead.
    if (a.bulk && tx == 0) {
      const int64_t ahead = row + static_cast<int64_t>(kQStages - 1) * step;
      if (ahead < a.rows) issue(ahead, (it + kQStages - 1) % kQStages);
    }
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
    const float m = resolve_row_m<DT, VPT>(h, lsum, lw, a.V, a.n, a.eps, a.flags, sm, sm.rows);
    if (*abort_flag) {
      if (tx == 0) {
        report_status(a.status, CB200_STATUS_WAIT_TIMEOUT, row, static_cast<int64_t>(id), a.vocab);
        // bounded second chance for every copy still in flight, so that none lands in shared
        // memory after the CTA has retired
        for (int j = 0; j < kQStages; ++j) {
          const int64_t r = row + static_cast<int64_t>(j) * step;
          uint64_t rid;
          if (r >= a.rows || classify(r, rid) != 0) continue;
          const int s = (it + j) % kQStages;
          const uint32_t par = (j == 0) ? (((phase >> s) & 1u) ^ 1u) : ((phase >> s) & 1u);
          mbar_wait(&bars[s], par);
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
    // reads the published m before the next row's first barrier, so the refill issued at the
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

// A persistent grid: as many CTAs as are resident at once, but no more than there is work.
template <typename K>
static cudaError_t persistent_grid(K kern, int threads, size_t smem, int64_t work_items, unsigned& grid) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                       static_cast<int>(cudaSharedmemCarveoutMaxShared));
  if (e != cudaSuccess) return e;
  if (smem > 48 * 1024) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  int per_sm = 1;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, smem);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) per_sm = 1;
  int64_t g = static_cast<int64_t>(kSmCount) * per_sm;
  if (g > work_items) g = work_items;
  grid = static_cast<unsigned>(g);
  return cudaSuccess;
}

template <int DT, int VPT, int BT>
static cudaError_t launch_dense_t(const RmsRowRegArgs& a, int tpr, int rpc, cudaStream_t stream) {
  const size_t head = RowRegSmem::bytes(rpc, tpr, a.V, false);
  const size_t buf = static_cast<size_t>(rpc) * a.V * 16 * (a.res != nullptr ? 2 : 1);  // one ring slot of the CTA
  // ring depth: fill about 200 KB of an SM's shared memory with the CTAs the register cap admits
  const int ctas = rowreg_min_blocks<VPT, BT>();
  const size_t budget = (200 * 1024) / ctas;
  int stages = budget > head ? static_cast<int>((budget - head) / buf) : 1;
  if (stages > 4) stages = 4;
  if (stages < 1) stages = 1;
  const size_t smem = head + stages * buf;
  auto kern = rms_rowreg_kernel<DT, VPT, BT>;
  unsigned grid = 1;
  cudaError_t e = persistent_grid(kern, tpr * rpc, smem, (a.rows + rpc - 1) / rpc, grid);
  if (e != cudaSuccess) return e;
  kern<<<grid, dim3(tpr, rpc), smem, stream>>>(a, stages);
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
  const size_t smem =
      RowRegSmem::bytes(1, tpr, a.V, true) + static_cast<size_t>(kQStages) * stage_bytes + kQStages * 8 + 8;
  auto kern = qrms_rowreg_kernel<QT, DT, VPT, BT>;
  unsigned grid = 1;
  cudaError_t e = persistent_grid(kern, tpr, smem, a.rows, grid);
  if (e != cudaSuccess) return e;
  kern<<<grid, tpr, smem, stream>>>(a);
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
