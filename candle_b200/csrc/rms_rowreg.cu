// Kernels and launchers of the register-resident RMS norm (see rms_rowreg.cuh for the method):
// dense rows (optionally + residual), rows gathered from a dense table, and rows decoded on the
// fly from a Q4_0 / Q8_0 table staged into shared memory by the bulk-copy engine.
//
// All kernels are persistent: the grid is as many CTAs as fit on the device and each CTA walks
// rows with a stride.  An SM needs on the order of 100 KB of reads in flight at all times to
// saturate HBM; the dense kernel gets there with 768 resident threads that each have up to eight
// 16-byte loads outstanding, the quantised kernel by keeping a ring of bulk copies in flight.
#include "launch.h"
#include "qblocks.cuh"
#include "rms_rowreg.cuh"

namespace cb200 {

// Dense rows: a grid-stride walk with the row held in registers.  Rows are exactly VPT vectors per
// thread (the launcher picks threads-per-row so), which keeps the loop free of bounds checks;
// alpha and the position weights stay in registers for the whole walk.  Three 256-thread CTAs per
// SM, each thread with up to eight 16-byte loads outstanding, keep about 100 KB of reads in flight
// per SM, which measurement shows is what saturates HBM on B200 as long as the loop stays lean:
// the rare exact replay is kept out of line for that reason.
template <int DT, int VPT, int BT, bool GATHER>
__global__ void __launch_bounds__(BT, 768 / BT) rms_rowreg_kernel(const RmsRowRegArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tx = threadIdx.x, ty = threadIdx.y, tpr = blockDim.x, rpc = blockDim.y;
  RowRegSmem sm(smem_raw, rpc, tpr, a.V, ty);
  const bool has_res = !GATHER && a.res != nullptr;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * rpc;

  uint4 al[VPT];
  float wv[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    al[k] = __ldg(a.alpha + k * tpr + tx);
    wv[k] = static_cast<float>(a.n - 8 * (k * tpr + tx));
  }

  // gathered rows: the id of the next row is loaded one iteration early, off the critical path
  uint64_t id_next = 0;
  if (GATHER && static_cast<int64_t>(blockIdx.x) * rpc + ty < a.rows)
    id_next = read_id(a.ids, a.id_dtype, static_cast<int64_t>(blockIdx.x) * rpc + ty);

  for (int64_t row = static_cast<int64_t>(blockIdx.x) * rpc + ty; row < a.rows; row += stride) {
    const uint4* xr;
    bool live = true;
    if (GATHER) {
      const uint64_t id = id_next;
      if (row + stride < a.rows) id_next = read_id(a.ids, a.id_dtype, row + stride);
      live = id < static_cast<uint64_t>(a.vocab);
      if (!live && tx == 0) report_status(a.status, CB200_STATUS_INVALID_INDEX, row, static_cast<int64_t>(id), a.vocab);
      xr = a.x + (live ? id : 0) * a.V + tx;
    } else {
      xr = a.x + row * a.V + tx;
    }
    uint4 h[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) h[k] = ldg_stream(xr + k * tpr);
    if (has_res) {
      const uint4* rr = a.res + row * a.V + tx;
      uint4 rv[VPT];
#pragma unroll
      for (int k = 0; k < VPT; ++k) rv[k] = ldg_stream(rr + k * tpr);
#pragma unroll
      for (int k = 0; k < VPT; ++k) h[k] = add_round_vec<DT>(h[k], rv[k]);
    }
    float lsum = 0.0f, lw = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) accumulate_vec_w<DT>(h[k], wv[k], lsum, lw);
    bool replayed;
    const float m = resolve_row_m<DT, VPT>(h, lsum, lw, a.V, a.n, a.eps, a.flags, sm, sm.rows, replayed);
    if (replayed) {  // rare: nothing was kept in registers across the replay
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        al[k] = __ldg(a.alpha + k * tpr + tx);
        wv[k] = static_cast<float>(a.n - 8 * (k * tpr + tx));
      }
    }
    if (live) {
      if (a.sum_out != nullptr) {
        uint4* so = a.sum_out + row * a.V + tx;
#pragma unroll
        for (int k = 0; k < VPT; ++k) stg_stream(so + k * tpr, h[k]);
      }
      // 2^-60 <= m <= 2^60: the reciprocal is a normal number and the margin argument applies
      const bool fast_div = (DT == kDtBF16) && (m >= 8.6736174e-19f) && (m <= 1.1529215e18f);
      const float r = fast_div ? __frcp_rn(m) : 0.0f;
      uint4* yr = a.y + row * a.V + tx;
#pragma unroll
      for (int k = 0; k < VPT; ++k) stg_stream(yr + k * tpr, rms_output_vec<DT>(h[k], al[k], m, r, fast_div));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Quantised source: each CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ... through a ring of
// shared-memory row buffers that thread 0 keeps filled with bulk copies kQStages-1 rows ahead.
// Thread 0 is the only reader of the ids; it loads each id one iteration before it needs it and
// publishes what kind of row a ring slot holds, so no id load sits on anybody's critical path.
// ---------------------------------------------------------------------------------------------
constexpr int kQStages = 8;
constexpr int kRowDecode = 0, kRowMasked = 1, kRowBadId = 2;

template <int QT, int DT, int VPT, int BT>
__global__ void __launch_bounds__(BT, 1024 / BT) qrms_rowreg_kernel(const QRmsArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tx = threadIdx.x, tpr = blockDim.x;
  RowRegSmem sm(smem_raw, 1, tpr, a.V, 0);
  const size_t core_bytes = RowRegSmem::bytes(1, tpr, a.V, true);
  const int stage_bytes = (a.row_bytes + 15) & ~15;
  unsigned char* stage0 = smem_raw + core_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage0 + kQStages * stage_bytes);
  volatile int* kinds = reinterpret_cast<volatile int*>(bars + kQStages);  // [kQStages]
  volatile int* abort_flag = kinds + kQStages;

  const int64_t first = blockIdx.x, step = gridDim.x;
  uint64_t id_ahead = 0;  // thread 0: id of the next row to be issued, already loaded

  // thread 0: classify row (whose id is `id`), publish its kind and start its copy into `stage`
  auto issue = [&](int64_t row, uint64_t id, int stage) {
    int kind = kRowDecode;
    if (id >= static_cast<uint64_t>(a.vocab)) {
      kind = kRowBadId;
      report_status(a.status, CB200_STATUS_INVALID_INDEX, row, static_cast<int64_t>(id), a.vocab);
    } else if (id < static_cast<uint64_t>(a.vocab_begin) || id >= static_cast<uint64_t>(a.vocab_end)) {
      kind = kRowMasked;
    }
    kinds[stage] = kind;
    if (kind == kRowDecode && a.bulk) {
      const unsigned char* src = a.qtable + (id - a.vocab_begin) * static_cast<uint64_t>(a.row_bytes);
      mbar_expect_tx(&bars[stage], static_cast<uint32_t>(a.row_bytes));
      bulk_g2s(stage0 + stage * stage_bytes, src, static_cast<uint32_t>(a.row_bytes), &bars[stage]);
    }
  };

  if (tx == 0) {
    for (int s = 0; s < kQStages; ++s) mbar_init(&bars[s], 1);
    mbar_init_fence();
    *abort_flag = 0;
    for (int j = 0; j < kQStages - 1; ++j) {
      const int64_t r = first + j * step;
      if (r < a.rows) issue(r, read_id(a.ids, a.id_dtype, r), j);
    }
    const int64_t r = first + static_cast<int64_t>(kQStages - 1) * step;
    if (r < a.rows) id_ahead = read_id(a.ids, a.id_dtype, r);
  }
  __syncthreads();

  // Each thread owns VPT/2 half blocks: vectors 2p and 2p+1 for p = j*tpr + tx.  They share one
  // block scale and make 32 contiguous output bytes.
  constexpr int HB = VPT / 2;
  uint4 al[VPT];
  float wv[VPT];
#pragma unroll
  for (int j = 0; j < HB; ++j) {
    const int p = j * tpr + tx;
    al[2 * j] = __ldg(a.alpha + 2 * p);
    al[2 * j + 1] = __ldg(a.alpha + 2 * p + 1);
    wv[2 * j] = static_cast<float>(a.n - 16 * p);
    wv[2 * j + 1] = static_cast<float>(a.n - 16 * p - 8);
  }

  uint32_t phase = 0;  // one parity bit per stage
  int stage = 0;
  for (int64_t row = first; row < a.rows; row += step) {
    unsigned char* buf = stage0 + stage * stage_bytes;
    // The stage used by the previous row is free: its readers finished before that row's first
    // barrier, which thread 0 has passed.  Refill it with the row kQStages-1 ahead, then start
    // loading the id that the next iteration will need.
    if (tx == 0) {
      const int64_t ahead = row + static_cast<int64_t>(kQStages - 1) * step;
      if (ahead < a.rows) {
        issue(ahead, id_ahead, stage == 0 ? kQStages - 1 : stage - 1);
        if (ahead + step < a.rows) id_ahead = read_id(a.ids, a.id_dtype, ahead + step);
      }
    }
    const int kind = kinds[stage];
    if (kind == kRowDecode) {
      if (a.bulk) {
        // A wait that runs out is recorded and acted on after the row's barriers, where the
        // whole CTA sees the flag and can leave together.
        if (!mbar_wait(&bars[stage], (phase >> stage) & 1u)) *abort_flag = 1;
        phase ^= 1u << stage;
      } else {
        // rows that are not 16-byte multiples: cooperative 2-byte copies (ids re-read: slow path)
        const uint64_t id = read_id(a.ids, a.id_dtype, row);
        const uint16_t* src =
            reinterpret_cast<const uint16_t*>(a.qtable + (id - a.vocab_begin) * static_cast<uint64_t>(a.row_bytes));
        uint16_t* dst = reinterpret_cast<uint16_t*>(buf);
        for (int i = tx; i < a.row_bytes / 2; i += tpr) dst[i] = src[i];
        __syncthreads();
      }
    }

    uint4 h[VPT];
    float hf[VPT][8];
    float lsum = 0.0f, lw = 0.0f, dmin = 3.0e38f;
    if (kind == kRowDecode) {
#pragma unroll
      for (int j = 0; j < HB; ++j) {
        float d;
        decode_half_block<QT, DT>(buf, j * tpr + tx, h[2 * j], h[2 * j + 1], d);
        widen_accumulate<DT>(h[2 * j], wv[2 * j], hf[2 * j], lsum, lw);
        widen_accumulate<DT>(h[2 * j + 1], wv[2 * j + 1], hf[2 * j + 1], lsum, lw);
        d = fabsf(d);
        dmin = fminf(dmin, d == 0.0f ? 3.0e38f : d);  // a zero scale makes exact zeros only
      }
    } else {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        h[k] = (kind == kRowMasked) ? neg_zero_vec<DT>() : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < 8; ++i) hf[k][i] = (kind == kRowMasked) ? -0.0f : 0.0f;
      }
    }
    bool replayed;
    float row_dmin;
    const float m = resolve_row_m<DT, VPT>(h, lsum, lw, a.V, a.n, a.eps, a.flags, sm, sm.rows, replayed, dmin, &row_dmin,
                                           /*pair_layout=*/true);
    if (replayed) {  // rare: nothing was kept in registers across the replay
      float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
      for (int j = 0; j < HB; ++j) {
        const int p = j * tpr + tx;
        al[2 * j] = __ldg(a.alpha + 2 * p);
        al[2 * j + 1] = __ldg(a.alpha + 2 * p + 1);
        wv[2 * j] = static_cast<float>(a.n - 16 * p);
        wv[2 * j + 1] = static_cast<float>(a.n - 16 * p - 8);
        widen_accumulate<DT>(h[2 * j], 0.0f, hf[2 * j], s0, s1);
        widen_accumulate<DT>(h[2 * j + 1], 0.0f, hf[2 * j + 1], s0, s1);
      }
    }
    if (*abort_flag) {
      if (tx == 0) {
        report_status(a.status, CB200_STATUS_WAIT_TIMEOUT, row, 0, a.vocab);
        // bounded second chance for every copy still in flight, so that none lands in shared
        // memory after the CTA has retired
        for (int j = 0; j < kQStages - 1; ++j) {
          const int64_t r = row + static_cast<int64_t>(j) * step;
          const int s = (stage + j) % kQStages;
          if (r >= a.rows || kinds[s] != kRowDecode) continue;
          const uint32_t par = (j == 0) ? (((phase >> s) & 1u) ^ 1u) : ((phase >> s) & 1u);
          mbar_wait(&bars[s], par);
        }
      }
      return;
    }
    if (kind != kRowBadId) {
      if (a.gathered != nullptr) {
        uint4* g = a.gathered + row * a.V;
#pragma unroll
        for (int j = 0; j < HB; ++j) {
          const int p = j * tpr + tx;
          stg_stream(g + 2 * p, h[2 * j]);
          stg_stream(g + 2 * p + 1, h[2 * j + 1]);
        }
      }
      const bool fast_div = (DT == kDtBF16) && (m >= 8.6736174e-19f) && (m <= 1.1529215e18f);
      const float r = fast_div ? __frcp_rn(m) : 0.0f;
      uint4* yr = a.y + row * a.V;
      // |h| >= the smallest block scale for every non-zero element: above 2^-40 no product with
      // 1/m (m <= 2^60) can fall under 2^-100, and the guard can go.
      if (row_dmin >= 9.0949470e-13f) {
#pragma unroll
        for (int j = 0; j < HB; ++j) {
          const int p = j * tpr + tx;
          stg_stream(yr + 2 * p, rms_output_floats<DT, false>(hf[2 * j], al[2 * j], m, r, fast_div));
          stg_stream(yr + 2 * p + 1, rms_output_floats<DT, false>(hf[2 * j + 1], al[2 * j + 1], m, r, fast_div));
        }
      } else {
#pragma unroll
        for (int j = 0; j < HB; ++j) {
          const int p = j * tpr + tx;
          stg_stream(yr + 2 * p, rms_output_floats<DT, true>(hf[2 * j], al[2 * j], m, r, fast_div));
          stg_stream(yr + 2 * p + 1, rms_output_floats<DT, true>(hf[2 * j + 1], al[2 * j + 1], m, r, fast_div));
        }
      }
    }
    stage = stage + 1 == kQStages ? 0 : stage + 1;
    // No barrier here: every thread finished decoding `buf` before the row's first barrier and
    // reads the published m before the next row's first barrier, so the refill issued at the
    // top of the next iteration and the next row's scratch writes cannot race with this row.
  }
}

// ---------------------------------------------------------------------------------------------
// Launchers
// ---------------------------------------------------------------------------------------------
// Threads per row and vectors per thread for a row of V vectors: V == tpr * vpt exactly, tpr a
// multiple of 32 up to 512, preferring four vectors per thread.  Returns false if V has no such split.
static bool rowreg_shape(int V, int& tpr, int& vpt, int& rpc) {
  static const int prefs[] = {4, 3, 5, 2, 6, 7, 8, 1};
  for (int cand : prefs) {
    if (V % cand != 0) continue;
    const int t = V / cand;
    if (t % 32 != 0 || t > 512) continue;
    tpr = t;
    vpt = cand;
    rpc = tpr >= 128 ? 1 : 128 / tpr;
    return true;
  }
  return false;
}

// Shape of the quantised-source kernel: one row per CTA, V == tpr * vpt exactly, preferring two
// vectors per thread (the decoder needs the registers).
static bool qrowreg_shape(int V, int& tpr, int& vpt) {
  static const int prefs[] = {2, 4, 6, 8};  // whole half blocks (vector pairs) per thread
  for (int cand : prefs) {
    if (V % cand != 0) continue;
    const int t = V / cand;
    if (t % 32 != 0 || t < 64 || t > 512) continue;
    tpr = t;
    vpt = cand;
    return true;
  }
  return false;
}

bool rms_rowreg_supported(int dtype, int cols) {
  int tpr, vpt, rpc;
  return (dtype == kDtBF16 || dtype == kDtF16) && cols % 8 == 0 && cols >= 256 && cols <= 32768 &&
         rowreg_shape(cols / 8, tpr, vpt, rpc);
}

bool qrms_rowreg_supported(int dtype, int cols) {
  int tpr, vpt;
  return (dtype == kDtBF16 || dtype == kDtF16) && cols % 32 == 0 && cols <= 32768 && qrowreg_shape(cols / 8, tpr, vpt);
}

// A persistent grid: as many CTAs as are resident at once, but no more than there is work.
// `ctas_wanted` CTAs per SM should fit: the shared-memory carve-out is set to just what they need,
// because every byte given to shared memory is taken from L1, and L1 is where the data of loads
// in flight lands -- a maximal carve-out caps an SM at a fraction of the ~100 KB of outstanding
// reads that saturating HBM takes.
template <typename K>
static cudaError_t persistent_grid(K kern, int threads, size_t smem, int ctas_wanted, int64_t work_items,
                                   unsigned& grid) {
  const size_t per_cta = smem + 1024;  // the driver reserves 1 KB per CTA
  int percent = static_cast<int>((per_cta * ctas_wanted * 100 + 228 * 1024 - 1) / (228 * 1024));
  if (percent > 100) percent = 100;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, percent);
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

template <int DT, int VPT, int BT, bool GATHER>
static cudaError_t launch_dense_t(const RmsRowRegArgs& a, int tpr, int rpc, cudaStream_t stream) {
  const bool with_rows = !(a.flags & CB200_FLAG_FAST_SUM);
  const size_t smem = RowRegSmem::bytes(rpc, tpr, a.V, with_rows);
  auto kern = rms_rowreg_kernel<DT, VPT, BT, GATHER>;
  unsigned grid = 1;
  cudaError_t e = persistent_grid(kern, tpr * rpc, smem, 768 / BT, (a.rows + rpc - 1) / rpc, grid);
  if (e != cudaSuccess) return e;
  kern<<<grid, dim3(tpr, rpc), smem, stream>>>(a);
  return cudaGetLastError();
}

template <int DT, int VPT>
static cudaError_t launch_dense_bt(const RmsRowRegArgs& a, int tpr, int rpc, cudaStream_t stream) {
  const bool gather = a.ids != nullptr;
  if (tpr * rpc <= 256)
    return gather ? launch_dense_t<DT, VPT, 256, true>(a, tpr, rpc, stream)
                  : launch_dense_t<DT, VPT, 256, false>(a, tpr, rpc, stream);
  return gather ? launch_dense_t<DT, VPT, 512, true>(a, tpr, rpc, stream)
                : launch_dense_t<DT, VPT, 512, false>(a, tpr, rpc, stream);
}

template <int DT>
static cudaError_t launch_dense_dt(const RmsRowRegArgs& a, cudaStream_t stream) {
  int tpr = 0, vpt = 0, rpc = 0;
  if (!rowreg_shape(a.V, tpr, vpt, rpc)) return cudaErrorInvalidValue;
  switch (vpt) {
    case 1:
      return launch_dense_bt<DT, 1>(a, tpr, rpc, stream);
    case 2:
      return launch_dense_bt<DT, 2>(a, tpr, rpc, stream);
    case 3:
      return launch_dense_bt<DT, 3>(a, tpr, rpc, stream);
    case 4:
      return launch_dense_bt<DT, 4>(a, tpr, rpc, stream);
    case 5:
      return launch_dense_bt<DT, 5>(a, tpr, rpc, stream);
    case 6:
      return launch_dense_bt<DT, 6>(a, tpr, rpc, stream);
    case 7:
      return launch_dense_bt<DT, 7>(a, tpr, rpc, stream);
    default:
      return launch_dense_bt<DT, 8>(a, tpr, rpc, stream);
  }
}

cudaError_t launch_rms_rowreg(int dtype, const RmsRowRegArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  return dtype == kDtBF16 ? launch_dense_dt<kDtBF16>(a, stream) : launch_dense_dt<kDtF16>(a, stream);
}

template <int QT, int DT, int VPT, int BT>
static cudaError_t launch_q_t(const QRmsArgs& a, int tpr, cudaStream_t stream) {
  const int stage_bytes = (a.row_bytes + 15) & ~15;
  const size_t smem = RowRegSmem::bytes(1, tpr, a.V, true) + static_cast<size_t>(kQStages) * stage_bytes +
                      kQStages * 8 + (kQStages + 1) * 4 + 4;
  auto kern = qrms_rowreg_kernel<QT, DT, VPT, BT>;
  unsigned grid = 1;
  cudaError_t e = persistent_grid(kern, tpr, smem, 1024 / BT, a.rows, grid);
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
  int tpr = 0, vpt = 0;
  if (!qrowreg_shape(a.V, tpr, vpt)) return cudaErrorInvalidValue;
  switch (vpt) {
    case 2:
      return launch_q_bt<QT, DT, 2>(a, tpr, stream);
    case 4:
      return launch_q_bt<QT, DT, 4>(a, tpr, stream);
    case 6:
      return launch_q_bt<QT, DT, 6>(a, tpr, stream);
    default:
      return launch_q_bt<QT, DT, 8>(a, tpr, stream);
  }
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
