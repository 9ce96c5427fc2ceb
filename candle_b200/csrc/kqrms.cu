// Lookup + RMS norm in one launch for tables in the K-quant super-block formats (Q2K ... Q8K,
// candle-core/src/quantized/k_quants.rs:698-1883) and in the 32-element formats the row-slot kernel
// has no decoder for (Q4_1, Q5_0, Q5_1, k_quants.rs:50-84): what candle computes as
//   dequantize(table) -> to_dtype(T) -> embedding(ids) -> rms_norm(alpha, eps)
// (candle-transformers/src/models/quantized_llama.rs:378-379, candle-nn/src/ops.rs:447-508).
//
// The row-register scheme of the dense RMS norm with a decoder in front: a CTA is `rpc` row slots of
// `tpr` threads; the slot's first thread bulk-copies the quantised row of the NEXT token into one of two
// staging buffers while the slot works on this one; every thread decodes its VPT 16-byte vectors (vector
// k * tpr + tx -- tpr is a multiple of 32, so a thread's position inside a super-block is the same for
// every row) into registers, and from there the row is an ordinary row of T: tree sums, interval
// decision, exact replay from the parked row where needed, guarded output.
#include "launch.h"
#include "qblocks.cuh"
#include "rms_rowreg.cuh"

namespace cb200 {

namespace {

constexpr int kRowDecode = 0, kRowMasked = 1, kRowBadId = 2;

// Per row slot, after the RowRegSmem area of the CTA: a ring of staging buffers, their barriers, the
// kinds of the rows they hold and the slot's abort flag.
constexpr int kKqStages = 3;
struct KqStage {
  unsigned char* buf;
  uint64_t* bars;
  volatile int* kinds;
  volatile int* abort_flag;
  __device__ KqStage(unsigned char* base, int stage_bytes) {
    buf = base;
    bars = reinterpret_cast<uint64_t*>(base + kKqStages * static_cast<size_t>(stage_bytes));
    kinds = reinterpret_cast<volatile int*>(bars + kKqStages);
    abort_flag = kinds + kKqStages;
  }
  __host__ __device__ static size_t bytes(int stage_bytes) {
    return (kKqStages * static_cast<size_t>(stage_bytes) + kKqStages * 8 + (kKqStages + 1) * 4 + 15) & ~static_cast<size_t>(15);
  }
};

template <int QT, int DT, int VPT>
__global__ void __launch_bounds__(256, 4) kq_rowreg_kernel(const QRmsArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tx = threadIdx.x, ty = threadIdx.y, tpr = blockDim.x, rpc = blockDim.y;
  RowRegSmem sm(smem_raw, rpc, tpr, a.V, ty);
  const int stage_bytes = (a.row_bytes + 15) & ~15;
  KqStage st(smem_raw + RowRegSmem::bytes(rpc, tpr, a.V, true) + ty * KqStage::bytes(stage_bytes), stage_bytes);
  const int bar_id = 1 + ty;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * rpc;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * rpc + ty;

  // (alpha is re-read through L1 for every row: keeping it in registers would cost the fourth CTA per SM)
  float wv[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) wv[k] = static_cast<float>(a.n - 8 * (k * tpr + tx));

  // issuing thread: classify `row`, publish its kind, start its copy into stage `s`
  auto issue = [&](int64_t row, int s) {
    const uint64_t id = read_id(a.ids, a.id_dtype, row);
    int kind = kRowDecode;
    if (id >= static_cast<uint64_t>(a.vocab)) {
      kind = kRowBadId;
      report_status(a.status, CB200_STATUS_INVALID_INDEX, row, static_cast<int64_t>(id), a.vocab);
    } else if (id < static_cast<uint64_t>(a.vocab_begin) || id >= static_cast<uint64_t>(a.vocab_end)) {
      kind = kRowMasked;
    }
    st.kinds[s] = kind;
    if (kind == kRowDecode) {
      const unsigned char* src = a.qtable + (id - a.vocab_begin) * static_cast<uint64_t>(a.row_bytes);
      mbar_expect_tx(&st.bars[s], static_cast<uint32_t>(a.row_bytes) + a.wt.extra_tx);
      bulk_g2s(st.buf + static_cast<size_t>(s) * stage_bytes, src, static_cast<uint32_t>(a.row_bytes), &st.bars[s]);
    }
  };
  auto slot_sync = [&]() {
    if (tpr > 32)
      row_barrier(bar_id, tpr);
    else
      __syncwarp();
  };

  if (tx == 0) {
    for (int s = 0; s < kKqStages; ++s) mbar_init(&st.bars[s], 1);
    mbar_init_fence();
    *st.abort_flag = 0;
    for (int j = 0; j < kKqStages - 1; ++j)
      if (first + j * stride < a.rows) issue(first + j * stride, j);
  }
  slot_sync();

  uint32_t phase = 0;  // one parity bit per stage
  int stage = 0;
  for (int64_t row = first; row < a.rows; row += stride, stage = stage + 1 == kKqStages ? 0 : stage + 1) {
    // The buffer of the previous row is free: its readers are past their decode, which precedes the
    // slot-wide synchronisation every row ends with.  Refill it with the row kKqStages - 1 ahead.
    if (tx == 0) {
      const int64_t ahead = row + static_cast<int64_t>(kKqStages - 1) * stride;
      if (ahead < a.rows) issue(ahead, stage == 0 ? kKqStages - 1 : stage - 1);
    }
    const int kind = st.kinds[stage];
    const unsigned char* buf = st.buf + static_cast<size_t>(stage) * stage_bytes;
    bool wait_ok = true;
    if (kind == kRowDecode) {
      wait_ok = mbar_wait(&st.bars[stage], (phase >> stage) & 1u, a.wt.spins);
      if (wait_ok)
        phase ^= 1u << stage;
      else
        *st.abort_flag = 1;  // acted on after the row's synchronisation points, where the slot can leave together
    }
    uint4 h[VPT];
    if (kind == kRowDecode) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        float f[8];
        decode8<QT, true>(buf, k * tpr + tx, f);  // the staged row starts on a 16-byte boundary
        h[k] = make_uint4(pack2<DT>(f[0], f[1]), pack2<DT>(f[2], f[3]), pack2<DT>(f[4], f[5]), pack2<DT>(f[6], f[7]));
      }
    } else {
#pragma unroll
      for (int k = 0; k < VPT; ++k) h[k] = masked_row_vec();  // masked row or bad id
    }
    float lsum = 0.0f, lw = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) accumulate_vec_w<DT>(h[k], wv[k], lsum, lw);
    bool replayed;
    const float m = resolve_row_m<DT, VPT>(h, lsum, lw, a.V, a.n, a.eps, a.flags, sm, sm.rows, replayed);
    // (slots wider than a warp passed two named barriers inside resolve_row_m: every thread is past its
    // decode and sees the abort flag)
    if (tpr == 32) __syncwarp();
    if (*st.abort_flag) {
      if (tx == 0) {
        report_status(a.status, CB200_STATUS_WAIT_TIMEOUT, row, 0, a.vocab);
        // bounded second chance for the copies still in flight before the slot retires
        for (int j = 0; j < kKqStages; ++j) {
          const int64_t rj = row + static_cast<int64_t>((j - stage + kKqStages) % kKqStages) * stride;
          if (rj < a.rows && st.kinds[j] == kRowDecode && !(j == stage && wait_ok))
            mbar_wait(&st.bars[j], (phase >> j) & 1u, a.wt.spins);
        }
        drain_pause();
      }
      return;
    }
    if (replayed) {  // nothing was kept in registers across the out-of-line replay
#pragma unroll
      for (int k = 0; k < VPT; ++k) wv[k] = static_cast<float>(a.n - 8 * (k * tpr + tx));
    }
    if (kind != kRowBadId) {
      if (a.gathered != nullptr) {
        uint4* g = a.gathered + row * a.V + tx;
#pragma unroll
        for (int k = 0; k < VPT; ++k) stg_stream(g + k * tpr, h[k]);
      }
      // 2^-60 <= m <= 2^60: the reciprocal is a normal number and the margin argument applies
      const bool fast_div = (m >= 8.6736174e-19f) && (m <= 1.1529215e18f);
      const float r = fast_div ? __frcp_rn(m) : 0.0f;
      uint4* yr = a.y + row * a.V + tx;
#pragma unroll
      for (int k = 0; k < VPT; ++k)
        stg_stream(yr + k * tpr, rms_output_vec<DT>(h[k], __ldg(a.alpha + k * tpr + tx), m, r, fast_div));
    }
  }
}

// tpr * vpt == V exactly, tpr a multiple of 32 up to 256 (a whole row per slot of one CTA of 256 threads)
bool kq_shape(int V, int& tpr, int& vpt, int& rpc) {
  static const int prefs[] = {4, 2, 8, 1};
  for (int cand : prefs) {
    if (V % cand != 0) continue;
    const int t = V / cand;
    if (t % 32 != 0 || t > 256) continue;
    tpr = t;
    vpt = cand;
    rpc = 256 / tpr;
    return true;
  }
  return false;
}

template <int QT, int DT, int VPT>
cudaError_t launch_kq_t(const QRmsArgs& a_in, int tpr, int rpc, cudaStream_t stream) {
  QRmsArgs a = a_in;
  a.wt = wait_tuning();
  const int stage_bytes = (a.row_bytes + 15) & ~15;
  const size_t smem = RowRegSmem::bytes(rpc, tpr, a.V, true) + static_cast<size_t>(rpc) * KqStage::bytes(stage_bytes);
  if (smem > 56 * 1024) return cudaErrorInvalidValue;  // four CTAs per SM
  auto kern = kq_rowreg_kernel<QT, DT, VPT>;
  int per_sm = 1, sms = 1;
  cudaError_t e = kernel_launch_config(reinterpret_cast<const void*>(kern), 256, smem,
                                       static_cast<int>(((smem + 1024) * 4 * 100 + 228 * 1024 - 1) / (228 * 1024)), &per_sm);
  if (e != cudaSuccess) return e;
  e = device_sm_count(&sms);
  if (e != cudaSuccess) return e;
  int64_t grid = static_cast<int64_t>(sms) * per_sm;
  const int64_t work = (a.rows + rpc - 1) / rpc;
  if (grid > work) grid = work;
  kern<<<static_cast<unsigned>(grid), dim3(tpr, rpc), smem, stream>>>(a);
  return cudaGetLastError();
}

template <int QT, int DT>
cudaError_t launch_kq_dt(const QRmsArgs& a, cudaStream_t stream) {
  int tpr = 0, vpt = 0, rpc = 0;
  if (!kq_shape(a.V, tpr, vpt, rpc)) return cudaErrorInvalidValue;
  switch (vpt) {
    case 1:
      return launch_kq_t<QT, DT, 1>(a, tpr, rpc, stream);
    case 2:
      return launch_kq_t<QT, DT, 2>(a, tpr, rpc, stream);
    case 4:
      return launch_kq_t<QT, DT, 4>(a, tpr, rpc, stream);
    default:
      return launch_kq_t<QT, DT, 8>(a, tpr, rpc, stream);
  }
}

template <int QT>
cudaError_t launch_kq(int dtype, const QRmsArgs& a, cudaStream_t stream) {
  return dtype == kDtBF16 ? launch_kq_dt<QT, kDtBF16>(a, stream) : launch_kq_dt<QT, kDtF16>(a, stream);
}

}  // namespace

// Row lengths the kernel takes: 16-bit output, a whole number of blocks, V = tpr * vpt with the
// split above, the staged rows and the parked row within the shared memory of a quarter of an SM.
bool kqrms_supported(int qtype, int dtype, int cols) {
  int tpr, vpt, rpc;
  const bool takes = is_kquant(qtype) || qtype == CB200_QTYPE_Q4_1 || qtype == CB200_QTYPE_Q5_0 || qtype == CB200_QTYPE_Q5_1;
  if (!takes || (dtype != kDtBF16 && dtype != kDtF16) || cols <= 0 || cols % qblock_elems(qtype) != 0) return false;
  if (!kq_shape(cols / 8, tpr, vpt, rpc)) return false;
  const int row_bytes = cols / qblock_elems(qtype) * qblock_bytes(qtype);
  if (row_bytes % 16 != 0) return false;
  return RowRegSmem::bytes(rpc, tpr, cols / 8, true) + static_cast<size_t>(rpc) * KqStage::bytes(row_bytes) <= 56 * 1024;
}

cudaError_t launch_kqrms(int qtype, int dtype, const QRmsArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  switch (qtype) {
    case CB200_QTYPE_Q2K:
      return launch_kq<CB200_QTYPE_Q2K>(dtype, a, stream);
    case CB200_QTYPE_Q3K:
      return launch_kq<CB200_QTYPE_Q3K>(dtype, a, stream);
    case CB200_QTYPE_Q4K:
      return launch_kq<CB200_QTYPE_Q4K>(dtype, a, stream);
    case CB200_QTYPE_Q5K:
      return launch_kq<CB200_QTYPE_Q5K>(dtype, a, stream);
    case CB200_QTYPE_Q6K:
      return launch_kq<CB200_QTYPE_Q6K>(dtype, a, stream);
    case CB200_QTYPE_Q8K:
      return launch_kq<CB200_QTYPE_Q8K>(dtype, a, stream);
    case CB200_QTYPE_Q4_1:
      return launch_kq<CB200_QTYPE_Q4_1>(dtype, a, stream);
    case CB200_QTYPE_Q5_0:
      return launch_kq<CB200_QTYPE_Q5_0>(dtype, a, stream);
    case CB200_QTYPE_Q5_1:
      return launch_kq<CB200_QTYPE_Q5_1>(dtype, a, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace cb200
