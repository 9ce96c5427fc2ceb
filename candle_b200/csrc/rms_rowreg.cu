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
// Look-ahead (kModeAhead): the next row is loaded into a second set of registers before the
// current one is worked on, so that an SM's loads never pause for the per-row reduction and
// decision.  Without a residual a row brings only half the bytes and this is what keeps enough of
// them in flight; with a residual (kModeAheadRes) x and the residual of the next row are both held,
// and the registers for that come from not keeping alpha resident (it is re-read through L1).
// kModeGather: rows come from a table by id.  The launcher enables look-ahead only for the
// vectors-per-thread counts whose register need fits.
constexpr int kModeGather = 1, kModeAhead = 2, kModeAheadRes = 4;

template <int DT, int VPT, int BT, int MODE>
__global__ void __launch_bounds__(BT, 768 / BT) rms_rowreg_kernel(const RmsRowRegArgs a) {
  constexpr bool GATHER = (MODE & kModeGather) != 0;
  constexpr bool AHEAD_RES = (MODE & kModeAheadRes) != 0;
  constexpr bool AHEAD = (MODE & kModeAhead) != 0 || AHEAD_RES;
  constexpr bool ALPHA_REGS = !AHEAD_RES;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tx = threadIdx.x, ty = threadIdx.y, tpr = blockDim.x, rpc = blockDim.y;
  RowRegSmem sm(smem_raw, rpc, tpr, a.V, ty);
  const bool has_res = !GATHER && !AHEAD && a.res != nullptr;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * rpc;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * rpc + ty;

  uint4 al[ALPHA_REGS ? VPT : 1];
  float wv[ALPHA_REGS ? VPT : 1];
  if (ALPHA_REGS) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      al[k] = __ldg(a.alpha + k * tpr + tx);
      wv[k] = static_cast<float>(a.n - 8 * (k * tpr + tx));
    }
  }

  // The row one step ahead (AHEAD) and, for gathered rows, its id and the id two steps ahead:
  // ids are loaded a whole iteration before the address they make is needed.
  uint4 nx[AHEAD ? VPT : 1], nr[AHEAD_RES ? VPT : 1];
  uint64_t id_ahead = 0, id_ahead2 = 0;
  if (GATHER && !AHEAD && first < a.rows) id_ahead = read_id(a.ids, a.id_dtype, first);
  if (AHEAD && first < a.rows) {
    if (GATHER) {
      id_ahead = read_id(a.ids, a.id_dtype, first);
      if (first + stride < a.rows) id_ahead2 = read_id(a.ids, a.id_dtype, first + stride);
    }
    const uint4* xr = a.x + (GATHER ? (id_ahead < static_cast<uint64_t>(a.vocab) ? id_ahead : 0) : first) * a.V + tx;
#pragma unroll
    for (int k = 0; k < VPT; ++k) nx[k] = ldg_stream(xr + k * tpr);
    if (AHEAD_RES) {
      const uint4* rr = a.res + first * a.V + tx;
#pragma unroll
      for (int k = 0; k < VPT; ++k) nr[k] = ldg_stream(rr + k * tpr);
    }
  }

  for (int64_t row = first; row < a.rows; row += stride) {
    bool live = true;
    uint4 h[VPT];
    if (AHEAD) {
      const uint64_t id = id_ahead;
      if (GATHER) {
        live = id < static_cast<uint64_t>(a.vocab);
        if (!live && tx == 0) report_status(a.status, CB200_STATUS_INVALID_INDEX, row, static_cast<int64_t>(id), a.vocab);
      }
#pragma unroll
      for (int k = 0; k < VPT; ++k) h[k] = AHEAD_RES ? add_round_vec<DT>(nx[k], nr[k]) : nx[k];
      if (row + stride < a.rows) {
        if (GATHER) {
          id_ahead = id_ahead2;
          if (row + 2 * stride < a.rows) id_ahead2 = read_id(a.ids, a.id_dtype, row + 2 * stride);
        }
        const uint4* xn =
            a.x + (GATHER ? (id_ahead < static_cast<uint64_t>(a.vocab) ? id_ahead : 0) : row + stride) * a.V + tx;
#pragma unroll
        for (int k = 0; k < VPT; ++k) nx[k] = ldg_stream(xn + k * tpr);
        if (AHEAD_RES) {
          const uint4* rn = a.res + (row + stride) * a.V + tx;
#pragma unroll
          for (int k = 0; k < VPT; ++k) nr[k] = ldg_stream(rn + k * tpr);
        }
      }
    } else {
      const uint4* xr;
      if (GATHER) {  // the id of the next row is loaded one iteration early, off the critical path
        const uint64_t id = id_ahead;
        if (row + stride < a.rows) id_ahead = read_id(a.ids, a.id_dtype, row + stride);
        live = id < static_cast<uint64_t>(a.vocab);
        if (!live && tx == 0) report_status(a.status, CB200_STATUS_INVALID_INDEX, row, static_cast<int64_t>(id), a.vocab);
        xr = a.x + (live ? id : 0) * a.V + tx;
      } else {
        xr = a.x + row * a.V + tx;
      }
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
    }
    float lsum = 0.0f, lw = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
      accumulate_vec_w<DT>(h[k], ALPHA_REGS ? wv[k] : static_cast<float>(a.n - 8 * (k * tpr + tx)), lsum, lw);
    bool replayed;
    const float m = resolve_row_m<DT, VPT>(h, lsum, lw, a.V, a.n, a.eps, a.flags, sm, sm.rows, replayed);
    if (replayed) {  // rare: nothing was kept in registers across the replay
      if (ALPHA_REGS) {
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          al[k] = __ldg(a.alpha + k * tpr + tx);
          wv[k] = static_cast<float>(a.n - 8 * (k * tpr + tx));
        }
      }
      if (AHEAD && row + stride < a.rows) {
        const uint4* xn =
            a.x + (GATHER ? (id_ahead < static_cast<uint64_t>(a.vocab) ? id_ahead : 0) : row + stride) * a.V + tx;
#pragma unroll
        for (int k = 0; k < VPT; ++k) nx[k] = ldg_stream(xn + k * tpr);
        if (AHEAD_RES) {
          const uint4* rn = a.res + (row + stride) * a.V + tx;
#pragma unroll
          for (int k = 0; k < VPT; ++k) nr[k] = ldg_stream(rn + k * tpr);
        }
      }
    }
    if (live) {
      if (a.sum_out != nullptr) {
        uint4* so = a.sum_out + row * a.V + tx;
#pragma unroll
        for (int k = 0; k < VPT; ++k) stg_stream(so + k * tpr, h[k]);
      }
      // 2^-60 <= m <= 2^60: the reciprocal is a normal number and the margin argument applies
      const bool fast_div = (m >= 8.6736174e-19f) && (m <= 1.1529215e18f);
      const float r = fast_div ? __frcp_rn(m) : 0.0f;
      uint4* yr = a.y + row * a.V + tx;
#pragma unroll
      for (int k = 0; k < VPT; ++k)
        stg_stream(yr + k * tpr,
                   rms_output_vec<DT>(h[k], ALPHA_REGS ? al[k] : __ldg(a.alpha + k * tpr + tx), m, r, fast_div));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Quantised source.  A CTA is a set of independent row slots (threadIdx.y), each served by a
// warp (two for rows beyond 4096 columns): a slot walks its own rows, owns a small ring of
// shared-memory row buffers that its first lane keeps filled with bulk copies, and synchronises
// with nobody else -- per row there is one decode, one set of warp shuffles, no CTA barrier.
// The slot's first lane is the only reader of the ids: it loads each id one iteration before it
// needs it and publishes what kind of row a ring slot holds.  A replay decodes the staged blocks
// again in contiguous chunks instead of parking h.
// ---------------------------------------------------------------------------------------------
constexpr int kRowDecode = 0, kRowMasked = 1, kRowBadId = 2;

// decode_half_block out of line, for the rare re-decode after a replay: one copy of the code.
struct HalfBlockVecs {
  uint4 lo, hi;
};
template <int QT, int DT>
__device__ __noinline__ HalfBlockVecs decode_half_block_cold(const unsigned char* row, int p) {
  HalfBlockVecs r;
  float d;
  decode_half_block<QT, DT>(row, p, r.lo, r.hi, d);
  return r;
}

template <int QT, int DT>
struct QuantRow {
  const unsigned char* buf;
  __device__ __forceinline__ uint4 vec(int v) const { return decode_vec8<QT, DT>(buf, v); }
};

// Per-slot shared-memory layout; `stages` buffers of `stage_bytes` first (16-byte aligned).
struct QSlot {
  unsigned char* ring;
  unsigned char* head;  // RowRegSmem area
  uint64_t* bars;
  volatile int* kinds;       // [stages]
  volatile int* abort_flag;  // a bounded wait of this slot ran out
  __device__ QSlot(unsigned char* base, int stages, int stage_bytes, int tpr) {
    ring = base;
    head = base + static_cast<size_t>(stages) * stage_bytes;
    bars = reinterpret_cast<uint64_t*>(head + RowRegSmem::slot_bytes(tpr));
    kinds = reinterpret_cast<volatile int*>(bars + stages);
    abort_flag = kinds + stages;
  }
  __host__ __device__ static size_t bytes(int stages, int stage_bytes, int tpr) {
    size_t b = static_cast<size_t>(stages) * stage_bytes + RowRegSmem::slot_bytes(tpr) + stages * 8 + (stages + 1) * 4;
    return (b + 15) & ~static_cast<size_t>(15);
  }
};

constexpr int kOwnerNone = 0, kOwnerToAll = 1, kOwnerToRowOwner = 2;


template <int QT, int DT, int HB, int OWNER>
__global__ void __launch_bounds__(128, 4) qrms_rowslot_kernel(const QRmsArgs a, int stages) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tx = threadIdx.x, ty = threadIdx.y, tpr = blockDim.x, rpc = blockDim.y;
  const int stage_bytes = (a.row_bytes + 15) & ~15;
  QSlot slot(smem_raw + ty * QSlot::bytes(stages, stage_bytes, tpr), stages, stage_bytes, tpr);
  RowRegSmem sm(slot.head, 1, tpr, a.V, 0);
  const int bar_id = 1 + ty;

  const int64_t first = static_cast<int64_t>(blockIdx.x) * rpc + ty;
  const int64_t step = static_cast<int64_t>(gridDim.x) * rpc;
  uint64_t id_ahead = 0;  // issuing lane: id of the next row to be issued, already loaded

  // row-invariant: this thread's alpha vectors and the position weights n - 16 p of its half blocks
  // (with eight half blocks per thread alpha does not fit and is re-read through L1)
  // Half block j of this thread: interleaved over the slot's threads, so that a warp's 16-byte stores
  // are contiguous.  (Giving each thread HB consecutive half blocks makes the 32-bit block loads
  // conflict-free -- lanes 17 words apart -- but spreads a lane's stores 128 bytes apart: measured
  // 252 us against 215 us on the Q8_0 lookup of 65536 rows of 4096 columns.)
  auto half_block = [&](int j) -> int { return j * tpr + tx; };
  constexpr bool ALPHA_REGS = HB <= 4;
  uint4 al[ALPHA_REGS ? 2 * HB : 1];
  float wj[HB];
#pragma unroll
  for (int j = 0; j < HB; ++j) {
    const int p = half_block(j);
    if (ALPHA_REGS) {
      al[2 * j] = __ldg(a.alpha + 2 * p);
      al[2 * j + 1] = __ldg(a.alpha + 2 * p + 1);
    }
    wj[j] = static_cast<float>(a.n - 16 * p);
  }
  auto alpha_vec = [&](int k) -> uint4 { return ALPHA_REGS ? al[ALPHA_REGS ? k : 0] : __ldg(a.alpha + 2 * half_block(k >> 1) + (k & 1)); };

  // without an id list the rows are taken in order (a dense source)
  auto row_id = [&](int64_t r) -> uint64_t {
    return a.ids != nullptr ? read_id(a.ids, a.id_dtype, r) : static_cast<uint64_t>(r);
  };
  // issuing lane: classify row (whose id is `id`), publish its kind, start its copy into `stage`
  auto issue = [&](int64_t row, uint64_t id, int stage) {
    int kind = kRowDecode;
    if (id >= static_cast<uint64_t>(a.vocab)) {
      kind = kRowBadId;
      report_status(a.status, CB200_STATUS_INVALID_INDEX, row, static_cast<int64_t>(id), a.vocab);
    } else if (id < static_cast<uint64_t>(a.vocab_begin) || id >= static_cast<uint64_t>(a.vocab_end)) {
      kind = kRowMasked;
    }
    slot.kinds[stage] = kind;
    if (kind == kRowDecode) {
      const unsigned char* src = a.qtable + (id - a.vocab_begin) * static_cast<uint64_t>(a.row_bytes);
      mbar_expect_tx(&slot.bars[stage], static_cast<uint32_t>(a.row_bytes) + a.wt.extra_tx);
      bulk_g2s(slot.ring + stage * stage_bytes, src, static_cast<uint32_t>(a.row_bytes), &slot.bars[stage]);
    }
  };

  if (tx == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&slot.bars[s], 1);
    mbar_init_fence();
    *slot.abort_flag = 0;
    for (int j = 0; j < stages - 1; ++j) {
      const int64_t r = first + j * step;
      if (r < a.rows) issue(r, row_id(r), j);
    }
    const int64_t r = first + static_cast<int64_t>(stages - 1) * step;
    if (r < a.rows) id_ahead = row_id(r);
  }
  if (tpr > 32)
    row_barrier(bar_id, tpr);
  else
    __syncwarp();

  uint32_t phase = 0;  // one parity bit per stage
  int stage = 0;
  for (int64_t row = first; row < a.rows; row += step) {
    unsigned char* buf = slot.ring + stage * stage_bytes;
    // The buffer of the previous row is free (its readers are past that row's last use of it,
    // which precedes the slot-wide synchronisation every row ends with).  Refill it with the row
    // stages-1 ahead, then start loading the id the next iteration will need.
    if (tx == 0) {
      const int64_t ahead = row + static_cast<int64_t>(stages - 1) * step;
      if (ahead < a.rows) {
        issue(ahead, id_ahead, stage == 0 ? stages - 1 : stage - 1);
        if (ahead + step < a.rows) id_ahead = row_id(ahead + step);
      }
    }
    const int kind = slot.kinds[stage];
    if (OWNER != kOwnerNone && kind == kRowMasked) {  // another rank owns this row and writes it
      if (tpr > 32)
        row_barrier(bar_id, tpr);
      else
        __syncwarp();
      stage = stage + 1 == stages ? 0 : stage + 1;
      continue;
    }
    bool wait_ok = true;
    if (kind == kRowDecode) {
      // a wait that runs out is recorded and acted on after the row's synchronisation points,
      // where the whole slot sees the flag and can leave together; the stage's parity bit moves on
      // only when its phase really completed
      wait_ok = mbar_wait(&slot.bars[stage], (phase >> stage) & 1u, a.wt.spins);
      if (wait_ok)
        phase ^= 1u << stage;
      else
        *slot.abort_flag = 1;
    }

    // Each thread owns HB half blocks: vectors 2p and 2p+1 for p = j*tpr + tx share one scale
    // and make 32 contiguous output bytes.
    uint4 h[2 * HB];
    float lsum = 0.0f, lw = 0.0f, dmin = 3.0e38f;
    if (kind == kRowDecode) {
#pragma unroll
      for (int j = 0; j < HB; ++j) {
        const int p = half_block(j);
        float d;
        decode_half_block<QT, DT>(buf, p, h[2 * j], h[2 * j + 1], d);
        accumulate_vec_w<DT>(h[2 * j], wj[j], lsum, lw);
        accumulate_vec_w<DT>(h[2 * j + 1], wj[j] - 8.0f, lsum, lw);
        d = fabsf(d);
        dmin = fminf(dmin, d == 0.0f ? 3.0e38f : d);  // a zero scale makes exact zeros only
      }
    } else {
#pragma unroll
      for (int k = 0; k < 2 * HB; ++k) h[k] = masked_row_vec();  // masked row or bad id
    }
    bool need;
    float row_dmin;
    // (the slot's warps meet again at the end of the row, before sm.red is written for the next one)
    float m = decide_row<DT, true>(lsum, lw, a.n, a.eps, a.flags, sm, need, dmin, &row_dmin);
    if (need && kind == kRowDecode) {
      // The replay reuses sm.red, which the slot's other warps may still be reading for their own
      // copy of the decision: they all reach the same verdict, so they can all meet here first.
      if (tpr > 32) row_barrier(bar_id, tpr);
      m = replay_row<DT, QuantRow<QT, DT>>(QuantRow<QT, DT>{buf}, a.V, a.n, a.eps, sm);
#pragma unroll
      for (int j = 0; j < HB; ++j) {  // nothing was kept in registers across the replay
        const HalfBlockVecs hb = decode_half_block_cold<QT, DT>(buf, half_block(j));
        h[2 * j] = hb.lo;
        h[2 * j + 1] = hb.hi;
      }
    }
    if (tpr == 32) __syncwarp();  // (wider slots passed named barriers inside decide_row)
    if (*slot.abort_flag) {
      if (tx == 0) {
        report_status(a.status, CB200_STATUS_WAIT_TIMEOUT, row, 0, a.vocab);
        // Bounded second chance for the copies still in flight: every stage that holds a row to be
        // decoded has one, except this row's own stage if this thread saw it complete.
        for (int j = 0; j < stages; ++j)
          if (slot.kinds[j] == kRowDecode && !(j == stage && wait_ok && kind == kRowDecode))
            mbar_wait(&slot.bars[j], (phase >> j) & 1u, a.wt.spins);
        drain_pause();
      }
      return;
    }
    if (kind != kRowBadId) {
      if (a.gathered != nullptr) {
        uint4* g = a.gathered + row * a.V;
#pragma unroll
        for (int j = 0; j < HB; ++j) {
          const int p = half_block(j);
          stg_stream_pair(g + 2 * p, h[2 * j], h[2 * j + 1], a.wide);
        }
      }
      const bool fast_div = (m >= 8.6736174e-19f) && (m <= 1.1529215e18f);
      const float r = fast_div ? __frcp_rn(m) : 0.0f;
      uint4* yr = a.y + row * a.V;
      if (OWNER == kOwnerToRowOwner) {
        // the one destination of this row: the buffer of the rank whose row block contains it
        int r = 0;
#pragma unroll
        for (int d = 1; d < 8; ++d)
          if (d <= a.n_more && row >= a.row_bounds[d]) r = d;
        yr = (r == 0 ? a.y : a.y_more[r - 1]) + (row - a.row_bounds[r]) * a.V;
      }
      // |h| >= the smallest block scale for every non-zero element: above 2^-40 no product with
      // 1/m (m <= 2^60) can fall under 2^-100, and the guard can go.
      // one finished 32-byte piece to the local buffer and to every further destination
      auto put = [&](int p, const uint4& lo, const uint4& hi) {
        stg_stream_pair(yr + 2 * p, lo, hi, a.wide);
        if (OWNER == kOwnerToAll) {
#pragma unroll
          for (int d = 0; d < 7; ++d) {
            if (d < a.n_more) stg_stream_pair(a.y_more[d] + row * a.V + 2 * p, lo, hi, a.wide);
          }
        }
      };
      // The common case -- every non-zero |h| is at least the smallest block scale >= 2^-40, so no
      // quotient can fall under 2^-100, and m allows the reciprocal -- runs unrolled with nothing but
      // the multiplications; anything else calls the guarded form out of line.
      // (rows of a dense table carry no scales to bound their elements by: bf16 keeps the guard)
      const bool plain =
          fast_div && ((DT != kDtBF16) || (QT != kQTypeDense16 && row_dmin >= 9.0949470e-13f));
      if (QT == kQTypeDense16 && !plain) {
#pragma unroll
        for (int j = 0; j < HB; ++j) {
          const int p = half_block(j);
          put(p, rms_output_vec<DT, true>(h[2 * j], alpha_vec(2 * j), m, r, fast_div),
              rms_output_vec<DT, true>(h[2 * j + 1], alpha_vec(2 * j + 1), m, r, fast_div));
        }
      } else if (plain) {
#pragma unroll
        for (int j = 0; j < HB; ++j) {
          const int p = half_block(j);
          put(p, rms_output_plain<DT>(h[2 * j], alpha_vec(2 * j), m, r),
              rms_output_plain<DT>(h[2 * j + 1], alpha_vec(2 * j + 1), m, r));
        }
      } else {
#pragma unroll
        for (int j = 0; j < HB; ++j) {
          const int p = half_block(j);
          put(p, rms_output_rare<DT>(h[2 * j], alpha_vec(2 * j), m, r, fast_div),
              rms_output_rare<DT>(h[2 * j + 1], alpha_vec(2 * j + 1), m, r, fast_div));
        }
      }
    }
    // all lanes are done with `buf` (decode and, if any, replay) before the next refill
    if (tpr > 32)
      row_barrier(bar_id, tpr);
    else
      __syncwarp();
    stage = stage + 1 == stages ? 0 : stage + 1;
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

// Shape of the quantised-source kernel: HB half blocks (16 elements) per thread, a warp per row
// up to 4096 columns.  V == 2 * HB * tpr exactly.
static bool qrowreg_shape(int V, int& tpr, int& hb) {
  // (a whole 4096-column row in one warp, eight half blocks per thread, was measured slower on the
  // Q8_0 lookup: 252 us against 216 us for two warps per row)
  for (int t = 32; t <= 128; t <<= 1) {
    for (int cand = 4; cand >= 1; --cand) {
      if (V == 2 * cand * t) {
        tpr = t;
        hb = cand;
        return true;
      }
    }
  }
  return false;
}

bool rms_rowreg_supported(int dtype, int cols) {
  int tpr, vpt, rpc;
  return (dtype == kDtBF16 || dtype == kDtF16) && cols % 8 == 0 && cols >= 256 && cols <= 32768 &&
         rowreg_shape(cols / 8, tpr, vpt, rpc);
}

bool qrms_rowreg_supported(int dtype, int cols) {
  int tpr, hb;
  return (dtype == kDtBF16 || dtype == kDtF16) && cols % 32 == 0 && qrowreg_shape(cols / 8, tpr, hb);
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
  int per_sm = 1, sms = 1;
  cudaError_t e = kernel_launch_config(reinterpret_cast<const void*>(kern), threads, smem, percent, &per_sm);
  if (e != cudaSuccess) return e;
  e = device_sm_count(&sms);
  if (e != cudaSuccess) return e;
  int64_t g = static_cast<int64_t>(sms) * per_sm;
  if (g > work_items) g = work_items;
  grid = static_cast<unsigned>(g);
  return cudaSuccess;
}

template <int DT, int VPT, int BT, int MODE>
static cudaError_t launch_dense_t(const RmsRowRegArgs& a, int tpr, int rpc, cudaStream_t stream) {
  const bool with_rows = !(a.flags & CB200_FLAG_FAST_SUM);
  const size_t smem = RowRegSmem::bytes(rpc, tpr, a.V, with_rows);
  auto kern = rms_rowreg_kernel<DT, VPT, BT, MODE>;
  unsigned grid = 1;
  cudaError_t e = persistent_grid(kern, tpr * rpc, smem, 768 / BT, (a.rows + rpc - 1) / rpc, grid);
  if (e != cudaSuccess) return e;
  kern<<<grid, dim3(tpr, rpc), smem, stream>>>(a);
  return cudaGetLastError();
}

template <int DT, int VPT>
static cudaError_t launch_dense_bt(const RmsRowRegArgs& a, int tpr, int rpc, cudaStream_t stream) {
  // beyond these sizes the second set of registers spills
  constexpr int kAhead = VPT <= 4 ? kModeAhead : 0;
  constexpr int kAheadG = VPT <= 3 ? kModeAhead : 0;
  const bool gather = a.ids != nullptr, plain = a.res != nullptr;
  if (tpr * rpc <= 256) {
    if (gather) return launch_dense_t<DT, VPT, 256, kModeGather | kAheadG>(a, tpr, rpc, stream);
    if (plain) {
      // look-ahead with a residual pays for rows of up to 4096 columns when there are many of them
      // (measured: 0.77 -> 0.80 of peak at 4096 columns, 0.75 -> 0.81 at 2048; nothing at 8192, and
      // a loss when each CTA sees only a few rows)
      if (kAhead != 0 && tpr <= 128 && a.rows >= 16384)
        return launch_dense_t<DT, VPT, 256, kAhead ? kModeAheadRes : 0>(a, tpr, rpc, stream);
      return launch_dense_t<DT, VPT, 256, 0>(a, tpr, rpc, stream);
    }
    return launch_dense_t<DT, VPT, 256, kAhead>(a, tpr, rpc, stream);
  }
  if (gather) return launch_dense_t<DT, VPT, 512, kModeGather | kAheadG>(a, tpr, rpc, stream);
  if (plain) return launch_dense_t<DT, VPT, 512, 0>(a, tpr, rpc, stream);
  return launch_dense_t<DT, VPT, 512, kAhead>(a, tpr, rpc, stream);
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

template <int QT, int DT, int HB>
static cudaError_t launch_q_t(const QRmsArgs& a_in, int tpr, cudaStream_t stream) {
  QRmsArgs a = a_in;
  a.wt = wait_tuning();
  // every output buffer on a 32-byte boundary (rows are multiples of 64 bytes): 256-bit stores
  auto aligned32 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; };
  a.wide = aligned32(a.y) && aligned32(a.gathered);
  for (int d = 0; d < a.n_more && d < 7; ++d) a.wide = a.wide && aligned32(a.y_more[d]);
  const int rpc = 128 / tpr;  // row slots per 128-thread CTA
  const int ctas = 4;         // CTAs per SM: the register budget (alpha stays resident) and the barriers admit four
  const int stage_bytes = (a.row_bytes + 15) & ~15;
  // ring depth: what 196 KB of shared memory per SM (a carve-out the hardware offers; the next one
  // is all 228 KB) allows with `ctas` CTAs resident and 1 KB reserved per CTA; at least 2 (one row ahead)
  int stages = 2;
  while (stages < 4 && (QSlot::bytes(stages + 1, stage_bytes, tpr) * rpc + 1024) * ctas <= 196 * 1024) ++stages;
  const size_t smem = QSlot::bytes(stages, stage_bytes, tpr) * rpc;
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  // the owner-writes-to-all mode is a variant of its own: the plain lookup carries none of its code
  auto kern = qrms_rowslot_kernel<QT, DT, HB, kOwnerNone>;
  if constexpr (QT != kQTypeDense16) {
    if (a.owned_only == 1) kern = qrms_rowslot_kernel<QT, DT, HB, kOwnerToAll>;
    if (a.owned_only == 2) kern = qrms_rowslot_kernel<QT, DT, HB, kOwnerToRowOwner>;
  }
  unsigned grid = 1;
  cudaError_t e = persistent_grid(kern, 128, smem, ctas, (a.rows + rpc - 1) / rpc, grid);
  if (e != cudaSuccess) return e;
  kern<<<grid, dim3(tpr, rpc), smem, stream>>>(a, stages);
  return cudaGetLastError();
}

template <int QT, int DT>
static cudaError_t launch_q_dt(const QRmsArgs& a, cudaStream_t stream) {
  int tpr = 0, hb = 0;
  if (!qrowreg_shape(a.V, tpr, hb)) return cudaErrorInvalidValue;
  switch (hb) {
    case 1:
      return launch_q_t<QT, DT, 1>(a, tpr, stream);
    case 2:
      return launch_q_t<QT, DT, 2>(a, tpr, stream);
    case 3:
      return launch_q_t<QT, DT, 3>(a, tpr, stream);
    default:
      return launch_q_t<QT, DT, 4>(a, tpr, stream);
  }
}

cudaError_t launch_qrms_rowreg(int qtype, int dtype, const QRmsArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  if (qtype == kQTypeDense16)
    return dtype == kDtBF16 ? launch_q_dt<kQTypeDense16, kDtBF16>(a, stream)
                            : launch_q_dt<kQTypeDense16, kDtF16>(a, stream);
  if (qtype == CB200_QTYPE_Q8_0)
    return dtype == kDtBF16 ? launch_q_dt<CB200_QTYPE_Q8_0, kDtBF16>(a, stream)
                            : launch_q_dt<CB200_QTYPE_Q8_0, kDtF16>(a, stream);
  return dtype == kDtBF16 ? launch_q_dt<CB200_QTYPE_Q4_0, kDtBF16>(a, stream)
                          : launch_q_dt<CB200_QTYPE_Q4_0, kDtF16>(a, stream);
}

}  // namespace cb200
