// Lane-per-row norms: the exact-order kernels for layer norm (all dtypes) and f32 RMS norm.
//
// candle's CPU path accumulates each row's sum (and sum of squares) strictly left to right in
// f32 (candle-nn/src/ops.rs:484-490, 709-715).  For these ops nothing coarser than f32 absorbs
// the rounding of that sum, so bit-equal results need the same order: one LANE per row walks its
// row sequentially, 32 independent dependency chains per warp.  Three kernels share that walk and
// differ in how rows reach it:
//   norm_shortrow_kernel  rows of 512..2048 bytes, many of them: tiles of whole rows in a ring of
//                         shared-memory buffers, copies two tiles ahead, the walk hidden behind
//                         the previous tile's stores (each row read from HBM once);
//   norm_stream_kernel    rows of 512 bytes and more otherwise (long rows, few rows, gathered
//                         rows): rows streamed through a ring of 2 KB chunks, read a second time
//                         (L2) for the normalise-and-store pass;
//   norm_lanerow_kernel   rows under 512 bytes, and the cross-check of the two above: R whole rows
//                         staged per CTA (h = T(x + residual), or rows gathered by the bulk-copy
//                         engine), walk, then all threads normalise and store.
// Row pitches in shared memory are an odd number of 16-byte units so that the 16-byte loads of the
// lane-per-row walk are bank-conflict free.  norm_generic_kernel takes what is not 16-byte shaped.
#include "launch.h"
#include "rms_rowreg.cuh"

namespace cb200 {

constexpr int kLaneRowThreads = 256;
constexpr int kLaneRowWarps = kLaneRowThreads / 32;

template <int DT, int OP>
__global__ void __launch_bounds__(kLaneRowThreads) norm_lanerow_kernel(const LaneRowArgs a) {
  constexpr int PV = Elem<DT>::kPerVec;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* rowbuf = smem_raw;                                                  // [R][pitch]
  float2* stats = reinterpret_cast<float2*>(smem_raw + static_cast<size_t>(a.R) * a.pitch);  // [R]
  int* valid = reinterpret_cast<int*>(stats + a.R);                                  // [R]
  uint64_t* bar = reinterpret_cast<uint64_t*>(valid + a.R + (a.R & 1));              // 8-byte aligned

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * a.R;
  const int live = static_cast<int>(min(static_cast<int64_t>(a.R), a.rows - row0));
  const uint4* gx = static_cast<const uint4*>(a.x);

  // ---- fill ----
  if (a.ids != nullptr) {
    if (a.bulk) {
      if (tid == 0) {
        mbar_init(bar, 1);
        mbar_init_fence();
        uint32_t bytes = 0;
        for (int r = 0; r < live; ++r) {
          uint64_t id = read_id(a.ids, a.id_dtype, row0 + r);
          int ok = id < static_cast<uint64_t>(a.vocab);
          valid[r] = ok;
          if (ok)
            bytes += static_cast<uint32_t>(a.V) * 16u;
          else
            report_status(a.status, CB200_STATUS_INVALID_INDEX, row0 + r, static_cast<int64_t>(id), a.vocab);
        }
        mbar_expect_tx(bar, bytes + a.wt.extra_tx);
        for (int r = 0; r < live; ++r) {
          if (!valid[r]) continue;
          uint64_t id = read_id(a.ids, a.id_dtype, row0 + r);
          bulk_g2s(rowbuf + static_cast<size_t>(r) * a.pitch, gx + id * a.V, static_cast<uint32_t>(a.V) * 16u, bar);
        }
      }
      __syncthreads();
      const bool ok = mbar_wait(bar, 0, a.wt.spins);
      if (!__syncthreads_and(ok ? 1 : 0)) {
        // give the copies in flight one more bounded chance to land before the CTA retires
        if (tid == 0) {
          mbar_wait(bar, 0, a.wt.spins);
          drain_pause();
          report_status(a.status, CB200_STATUS_WAIT_TIMEOUT, row0, 0, a.vocab);
        }
        return;
      }
    } else {
      for (int r = warp; r < live; r += kLaneRowWarps) {
        uint64_t id = read_id(a.ids, a.id_dtype, row0 + r);
        int ok = id < static_cast<uint64_t>(a.vocab);
        if (lane == 0) {
          valid[r] = ok;
          if (!ok) report_status(a.status, CB200_STATUS_INVALID_INDEX, row0 + r, static_cast<int64_t>(id), a.vocab);
        }
        if (!ok) continue;
        uint4* dst = reinterpret_cast<uint4*>(rowbuf + static_cast<size_t>(r) * a.pitch);
        for (int v = lane; v < a.V; v += 32) dst[v] = ldg_stream(gx + id * a.V + v);
      }
      __syncthreads();
    }
  } else {
    const uint4* gr = static_cast<const uint4*>(a.res);
    uint4* gs = static_cast<uint4*>(a.sum_out);
    // Each warp fills rows warp, warp+8, ...; four rows at a time so that eight 16-byte loads
    // per lane are in flight before the first one is consumed.
    constexpr int RPW = 4;
    for (int rb = warp; rb < live; rb += kLaneRowWarps * RPW) {
      for (int v = lane; v < a.V; v += 32) {
        uint4 xv[RPW], rv[RPW];
#pragma unroll
        for (int j = 0; j < RPW; ++j) {
          const int r = rb + kLaneRowWarps * j;
          xv[j] = (r < live) ? ldg_stream(gx + (row0 + r) * a.V + v) : make_uint4(0, 0, 0, 0);
        }
        if (gr != nullptr) {
#pragma unroll
          for (int j = 0; j < RPW; ++j) {
            const int r = rb + kLaneRowWarps * j;
            rv[j] = (r < live) ? ldg_stream(gr + (row0 + r) * a.V + v) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int j = 0; j < RPW; ++j) {
            if constexpr (DT == kDtF32) {
              float fa[PV], fb[PV];
              vec_to_floats<DT>(xv[j], fa);
              vec_to_floats<DT>(rv[j], fb);
#pragma unroll
              for (int e = 0; e < PV; ++e) fa[e] = __fadd_rn(fa[e], fb[e]);
              xv[j] = floats_to_vec<DT>(fa);
            } else {
              xv[j] = add_round_vec<DT>(xv[j], rv[j]);  // rounds the sum to T, as Tensor::add does
            }
          }
        }
#pragma unroll
        for (int j = 0; j < RPW; ++j) {
          const int r = rb + kLaneRowWarps * j;
          if (r < live) {
            reinterpret_cast<uint4*>(rowbuf + static_cast<size_t>(r) * a.pitch)[v] = xv[j];
            if (gs != nullptr) stg_stream(gs + (row0 + r) * a.V + v, xv[j]);
          }
        }
      }
    }
    if (tid < live) valid[tid] = 1;
    __syncthreads();
  }

  // ---- pass 1: one lane per row, strictly sequential f32 accumulation ----
  if (tid < live && valid[tid]) {
    const uint4* row = reinterpret_cast<const uint4*>(rowbuf + static_cast<size_t>(tid) * a.pitch);
    float s = 0.0f, s2 = 0.0f;
#pragma unroll 4
    for (int v = 0; v < a.V; ++v) {
      float f[PV];
      vec_to_floats<DT>(row[v], f);
#pragma unroll
      for (int e = 0; e < PV; ++e) {
        if (OP == kOpLayerNorm) s = __fadd_rn(s, f[e]);
        s2 = __fadd_rn(s2, __fmul_rn(f[e], f[e]));
      }
    }
    const float nf = static_cast<float>(a.n);
    if (OP == kOpLayerNorm) {
      // candle-nn/src/ops.rs:716-718
      float mean = __fdiv_rn(s, nf);
      float var = __fsub_rn(__fdiv_rn(s2, nf), __fmul_rn(mean, mean));
      float inv_std = __frcp_rn(__fsqrt_rn(__fadd_rn(var, a.eps)));
      stats[tid] = make_float2(mean, inv_std);
    } else {
      // candle-nn/src/ops.rs:491-492
      stats[tid] = make_float2(round_to<DT>(rms_from_sum(s2, nf, a.eps)), 0.0f);
    }
  }
  __syncthreads();

  // ---- pass 2: normalise and store, 16 bytes per thread, coalesced ----
  const uint4* ga = static_cast<const uint4*>(a.alpha);
  const uint4* gb = static_cast<const uint4*>(a.beta);
  uint4* gy = static_cast<uint4*>(a.y);
  uint4* gg = (a.ids != nullptr) ? static_cast<uint4*>(a.sum_out) : nullptr;  // gathered rows
  for (int r = warp; r < live; r += kLaneRowWarps) {
    if (!valid[r]) continue;
    const float2 st = stats[r];
    const RowDivisor dv = make_row_divisor(st.x);  // (used by the RMS norm only)
    const int64_t base = (row0 + r) * a.V;
    const uint4* row = reinterpret_cast<const uint4*>(rowbuf + static_cast<size_t>(r) * a.pitch);
    for (int v = lane; v < a.V; v += 32) {
      const uint4 hv = row[v];
      float h[PV], g[PV], o[PV];
      vec_to_floats<DT>(hv, h);
      vec_to_floats<DT>(__ldg(ga + v), g);
      if (OP == kOpLayerNorm) {
        float b[PV];
        vec_to_floats<DT>(__ldg(gb + v), b);
#pragma unroll
        for (int e = 0; e < PV; ++e)
          o[e] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(h[e], st.x), st.y), g[e]), b[e]);
      } else {
#pragma unroll
        for (int e = 0; e < PV; ++e) o[e] = __fmul_rn(round_to<DT>(div_by_row(h[e], dv)), g[e]);
      }
      stg_stream(gy + base + v, floats_to_vec<DT>(o));
      if (gg != nullptr) stg_stream(gg + base + v, hv);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Short rows (V = 32 * VPL 16-byte vectors, VPL <= 4; e.g. 768 bf16 columns): a software-
// pipelined, persistent version of the same scheme.  One 512-thread CTA per SM walks tiles of
// 32 rows (24 for VPL = 4) through a ring of three row buffers:
//   * a tile's x rows (and residual rows) arrive in shared memory by asynchronous 16-byte
//     copies, which bypass L1 and registers, so the large shared-memory carve-out this kernel
//     needs does not limit the bytes in flight; the copies of tile t+1 are started as soon as
//     tile t has been turned into h = T(x + residual) (in place, each thread its own vectors);
//   * warp 0 then walks tile t sequentially, one lane per row, while the mover warps normalise
//     and store tile t-1 with gamma / beta held widened in registers and then refill its buffer
//     with the x rows of tile t+2.  The walk is a chain of dependent additions that runs at the
//     floating-point latency only while nothing else competes for its scheduler, so the movers
//     are the warps of the three other schedulers (warp index not a multiple of four); warps
//     4, 8 and 12 only take part in the CTA barriers.
// ---------------------------------------------------------------------------------------------
constexpr int kShortThreads = 512;
constexpr int kShortWarps = kShortThreads / 32;

// rows per tile: four buffers of (rows x (32 VPL + 1)) vectors must fit in 227 KB
template <int VPL>
struct ShortTile {
  static constexpr int kRows = VPL == 4 ? 24 : 32;
};

template <int DT, int OP, int VPL>
__global__ void __launch_bounds__(kShortThreads, 1) norm_shortrow_kernel(const LaneRowArgs a, const int tile_rows) {
  constexpr int PV = Elem<DT>::kPerVec;
  constexpr int V = 32 * VPL;
  constexpr int TR = ShortTile<VPL>::kRows;  // buffer rows; a tile has tile_rows <= TR of them
  constexpr int kPitchVecs = V + 1;  // odd number of 16-byte units: conflict-free lane-per-row walk
  constexpr int kBufVecs = TR * kPitchVecs;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* const smem_v = reinterpret_cast<uint4*>(smem_raw);  // x ring: buffers 0..2, then the residual buffer
  uint4* const rbuf = smem_v + 3 * kBufVecs;
  float2* const stats = reinterpret_cast<float2*>(rbuf + kBufVecs);  // [2][TR]: {sum, sum of squares}

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint4* gx = static_cast<const uint4*>(a.x);
  const uint4* gr = static_cast<const uint4*>(a.res);
  uint4* gs = static_cast<uint4*>(a.sum_out);
  uint4* gy = static_cast<uint4*>(a.y);
  const bool has_res = gr != nullptr;
  const int64_t n_tiles = (a.rows + tile_rows - 1) / tile_rows;

  // gamma / beta of this lane's vectors, widened once (filled below, after the first copies are on
  // their way)
  float gam[VPL][PV], bet[VPL][PV];

  // Mover m owns rows m + 12 k of every tile, vectors lane + 32 j, for the copies, the in-place
  // conversion and the stores alike, so a thread converts only what it copied itself.
  constexpr int kMovers = kShortWarps - kShortWarps / 4;
  const bool is_mover = (warp & 3) != 0;
  const int mover = (warp >> 2) * 3 + (warp & 3) - 1;
  constexpr int kRowsPerMover = (TR + kMovers - 1) / kMovers;
  auto issue_rows = [&](const uint4* __restrict__ g, uint4* buf, int64_t tile) {
    if (g != nullptr && tile < n_tiles && is_mover) {
#pragma unroll
      for (int k = 0; k < kRowsPerMover; ++k) {
        const int r = mover + kMovers * k;
        const int64_t row = tile * tile_rows + r;
        if (r < tile_rows && row < a.rows) {
#pragma unroll
          for (int j = 0; j < VPL; ++j) cp_async16(buf + r * kPitchVecs + lane + 32 * j, g + row * V + lane + 32 * j);
        }
      }
    }
    cp_async_commit();  // an empty group keeps the group count in step
  };

  // pass 2 of one tile
  auto store_tile = [&](int64_t tile, int slot, int parity) {
    const int64_t row0 = tile * tile_rows;
    const int live = static_cast<int>(min(static_cast<int64_t>(tile_rows), a.rows - row0));
    const uint4* xb = smem_v + slot * kBufVecs;
#pragma unroll
    for (int k = 0; k < kRowsPerMover; ++k) {
      const int r = mover + kMovers * k;
      if (r < live) {
        const float2 sums = stats[parity * TR + r];
        const float nf = static_cast<float>(a.n);
        float2 st;
        if (OP == kOpLayerNorm) {
          const float mean = __fdiv_rn(sums.x, nf);
          const float var = __fsub_rn(__fdiv_rn(sums.y, nf), __fmul_rn(mean, mean));
          st = make_float2(mean, __frcp_rn(__fsqrt_rn(__fadd_rn(var, a.eps))));
        } else {
          st = make_float2(round_to<DT>(rms_from_sum(sums.y, nf, a.eps)), 0.0f);
        }
        const RowDivisor dv = make_row_divisor(st.x);  // (used by the RMS norm only)
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
          const int v = lane + 32 * j;
          float h[PV], o[PV];
          vec_to_floats<DT>(xb[r * kPitchVecs + v], h);
          if (OP == kOpLayerNorm) {
#pragma unroll
            for (int e = 0; e < PV; ++e)
              o[e] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(h[e], st.x), st.y), gam[j][e]), bet[j][e]);
          } else {
#pragma unroll
            for (int e = 0; e < PV; ++e) o[e] = __fmul_rn(round_to<DT>(div_by_row(h[e], dv)), gam[j][e]);
          }
          stg_stream(gy + (row0 + r) * V + v, floats_to_vec<DT>(o));
        }
      }
    }
  };

  // Copy groups of a mover thread, in order: x(0), r(0), x(1), then per iteration r(t+1), x(t+2).
  // At the top of iteration t the groups x(t) and r(t) must have landed and only x(t+1), the
  // newest, may still be in flight.
  const int64_t stride = gridDim.x;
  issue_rows(gx, smem_v, blockIdx.x);
  issue_rows(gr, rbuf, blockIdx.x);
  issue_rows(gx, smem_v + kBufVecs, blockIdx.x + stride);
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    vec_to_floats<DT>(__ldg(static_cast<const uint4*>(a.alpha) + lane + 32 * j), gam[j]);
    if (OP == kOpLayerNorm) vec_to_floats<DT>(__ldg(static_cast<const uint4*>(a.beta) + lane + 32 * j), bet[j]);
  }

  int slot = 0, it = 0;
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += stride, ++it) {
    const int64_t row0 = tile * tile_rows;
    const int live = static_cast<int>(min(static_cast<int64_t>(tile_rows), a.rows - row0));
    uint4* xb = smem_v + slot * kBufVecs;
    const int next_slot = slot == 2 ? 0 : slot + 1;
    const int prev_slot = slot == 0 ? 2 : slot - 1;
    if (is_mover) {
      cp_async_wait_pending(1);
      if (has_res || gs != nullptr) {
#pragma unroll
        for (int k = 0; k < kRowsPerMover; ++k) {
          const int r = mover + kMovers * k;
          if (r < live) {
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
              const int v = lane + 32 * j;
              uint4* px = xb + r * kPitchVecs + v;
              uint4 h = *px;
              if (has_res) {
                if constexpr (DT == kDtF32) {
                  float fa[PV], fb[PV];
                  vec_to_floats<DT>(h, fa);
                  vec_to_floats<DT>(rbuf[r * kPitchVecs + v], fb);
#pragma unroll
                  for (int e = 0; e < PV; ++e) fa[e] = __fadd_rn(fa[e], fb[e]);
                  h = floats_to_vec<DT>(fa);
                } else {
                  h = add_round_vec<DT>(h, rbuf[r * kPitchVecs + v]);  // rounds the sum to T, as Tensor::add does
                }
                *px = h;
              }
              if (gs != nullptr) stg_stream(gs + (row0 + r) * V + v, h);
            }
          }
        }
      }
    }
    __syncthreads();  // tile t is h everywhere, the residual buffer is free, pass 1 of tile t-1 is done

    if (warp == 0) {
      // ---- pass 1 of tile t: one lane per row, strictly sequential f32 accumulation ----
      if (lane < live) {
        const uint4* row = xb + lane * kPitchVecs;
        float s = 0.0f, s2 = 0.0f;
        // Four vectors are fetched while the previous four are accumulated, so the chains of
        // dependent additions never wait for shared memory; the two register sets swap roles every
        // half trip instead of being copied (V is a multiple of 32: an even number of groups).
        auto add_vec = [&](const uint4& hv) {
          float f[PV];
          vec_to_floats<DT>(hv, f);
#pragma unroll
          for (int e = 0; e < PV; ++e) {
            if (OP == kOpLayerNorm) s = __fadd_rn(s, f[e]);
            // for 16-bit inputs f*f is exact in f32, so the fused form rounds like add(s2, mul(f, f))
            s2 = (DT == kDtF32) ? __fadd_rn(s2, __fmul_rn(f[e], f[e])) : fmaf(f[e], f[e], s2);
          }
        };
        uint4 ga[4], gb[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) ga[q] = row[q];
#pragma unroll 1
        for (int v = 0; v < V; v += 8) {
#pragma unroll
          for (int q = 0; q < 4; ++q) gb[q] = row[v + 4 + q];
#pragma unroll
          for (int q = 0; q < 4; ++q) add_vec(ga[q]);
          const int vn = v + 8 < V ? v + 8 : 0;
#pragma unroll
          for (int q = 0; q < 4; ++q) ga[q] = row[vn + q];
#pragma unroll
          for (int q = 0; q < 4; ++q) add_vec(gb[q]);
        }
        stats[(it & 1) * TR + lane] = make_float2(s, s2);
      }
    } else if (is_mover) {
      issue_rows(gr, rbuf, tile + stride);
      // ---- pass 2 of tile t-1, then its buffer takes the x rows of tile t+2 ----
      if (it > 0) store_tile(tile - stride, prev_slot, (it - 1) & 1);
      row_barrier(1, kMovers * 32);  // every mover is done reading that buffer
      issue_rows(gx, smem_v + prev_slot * kBufVecs, tile + 2 * stride);
    }
    slot = next_slot;
  }
  __syncthreads();
  if (is_mover && it > 0) store_tile(blockIdx.x + static_cast<int64_t>(it - 1) * stride, slot == 0 ? 2 : slot - 1, (it - 1) & 1);
  cp_async_wait_all();
}

// ---------------------------------------------------------------------------------------------
// Long rows: the sequential walk over rows that are STREAMED through shared memory instead of
// staged whole.  The walk is bound by the floating-point latency of its dependent additions, so
// a warp that walks 32 rows side by side consumes about as many bytes per second as an SM's share
// of HBM delivers -- provided the rows do not have to fit in shared memory.  Per CTA (one per SM,
// persistent over tiles of TR <= 32 rows):
//   * warp 0 owns a ring of D stages; a stage holds one chunk of CV vectors of each of the
//     tile's rows (and of the residual rows).  Each lane copies the chunks of its own row with
//     the bulk-copy engine, completion counted on the stage's mbarrier; the lane then walks the
//     chunk and refills the stage with the chunk D steps ahead, across tile boundaries.  No
//     other warp takes part, so the walk never waits for anything but memory.  The engine takes
//     about 35 ns per copy whatever its size, so one warp's copies deliver an SM's share of HBM
//     only from 2 KB per copy on, which is the chunk size (CV = 128).
//   * the other warps (those of the three schedulers warp 0 is not on) normalise the previous
//     tile meanwhile: they read its rows a second time -- from L2 as long as the tiles in flight
//     on all SMs fit there -- and store the result.
// ---------------------------------------------------------------------------------------------
constexpr int kStreamThreads = 768;
constexpr int kStreamWarps = kStreamThreads / 32;
constexpr int kStreamFinishers = kStreamWarps - kStreamWarps / 4;
constexpr int kStreamMaxStages = 8;
// vectors of a row per stage, and the bytes of a row's slot (an odd number of 16-byte units)
__host__ __device__ inline int stream_chunk_pitch(int cv) { return (cv + 1) * 16; }

struct StreamSmem {
  unsigned char* xring;
  unsigned char* rring;
  uint64_t* bars;    // [D]
  float2* stats;     // [2][32]: {sum, sum of squares} of the tile walked in iteration it & 1
  int64_t* src;      // [4][32]: source row of each tile row (-1: none), iteration it & 3
  volatile int* abort_flag;
  __device__ StreamSmem(unsigned char* base, int TR, int D, int cv, bool res) {
    const size_t ring = static_cast<size_t>(D) * TR * stream_chunk_pitch(cv);
    xring = base;
    rring = base + ring;
    bars = reinterpret_cast<uint64_t*>(base + ring * (res ? 2 : 1));
    stats = reinterpret_cast<float2*>(bars + kStreamMaxStages);
    src = reinterpret_cast<int64_t*>(stats + 64);
    abort_flag = reinterpret_cast<volatile int*>(src + 128);
  }
  static size_t bytes(int TR, int D, int cv, bool res) {
    return static_cast<size_t>(D) * TR * stream_chunk_pitch(cv) * (res ? 2 : 1) + kStreamMaxStages * 8 + 64 * 8 + 128 * 8 + 16;
  }
};

template <int DT, int OP, bool RES>
__global__ void __launch_bounds__(kStreamThreads, 1) norm_stream_kernel(const LaneRowArgs a, int TR, int D, int CV) {
  constexpr int PV = Elem<DT>::kPerVec;
  constexpr int G = RES ? 2 : 4;  // vectors fetched from shared memory ahead of the chain
  const int kChunkVecs = CV;  // vectors of a row per stage
  const int kChunkPitch = stream_chunk_pitch(CV);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  StreamSmem sm(smem_raw, TR, D, CV, RES);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = a.V;
  const int nc = (V + kChunkVecs - 1) / kChunkVecs;
  const int64_t tiles = (a.rows + TR - 1) / TR;
  const int64_t stride = gridDim.x;
  const bool gather = a.ids != nullptr;
  const uint4* gx = static_cast<const uint4*>(a.x);
  const uint4* gr = static_cast<const uint4*>(a.res);

  if (tid == 0) {
    for (int s = 0; s < D; ++s) mbar_init(&sm.bars[s], 1);
    mbar_init_fence();
    *sm.abort_flag = 0;
  }
  __syncthreads();

  // ---- pass 2 of one tile: the rows are cut into segments of 32 U vectors and the segments
  // dealt round-robin to `workers` warps (the finishers; every warp for the last tile) ----
  const bool is_finisher = (warp & 3) != 0;
  const int finisher = (warp >> 2) * 3 + (warp & 3) - 1;
  auto finish_tile = [&](int64_t tile, int it_t, int worker, int workers) {
    const uint4* ga = static_cast<const uint4*>(a.alpha);
    const uint4* gb = static_cast<const uint4*>(a.beta);
    uint4* gy = static_cast<uint4*>(a.y);
    uint4* gs = static_cast<uint4*>(a.sum_out);
    const float nf = static_cast<float>(a.n);
    // 32 registers of loads in flight per thread: the second read has to cover the latency of
    // L2, or of HBM where the rows have left L2
    constexpr int U = RES ? 4 : 8;
    const int segs = (V + 32 * U - 1) / (32 * U);
    for (int item = worker; item < TR * segs; item += workers) {
      const int r = item / segs;
      const int64_t src = sm.src[(it_t & 3) * 32 + r];
      if (src < 0) continue;
      const int64_t row = tile * TR + r;
      const float2 sums = sm.stats[(it_t & 1) * 32 + r];
      float2 st;
      if (OP == kOpLayerNorm) {
        const float mean = __fdiv_rn(sums.x, nf);  // candle-nn/src/ops.rs:716-718
        const float var = __fsub_rn(__fdiv_rn(sums.y, nf), __fmul_rn(mean, mean));
        st = make_float2(mean, __frcp_rn(__fsqrt_rn(__fadd_rn(var, a.eps))));
      } else {
        st = make_float2(round_to<DT>(rms_from_sum(sums.y, nf, a.eps)), 0.0f);  // ops.rs:491-492
      }
      const RowDivisor dv = make_row_divisor(st.x);  // (used by the RMS norm only)
      const uint4* xr = gx + src * V;
      const uint4* rr = RES ? gr + row * V : nullptr;
      uint4* yr = gy + row * V;
      uint4* so = gs != nullptr ? gs + row * V : nullptr;
      const int v0 = (item - r * segs) * 32 * U + lane;
      uint4 hv[U];
#pragma unroll
      for (int u = 0; u < U; ++u) hv[u] = (v0 + 32 * u < V) ? __ldg(xr + v0 + 32 * u) : make_uint4(0, 0, 0, 0);
      if (RES) {
        uint4 rv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) rv[u] = (v0 + 32 * u < V) ? __ldg(rr + v0 + 32 * u) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if constexpr (DT == kDtF32) {
            float fa[PV], fb[PV];
            vec_to_floats<DT>(hv[u], fa);
            vec_to_floats<DT>(rv[u], fb);
#pragma unroll
            for (int e = 0; e < PV; ++e) fa[e] = __fadd_rn(fa[e], fb[e]);
            hv[u] = floats_to_vec<DT>(fa);
          } else {
            hv[u] = add_round_vec<DT>(hv[u], rv[u]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + 32 * u;
        if (v < V) {
          float h[PV], g[PV], o[PV];
          vec_to_floats<DT>(hv[u], h);
          vec_to_floats<DT>(__ldg(ga + v), g);
          if (OP == kOpLayerNorm) {
            float b[PV];
            vec_to_floats<DT>(__ldg(gb + v), b);
#pragma unroll
            for (int e = 0; e < PV; ++e)
              o[e] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(h[e], st.x), st.y), g[e]), b[e]);
          } else {
#pragma unroll
            for (int e = 0; e < PV; ++e) o[e] = __fmul_rn(round_to<DT>(div_by_row(h[e], dv)), g[e]);
          }
          stg_stream(yr + v, floats_to_vec<DT>(o));
          if (so != nullptr) stg_stream(so + v, hv[u]);
        }
      }
    }
  };

  // ---- the walker's copy stream: chunk number g goes to stage g % D, parity (g / D) & 1 ----
  int64_t tile_i = blockIdx.x;  // tile, chunk and iteration the next copy belongs to
  int chunk_i = 0, it_i = 0;
  uint32_t g_i = 0, g_c = 0;    // chunks issued / consumed so far
  const unsigned char* xs_i = nullptr;
  const unsigned char* rs_i = nullptr;
  bool live_i = false;
  int nlive_i = 0;
  const size_t row_bytes = static_cast<size_t>(V) * 16;
  auto open_tile = [&]() {  // warp 0: sources of tile_i
    const int64_t row = tile_i * TR + lane;
    bool live = lane < TR && row < a.rows;
    int64_t src = row;
    if (gather && live) {
      const uint64_t id = read_id(a.ids, a.id_dtype, row);
      if (id >= static_cast<uint64_t>(a.vocab)) {
        report_status(a.status, CB200_STATUS_INVALID_INDEX, row, static_cast<int64_t>(id), a.vocab);
        live = false;
      } else {
        src = static_cast<int64_t>(id);
      }
    }
    sm.src[(it_i & 3) * 32 + lane] = live ? src : -1;
    xs_i = static_cast<const unsigned char*>(a.x) + (live ? src : 0) * row_bytes;
    rs_i = RES ? static_cast<const unsigned char*>(a.res) + (live ? row : 0) * row_bytes : nullptr;
    live_i = live;
    nlive_i = __popc(__ballot_sync(0xffffffffu, live));
  };
  auto issue_chunk = [&]() {
    const int stage = static_cast<int>(g_i % static_cast<uint32_t>(D));
    const int vecs = min(kChunkVecs, V - kChunkVecs * chunk_i);
    const uint32_t bytes = static_cast<uint32_t>(vecs) * 16u;
    if (lane == 0) mbar_expect_tx(&sm.bars[stage], static_cast<uint32_t>(nlive_i) * bytes * (RES ? 2u : 1u) + a.wt.extra_tx);
    if (live_i) {
      const size_t slot = (static_cast<size_t>(stage) * TR + lane) * kChunkPitch;
      const size_t off = static_cast<size_t>(chunk_i) * kChunkVecs * 16;
      bulk_g2s(sm.xring + slot, xs_i + off, bytes, &sm.bars[stage]);
      if (RES) bulk_g2s(sm.rring + slot, rs_i + off, bytes, &sm.bars[stage]);
    }
    ++g_i;
    if (++chunk_i == nc) {
      chunk_i = 0;
      tile_i += stride;
      ++it_i;
      if (tile_i < tiles) open_tile();
    }
  };

  if (warp == 0) {
    open_tile();
    while (g_i < static_cast<uint32_t>(D) && tile_i < tiles && it_i <= 1) issue_chunk();
  }

  int it = 0;
  int64_t tile = blockIdx.x;
  for (; tile < tiles; tile += stride, ++it) {
    if (warp == 0) {
      // ---- pass 1 of tile `tile`: strictly sequential f32 accumulation, one lane per row ----
      const bool live = sm.src[(it & 3) * 32 + lane] >= 0;
      float s = 0.0f, s2 = 0.0f;
      bool ok = true;
      for (int c = 0; c < nc && ok; ++c) {
        const int stage = static_cast<int>(g_c % static_cast<uint32_t>(D));
        ok = __all_sync(0xffffffffu, mbar_wait(&sm.bars[stage], (g_c / static_cast<uint32_t>(D)) & 1u, a.wt.spins));
        if (!ok) break;
        const int cnt = min(kChunkVecs, V - kChunkVecs * c);
        if (live) {
          const size_t slot = (static_cast<size_t>(stage) * TR + lane) * kChunkPitch;
          const uint4* xq = reinterpret_cast<const uint4*>(sm.xring + slot);
          const uint4* rq = reinterpret_cast<const uint4*>(sm.rring + slot);
          auto fetch = [&](int v) -> uint4 {
            uint4 hv = xq[v];  // v may run past cnt inside the padded slot; such vectors are not used
            if (RES) {
              if constexpr (DT == kDtF32) {
                float fa[PV], fb[PV];
                vec_to_floats<DT>(hv, fa);
                vec_to_floats<DT>(rq[v], fb);
#pragma unroll
                for (int e = 0; e < PV; ++e) fa[e] = __fadd_rn(fa[e], fb[e]);
                hv = floats_to_vec<DT>(fa);
              } else {
                hv = add_round_vec<DT>(hv, rq[v]);  // rounds the sum to T, as Tensor::add does
              }
            }
            return hv;
          };
          auto add_vec = [&](const uint4& hv) {
            float f[PV];
            vec_to_floats<DT>(hv, f);
#pragma unroll
            for (int e = 0; e < PV; ++e) {
              if (OP == kOpLayerNorm) s = __fadd_rn(s, f[e]);
              // for 16-bit inputs f*f is exact in f32, so the fused form rounds like add(s2, mul(f, f))
              s2 = (DT == kDtF32) ? __fadd_rn(s2, __fmul_rn(f[e], f[e])) : fmaf(f[e], f[e], s2);
            }
          };
          // Groups of G vectors, two per trip: while one register set is accumulated the other is
          // being fetched, and the sets swap roles instead of being copied (the copies cost issue
          // slots the chain needs).  A fetch past the chunk wraps to vector 0 and is not used.
          const int groups = cnt / G;
          auto load_group = [&](uint4 (&dst)[G], int g) {
            const int v = g * G < kChunkVecs ? g * G : 0;
#pragma unroll
            for (int q = 0; q < G; ++q) dst[q] = fetch(v + q);
          };
          uint4 ga[G], gb[G];
          load_group(ga, 0);
          int g = 0;
#pragma unroll 1
          for (; g + 1 < groups; g += 2) {
            load_group(gb, g + 1);
#pragma unroll
            for (int q = 0; q < G; ++q) add_vec(ga[q]);
            load_group(ga, g + 2);
#pragma unroll
            for (int q = 0; q < G; ++q) add_vec(gb[q]);
          }
          // ga holds group g here: the last whole group when their number is odd, else the ragged tail
          if (g < groups) {
            load_group(gb, g + 1);
#pragma unroll
            for (int q = 0; q < G; ++q) add_vec(ga[q]);
#pragma unroll
            for (int q = 0; q < G; ++q)
              if (groups * G + q < cnt) add_vec(gb[q]);
          } else {
#pragma unroll
            for (int q = 0; q < G; ++q)
              if (groups * G + q < cnt) add_vec(ga[q]);
          }
        }
        __syncwarp();
        ++g_c;
        // refill: keep the copy stream D chunks ahead, at most into the next tile
        while (g_i - g_c < static_cast<uint32_t>(D) && tile_i < tiles && it_i <= it + 1) issue_chunk();
      }
      if (!ok) {
        if (lane == 0) {
          report_status(a.status, CB200_STATUS_WAIT_TIMEOUT, tile * TR, 0, a.vocab);
          *sm.abort_flag = 1;
        }
      } else if (live) {
        sm.stats[(it & 1) * 32 + lane] = make_float2(s, s2);
      }
    } else if (is_finisher && it > 0) {
      finish_tile(tile - stride, it - 1, finisher, kStreamFinishers);
    }
    __syncthreads();
    if (*sm.abort_flag) {
      // bounded second chance for the copies still in flight before the CTA retires
      if (warp == 0) {
        for (uint32_t g = g_c; g != g_i; ++g)
          mbar_wait(&sm.bars[g % static_cast<uint32_t>(D)], (g / static_cast<uint32_t>(D)) & 1u, a.wt.spins);
        drain_pause();
      }
      return;
    }
  }
  if (it > 0) finish_tile(tile - stride, it - 1, warp, kStreamWarps);  // nothing left to walk: all warps
}

// ---------------------------------------------------------------------------------------------
// Any-shape fallback: one thread per row, scalar accesses, same arithmetic and order.  Used for
// rows that are not 16-byte multiples, misaligned bases, and rows too long for shared memory.
// ---------------------------------------------------------------------------------------------
template <int DT, int OP>
__global__ void norm_generic_kernel(const LaneRowArgs a) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= a.rows) return;
  int64_t src_row = row;
  if (a.ids != nullptr) {
    uint64_t id = read_id(a.ids, a.id_dtype, row);
    if (id >= static_cast<uint64_t>(a.vocab)) {
      report_status(a.status, CB200_STATUS_INVALID_INDEX, row, static_cast<int64_t>(id), a.vocab);
      return;
    }
    src_row = static_cast<int64_t>(id);
  }
  const int64_t xo = src_row * a.n, ro = row * a.n;
  const bool has_res = a.ids == nullptr && a.res != nullptr;
  float s = 0.0f, s2 = 0.0f;
  for (int c = 0; c < a.n; ++c) {
    float h = load_elem<DT>(a.x, xo + c);
    if (has_res) h = round_to<DT>(__fadd_rn(h, load_elem<DT>(a.res, ro + c)));
    if (OP == kOpLayerNorm) s = __fadd_rn(s, h);
    s2 = __fadd_rn(s2, __fmul_rn(h, h));
  }
  const float nf = static_cast<float>(a.n);
  float mean = 0.0f, scale;
  if (OP == kOpLayerNorm) {
    mean = __fdiv_rn(s, nf);
    float var = __fsub_rn(__fdiv_rn(s2, nf), __fmul_rn(mean, mean));
    scale = __frcp_rn(__fsqrt_rn(__fadd_rn(var, a.eps)));
  } else {
    scale = round_to<DT>(rms_from_sum(s2, nf, a.eps));
  }
  for (int c = 0; c < a.n; ++c) {
    float h = load_elem<DT>(a.x, xo + c);
    if (has_res) h = round_to<DT>(__fadd_rn(h, load_elem<DT>(a.res, ro + c)));
    float g = load_elem<DT>(a.alpha, c);
    float o;
    if (OP == kOpLayerNorm)
      o = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(h, mean), scale), g), load_elem<DT>(a.beta, c));
    else
      o = __fmul_rn(round_to<DT>(__fdiv_rn(h, scale)), g);
    store_elem<DT>(a.y, ro + c, o);
    if (a.sum_out != nullptr) store_elem<DT>(a.sum_out, ro + c, h);
  }
}

// ---------------------------------------------------------------------------------------------
// Launchers
// ---------------------------------------------------------------------------------------------
constexpr size_t kMaxDynSmem = 227 * 1024;

static size_t lanerow_smem(int R, int pitch) {
  return static_cast<size_t>(R) * pitch + static_cast<size_t>(R) * 8 + static_cast<size_t>(R + (R & 1)) * 4 + 16;
}

bool norm_lanerow_supported(int dtype, int cols) {
  int esz = dtype == kDtF32 ? 4 : 2;
  int64_t row_bytes = static_cast<int64_t>(cols) * esz;
  if (cols <= 0 || row_bytes % 16 != 0) return false;
  if (row_bytes >= 512) return true;  // streamed: any length
  return lanerow_smem(1, static_cast<int>(row_bytes) + 16) <= kMaxDynSmem;
}

template <int DT, int OP>
static cudaError_t launch_lanerow_t(LaneRowArgs a, cudaStream_t stream) {
  const int row_bytes = a.n * Elem<DT>::kBytes;
  a.wt = wait_tuning();
  a.V = row_bytes / 16;
  a.pitch = row_bytes + ((a.V & 1) ? 0 : 16);
  // rows per CTA: up to a warp's worth, sized so that several CTAs fit in an SM's shared memory
  // (their load / chain / store phases overlap), and small enough that small problems still
  // spread over all SMs
  int R = static_cast<int>((28 * 1024) / a.pitch);  // short rows: about eight CTAs per SM
  if (R < 4) R = static_cast<int>((72 * 1024) / a.pitch);  // long rows: about three
  if (R > 32) R = 32;
  if (R < 1) R = 1;
  const int sms = sm_count();
  int64_t spread = (a.rows + 2 * sms - 1) / (2 * sms);
  if (R > spread) R = static_cast<int>(spread);
  a.R = R;
  size_t smem = lanerow_smem(R, a.pitch);
  auto kern = norm_lanerow_kernel<DT, OP>;
  cudaError_t e = kernel_launch_config(reinterpret_cast<const void*>(kern), kLaneRowThreads, smem, -1, nullptr);
  if (e != cudaSuccess) return e;
  int64_t grid = (a.rows + R - 1) / R;
  kern<<<static_cast<unsigned>(grid), kLaneRowThreads, smem, stream>>>(a);
  return cudaGetLastError();
}

// Rows per tile for a persistent one-CTA-per-SM kernel: the smallest tile that still needs no more
// rounds over the SMs than tiles of `max_rows` would, so that every SM gets the same number of rows
// (16384 rows: 4 rounds of 28 rows instead of 4 of 32 on some SMs and 3 on the others).
static int balanced_tile_rows(int64_t rows, int max_rows) {
  const int sms = sm_count();
  const int64_t per_round = static_cast<int64_t>(max_rows) * sms;
  const int64_t rounds = (rows + per_round - 1) / per_round;
  int64_t tr = (rows + rounds * sms - 1) / (rounds * sms);
  if (tr > max_rows) tr = max_rows;
  if (tr < 1) tr = 1;
  return static_cast<int>(tr);
}

template <int DT, int OP, int VPL>
static cudaError_t launch_shortrow_t(const LaneRowArgs& a, cudaStream_t stream) {
  constexpr int TR = ShortTile<VPL>::kRows;
  const size_t smem = static_cast<size_t>(4) * TR * (32 * VPL + 1) * 16 + 2 * TR * sizeof(float2);
  auto kern = norm_shortrow_kernel<DT, OP, VPL>;
  cudaError_t e = kernel_launch_config(reinterpret_cast<const void*>(kern), kShortThreads, smem,
                                       static_cast<int>((smem + 1024) * 100 / (228 * 1024) + 1), nullptr);
  if (e != cudaSuccess) return e;
  const int tile_rows = balanced_tile_rows(a.rows, TR);
  int64_t tiles = (a.rows + tile_rows - 1) / tile_rows;
  const int sms = sm_count();
  int64_t grid = tiles < sms ? tiles : sms;
  kern<<<static_cast<unsigned>(grid), kShortThreads, smem, stream>>>(a, tile_rows);
  return cudaGetLastError();
}

// Rows of exactly 32, 64, 96 or 128 vectors, dense source, enough rows to fill the device.
static bool shortrow_applies(int dtype, const LaneRowArgs& a) {
  const int esz = dtype == kDtF32 ? 4 : 2;
  const int64_t row_bytes = static_cast<int64_t>(a.n) * esz;
  return a.ids == nullptr && row_bytes % 512 == 0 && row_bytes / 512 >= 1 && row_bytes / 512 <= 4 &&
         a.rows >= 2 * 32 * sm_count();
}

template <int DT, int OP>
static cudaError_t launch_shortrow_dt(const LaneRowArgs& a, cudaStream_t stream) {
  switch (a.n * Elem<DT>::kBytes / 512) {
    case 1:
      return launch_shortrow_t<DT, OP, 1>(a, stream);
    case 2:
      return launch_shortrow_t<DT, OP, 2>(a, stream);
    case 3:
      return launch_shortrow_t<DT, OP, 3>(a, stream);
    default:
      return launch_shortrow_t<DT, OP, 4>(a, stream);
  }
}

// Rows per tile, ring depth and grid of the streaming kernel.  Problems with fewer rows than the
// device has row slots get smaller tiles, so that every SM has one.
static void stream_shape(int64_t rows, bool res, int& TR, int& D, int& CV, int64_t& grid) {
  TR = balanced_tile_rows(rows, 32);
  // 2 KB per copy: the copy engine takes about 35 ns per copy whatever its size, and one warp's
  // copies deliver an SM's share of HBM only from that size on.  The ring is kept to 135 KB: what
  // shared memory does not take stays L1, which bounds the loads pass 2 can have in flight.
  CV = 128;
  const int budget = 135;
  const size_t stage = static_cast<size_t>(TR) * stream_chunk_pitch(CV) * (res ? 2 : 1);
  D = static_cast<int>((budget * 1024) / stage);
  if (D < 1) D = 1;
  if (D > kStreamMaxStages) D = kStreamMaxStages;
  const int64_t tiles = (rows + TR - 1) / TR;
  const int sms = sm_count();
  grid = tiles < sms ? tiles : sms;
}

static bool stream_applies(int dtype, const LaneRowArgs& a) {
  const int esz = dtype == kDtF32 ? 4 : 2;
  const int64_t row_bytes = static_cast<int64_t>(a.n) * esz;
  const bool fits_whole = lanerow_smem(1, static_cast<int>(row_bytes) + 16) <= kMaxDynSmem;
  return (!a.classic || !fits_whole) && row_bytes % 16 == 0 && row_bytes >= 512;
}

template <int DT, int OP, bool RES>
static cudaError_t launch_stream_r(LaneRowArgs a, cudaStream_t stream) {
  a.V = a.n * Elem<DT>::kBytes / 16;
  a.wt = wait_tuning();
  int TR, D, CV;
  int64_t grid;
  stream_shape(a.rows, RES, TR, D, CV, grid);
  const size_t smem = StreamSmem::bytes(TR, D, CV, RES);
  auto kern = norm_stream_kernel<DT, OP, RES>;
  int percent = static_cast<int>((smem + 1024) * 100 / (228 * 1024) + 1);
  if (percent > 100) percent = 100;
  cudaError_t e = kernel_launch_config(reinterpret_cast<const void*>(kern), kStreamThreads, smem, percent, nullptr);
  if (e != cudaSuccess) return e;
  kern<<<static_cast<unsigned>(grid), kStreamThreads, smem, stream>>>(a, TR, D, CV);
  return cudaGetLastError();
}

template <int DT, int OP>
static cudaError_t launch_stream_t(const LaneRowArgs& a, cudaStream_t stream) {
  return (a.ids == nullptr && a.res != nullptr) ? launch_stream_r<DT, OP, true>(a, stream)
                                                : launch_stream_r<DT, OP, false>(a, stream);
}

template <int DT, int OP>
static cudaError_t launch_generic_t(const LaneRowArgs& a, cudaStream_t stream) {
  const int threads = 64;
  int64_t grid = (a.rows + threads - 1) / threads;
  norm_generic_kernel<DT, OP><<<static_cast<unsigned>(grid), threads, 0, stream>>>(a);
  return cudaGetLastError();
}

template <int OP>
static cudaError_t dispatch_dt(int dtype, bool generic, const LaneRowArgs& a, cudaStream_t stream) {
  if (!generic && shortrow_applies(dtype, a)) {
    switch (dtype) {
      case kDtF32:
        return launch_shortrow_dt<kDtF32, OP>(a, stream);
      case kDtF16:
        return launch_shortrow_dt<kDtF16, OP>(a, stream);
      default:
        return launch_shortrow_dt<kDtBF16, OP>(a, stream);
    }
  }
  if (!generic && stream_applies(dtype, a)) {
    switch (dtype) {
      case kDtF32:
        return launch_stream_t<kDtF32, OP>(a, stream);
      case kDtF16:
        return launch_stream_t<kDtF16, OP>(a, stream);
      default:
        return launch_stream_t<kDtBF16, OP>(a, stream);
    }
  }
  switch (dtype) {
    case kDtF32:
      return generic ? launch_generic_t<kDtF32, OP>(a, stream) : launch_lanerow_t<kDtF32, OP>(a, stream);
    case kDtF16:
      return generic ? launch_generic_t<kDtF16, OP>(a, stream) : launch_lanerow_t<kDtF16, OP>(a, stream);
    default:
      return generic ? launch_generic_t<kDtBF16, OP>(a, stream) : launch_lanerow_t<kDtBF16, OP>(a, stream);
  }
}

cudaError_t launch_norm_lanerow(int dtype, int op, const LaneRowArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  return op == kOpLayerNorm ? dispatch_dt<kOpLayerNorm>(dtype, false, a, stream)
                            : dispatch_dt<kOpRmsNorm>(dtype, false, a, stream);
}

cudaError_t launch_norm_generic(int dtype, int op, const LaneRowArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  return op == kOpLayerNorm ? dispatch_dt<kOpLayerNorm>(dtype, true, a, stream)
                            : dispatch_dt<kOpRmsNorm>(dtype, true, a, stream);
}

}  // namespace cb200
