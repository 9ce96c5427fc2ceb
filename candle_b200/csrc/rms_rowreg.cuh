// Register-resident RMS norm for 16-bit element types (bf16 / f16).
//
// One row is spread over `tpr` threads (a warp up to 512 threads), each holding up to VPT 16-byte
// vectors of the row in registers, so the row is read from HBM exactly once.
//
// Bit-exactness with candle's CPU path (candle-nn/src/ops.rs:484-495) needs the row's sum of
// squares in strictly sequential f32 order, which a parallel reduction cannot give directly.
// But the CPU path rounds m = sqrt(sum/n + eps) to the 16-bit type before using it, so all that
// matters is T(m).  The kernel therefore
//   1. reduces sum(p_j) and W = sum(p_j * (n - j)) in tree order (p_j = h_j^2 is exact in f32
//      for 16-bit h_j),
//   2. bounds the sequential result rigorously: with u = 2^-24, |seq - exact| <= u(1+g) * W
//      (each of the n-1 additions errs by at most u times its partial sum, and the partial sums
//      add up to at most W) and |tree - exact| <= 128u * exact,
//   3. evaluates candle's f32 pipeline (all of it monotone) at both ends of the interval; if
//      T(m) agrees at both ends it IS the sequential answer,
//   4. otherwise (a few percent of rows at 8192 columns) replays the row from shared memory in
//      sequential order with one thread.
// The division x / m rounded to bf16 is evaluated as bf16(x * (1/m)): a quotient of two 8-bit
// significands is never closer than 2^-17 (relative) to a bf16 rounding boundary, far more than
// the 2^-22 error of the reciprocal product, so both round identically.  f16 has no such margin
// and uses the correctly rounded division.
#pragma once

#include "common.cuh"

namespace cb200 {

struct RmsRowRegArgs {
  const uint4* x;      // [rows, V] vectors, or the dense table [vocab, V] when ids != nullptr
  const uint4* res;    // optional residual [rows, V]
  const uint4* alpha;  // [V]
  uint4* y;            // [rows, V]
  uint4* sum_out;      // optional: h = x + res (or the gathered rows)
  const void* ids;     // optional row ids into x
  int id_dtype;
  int64_t vocab;
  cb200_status* status;
  int64_t rows;
  int V;  // 16-byte vectors per row = cols / 8
  int n;  // cols
  float eps;
  int flags;
};

// Arguments of the kernel whose rows come out of a Q4_0 / Q8_0 table.
struct QRmsArgs {
  const unsigned char* qtable;  // rows [vocab_begin, vocab_end) of the table
  const void* ids;
  const uint4* alpha;
  uint4* y;
  uint4* gathered;  // optional decoded rows
  int id_dtype;
  int64_t vocab, vocab_begin, vocab_end;
  cb200_status* status;
  int64_t rows;
  int V, n;
  int row_bytes;  // bytes of one quantised row
  int bulk;       // 1: rows are 16-byte multiples and the table is 16-byte aligned
  float eps;
  int flags;
};

// Shared-memory layout of one CTA of the row-register kernels.
struct RowRegSmem {
  float* red;    // [rpc][2][16] warp partials
  float* mslot;  // [rpc] resolved T(m) of replayed rows
  uint4* rows;   // [rpc][V] row replay buffers
  __device__ RowRegSmem(unsigned char* base, int rpc, int V, int ty) {
    red = reinterpret_cast<float*>(base) + ty * 32;
    mslot = reinterpret_cast<float*>(base) + rpc * 32 + ty;
    size_t off = (static_cast<size_t>(rpc) * 33 * sizeof(float) + 15) & ~static_cast<size_t>(15);
    rows = reinterpret_cast<uint4*>(base + off) + static_cast<size_t>(ty) * V;
  }
  __host__ __device__ static size_t bytes(int rpc, int V, bool with_rows) {
    size_t off = (static_cast<size_t>(rpc) * 33 * sizeof(float) + 15) & ~static_cast<size_t>(15);
    return off + (with_rows ? static_cast<size_t>(rpc) * V * 16 : 0);
  }
};

template <int DT>
__device__ __forceinline__ void accumulate_vec(const uint4& h, int first_col, int n, float& lsum, float& lw) {
  const uint32_t w[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = unpack2<DT>(w[i]);
    float p0 = __fmul_rn(f.x, f.x), p1 = __fmul_rn(f.y, f.y);
    lsum += p0;
    lsum += p1;
    lw = fmaf(p0, static_cast<float>(n - (first_col + 2 * i)), lw);
    lw = fmaf(p1, static_cast<float>(n - (first_col + 2 * i + 1)), lw);
  }
}

// Sequential replay of one row held in shared memory (candle's summation order).
template <int DT>
__device__ __forceinline__ float sequential_sum_sq(const uint4* row, int V) {
  float s = 0.0f;
#pragma unroll 4
  for (int v = 0; v < V; ++v) {
    uint4 q = row[v];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = unpack2<DT>(w[i]);
      s = __fadd_rn(s, __fmul_rn(f.x, f.x));
      s = __fadd_rn(s, __fmul_rn(f.y, f.y));
    }
  }
  return s;
}

// Resolves T(m) for the row held in h[] by the tpr threads of row slot ty.  Every thread of the
// CTA must call it (it contains CTA-wide barriers); `live` rows only matter for the result.
template <int DT, int VPT>
__device__ __forceinline__ float resolve_row_m(const uint4 (&h)[VPT], float lsum, float lw, int V, int n,
                                               float eps, int flags, RowRegSmem& sm) {
  const int tx = threadIdx.x, tpr = blockDim.x;
  const int lane = tx & 31, warp = tx >> 5, wpr = tpr >> 5;
  float s = warp_sum(lsum), w = warp_sum(lw);
  if (wpr > 1) {
    if (lane == 0) {
      sm.red[warp] = s;
      sm.red[16 + warp] = w;
    }
    __syncthreads();
    s = 0.0f;
    w = 0.0f;
    for (int i = 0; i < wpr; ++i) {  // fixed order: every thread of the row gets the same bits
      s += sm.red[i];
      w += sm.red[16 + i];
    }
  }
  const float nf = static_cast<float>(n);
  if (flags & CB200_FLAG_FAST_SUM) return round_to<DT>(rms_from_sum(s, nf, eps));

  constexpr float kU = 5.9604644775390625e-8f;  // 2^-24
  // |seq - tree| <= 1.01*u*W + 160*u*s covers both bounds and the f32 rounding of w and of
  // this expression itself.
  const float err = 1.01f * kU * w + 160.0f * kU * s;
  const float m_lo = round_to<DT>(rms_from_sum(s - err, nf, eps));
  const float m_hi = round_to<DT>(rms_from_sum(s + err, nf, eps));
  const bool replay = !(m_lo == m_hi);  // also true when anything is NaN
  float m = m_lo;
  if (__syncthreads_or(replay ? 1 : 0)) {
    if (replay) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        int v = k * tpr + tx;
        if (v < V) sm.rows[v] = h[k];
      }
    }
    __syncthreads();
    if (replay && tx == 0) *sm.mslot = round_to<DT>(rms_from_sum(sequential_sum_sq<DT>(sm.rows, V), nf, eps));
    __syncthreads();
    if (replay) m = *sm.mslot;
  }
  return m;
}

// y = T(T(h / m) * alpha) for the vectors this thread holds.
template <int DT, int VPT>
__device__ __forceinline__ void write_rms_row(const uint4 (&h)[VPT], float m, const uint4* __restrict__ alpha,
                                              uint4* __restrict__ yrow, int V) {
  const int tx = threadIdx.x, tpr = blockDim.x;
  // 2^-60 <= m <= 2^60: the reciprocal is a normal number and the margin argument applies.
  const bool fast_div = (DT == kDtBF16) && (m >= 8.6736174e-19f) && (m <= 1.1529215e18f);
  const float r = fast_div ? __frcp_rn(m) : 0.0f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    int v = k * tpr + tx;
    if (v >= V) continue;
    uint4 av = __ldg(alpha + v);
    const uint32_t hw[4] = {h[k].x, h[k].y, h[k].z, h[k].w};
    const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
    uint32_t ow[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 hf = unpack2<DT>(hw[i]);
      float2 af = unpack2<DT>(aw[i]);
      float q0, q1;
      if (fast_div) {
        q0 = __fmul_rn(hf.x, r);
        q1 = __fmul_rn(hf.y, r);
        // below 2^-100 the bf16 result may be subnormal: use the exact quotient there
        if (fabsf(q0) < 7.8886091e-31f && q0 != 0.0f) q0 = __fdiv_rn(hf.x, m);
        if (fabsf(q1) < 7.8886091e-31f && q1 != 0.0f) q1 = __fdiv_rn(hf.y, m);
      } else {
        q0 = __fdiv_rn(hf.x, m);
        q1 = __fdiv_rn(hf.y, m);
      }
      q0 = round_to<DT>(q0);
      q1 = round_to<DT>(q1);
      ow[i] = pack2<DT>(__fmul_rn(q0, af.x), __fmul_rn(q1, af.y));
    }
    stg_stream(yrow + v, make_uint4(ow[0], ow[1], ow[2], ow[3]));
  }
}

// h = T(x + res) for one vector.
template <int DT>
__device__ __forceinline__ uint4 add_round_vec(const uint4& a, const uint4& b) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
  const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
  uint32_t ow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 fa = unpack2<DT>(aw[i]);
    float2 fb = unpack2<DT>(bw[i]);
    ow[i] = pack2<DT>(__fadd_rn(fa.x, fb.x), __fadd_rn(fa.y, fb.y));
  }
  return make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

}  // namespace cb200
