// The norm's neighbours in a transformer block: softmax over the last dimension and the rotary
// embeddings, with the arithmetic of candle's CPU backend.
//
// softmax_last_dim (candle-nn/src/ops.rs:296-333), per row and entirely in T:
//   max = max(row); e[i] = exp(x[i] - max); sum = vec_reduce_sum(e); y[i] = e[i] / sum
// * f32: the sum is candle's AVX-ordered vec_sum (candle-core/src/cpu/mod.rs:113-135, cpu/avx.rs:54-66:
//   32 partial sums, partial l over elements l, l + 32, ..., folded over distances 8, 16, 4, 1, 2, then
//   the n % 32 leftovers one by one), which is exactly a warp with one partial per lane.  exp is
//   evaluated in double precision and rounded once, i.e. the correctly rounded f32 value; candle calls
//   the platform's expf, which glibc documents as correctly rounded in all but rare cases.
// * f16 / bf16: vec_reduce_sum is the default `*res += x` -- one T-rounded addition per element, in
//   order (candle-core/src/cpu/kernels.rs:26-31).  A chain like that cannot be split, so rows are
//   staged in shared memory and one LANE walks one row (32 rows side by side per warp) with the
//   T-rounded packed add instruction, one dependent instruction per element.  exp(v) for a T value is
//   T(expf(f32(v))): the kernel brackets expf between (1 -+ 2^-20) times the device's expf -- both
//   libm's and the true value lie inside -- and where both ends round to the same T that is the
//   answer; the rare other elements take the double-precision exp.
//
// rope_i / rope / rope_thd (candle-nn/src/rotary_emb.rs:47-60, 288-305, 540-558), all in T with each
// product and the final sum / difference rounded separately:
//   y1 = x1 * cos - x2 * sin,  y2 = x1 * sin + x2 * cos
#include "launch.h"
#include "rms_rowreg.cuh"

namespace cb200 {

namespace {

// ---------------------------------------------------------------------------------------------
// softmax, f32: one warp per row
// ---------------------------------------------------------------------------------------------
constexpr int kSoftmaxThreads = 256;

__device__ __forceinline__ float avx_fold(float v) {
  v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 8));
  v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 16));
  v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 4));
  v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 1));
  v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 2));
  return v;
}

// f32::max / half's max: a NaN operand is ignored
__device__ __forceinline__ float max_ignoring_nan(float a, float b) { return fmaxf(a, b); }

// exp(v) rounded once to f32.  Below -104 the value is under half the smallest subnormal: +0.
__device__ __forceinline__ float exp_correctly_rounded(float v) {
  if (v < -104.0f) return 0.0f;
  return static_cast<float>(exp(static_cast<double>(v)));
}

// exp(v) rounded once to f32 at a fraction of the cost of the library's double-precision exp, for the
// arguments a softmax produces (v = x - max <= 0, results in the normal f32 range):
//   v = k ln2/32 + r, |r| <= ln2/64;  exp(v) = 2^(k >> 5) * 2^((k & 31)/32) * exp(r)
// in double precision with a 32-entry table of 2^(j/32) (shared memory, filled by the CTA) and a
// degree-5 polynomial for exp(r) - 1 (truncation 2^-48.7).  The double result is good to well under
// 2^-46, so rounding it to f32 gives the correctly rounded value unless its 29 discarded fraction
// bits lie within 2^-42 (relative) of the half-way pattern; those arguments (about 4 in a million) and
// everything outside [-87, 88] -- subnormal results, NaN -- take the library path.
struct ExpTable {
  const double* pow2;  // [32] 2^(j/32)
};
__device__ __forceinline__ void fill_exp_table(double* table) {
  if (threadIdx.x < 32) table[threadIdx.x] = exp2(static_cast<double>(threadIdx.x) * 0.03125);
}
__device__ __forceinline__ float exp_rounded_once(float v, const ExpTable& tab) {
  if (!(v >= -87.0f && v <= 88.0f)) return exp_correctly_rounded(v);
  const double x = static_cast<double>(v);
  constexpr double kShift = 6755399441055744.0;  // 1.5 * 2^52: adding it leaves round(t) in the low word
  const double t = fma(x, 0x1.71547652b82fep+5, kShift);
  const int k = __double2loint(t);
  const double kd = t - kShift;
  double r = fma(kd, -0x1.62e42fefa3000p-6, x);  // ln2/32, 41 significant bits: the product is exact
  r = fma(kd, -0x1.3de6af278ece6p-47, r);
  double p = fma(r, 1.0 / 120.0, 1.0 / 24.0);
  p = fma(p, r, 1.0 / 6.0);
  p = fma(p, r, 0.5);
  p = fma(p * r, r, r);  // exp(r) - 1
  const double T = tab.pow2[k & 31];
  const double d = fma(T, p, T);
  const long long bits = __double_as_longlong(d) + (static_cast<long long>(k >> 5) << 52);
  const int low = static_cast<int>(static_cast<unsigned>(bits) & 0x1FFFFFFFu);  // the 29 bits f32 drops
  if (abs(low - (1 << 28)) < 1024) return exp_correctly_rounded(v);
  return static_cast<float>(__longlong_as_double(bits));
}

// Rows that are whole 16-byte vectors: a warp per row, the row staged in the warp's own shared-memory
// buffer (16-byte global accesses only, all loads of a row in flight at once); max, exp + AVX-order sum
// and the division run on shared memory with lane l on elements l, l + 32, ...
constexpr int kSoftmaxStagedMaxWarps = 24;
__global__ void __launch_bounds__(kSoftmaxStagedMaxWarps * 32) softmax_f32_staged_kernel(const uint4* __restrict__ x,
                                                                                        uint4* __restrict__ y,
                                                                                        int64_t rows, int n, int pitch) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* table = reinterpret_cast<double*>(smem_raw);
  fill_exp_table(table);
  __syncthreads();
  const ExpTable tab{table};
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, warps = blockDim.x >> 5;
  float* buf = reinterpret_cast<float*>(smem_raw + 256 + static_cast<size_t>(wib) * pitch);
  uint4* bufv = reinterpret_cast<uint4*>(buf);
  const int V = n / 4;
  const int np = n & ~31;
  constexpr int U = 8;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * warps + wib; row < rows;
       row += static_cast<int64_t>(gridDim.x) * warps) {
    const uint4* xr = x + row * V;
    float m = __int_as_float(0xff800000);  // -inf; every row has at least one element
    for (int v0 = lane; v0 < V; v0 += 32 * U) {
      uint4 q[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (v0 + 32 * u < V) q[u] = ldg_stream(xr + v0 + 32 * u);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (v0 + 32 * u < V) {
          bufv[v0 + 32 * u] = q[u];
          m = max_ignoring_nan(m, max_ignoring_nan(max_ignoring_nan(__uint_as_float(q[u].x), __uint_as_float(q[u].y)),
                                                   max_ignoring_nan(__uint_as_float(q[u].z), __uint_as_float(q[u].w))));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max_ignoring_nan(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    __syncwarp();
    float acc = 0.0f;
#pragma unroll 2
    for (int i = lane; i < np; i += 32) {
      const float e = exp_rounded_once(__fsub_rn(buf[i], m), tab);
      buf[i] = e;
      acc = __fadd_rn(acc, e);
    }
    float sum = avx_fold(acc);
    float tail = 0.0f;
    if (np + lane < n) {
      tail = exp_rounded_once(__fsub_rn(buf[np + lane], m), tab);
      buf[np + lane] = tail;
    }
    for (int i = 0; i < n - np; ++i) sum = __fadd_rn(sum, __shfl_sync(0xFFFFFFFFu, tail, i));
    __syncwarp();
    // the division has no order to keep: 16 bytes per lane, exact three-instruction division by the sum
    const RowDivisor dv = make_row_divisor(sum);
    uint4* yr = y + row * V;
#pragma unroll 2
    for (int v = lane; v < V; v += 32) {
      const uint4 q = bufv[v];
      stg_stream(yr + v, make_uint4(__float_as_uint(div_by_row(__uint_as_float(q.x), dv)),
                                    __float_as_uint(div_by_row(__uint_as_float(q.y), dv)),
                                    __float_as_uint(div_by_row(__uint_as_float(q.z), dv)),
                                    __float_as_uint(div_by_row(__uint_as_float(q.w), dv))));
    }
    __syncwarp();  // the buffer is refilled by the next row's loads
  }
}

// Any row length and alignment: scalar accesses on global memory, the library's exp.
__global__ void __launch_bounds__(kSoftmaxThreads) softmax_f32_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                                      int64_t rows, int n) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int np = n & ~31;
  for (int64_t row = warp; row < rows; row += n_warps) {
    const float* xr = x + row * n;
    float* yr = y + row * n;
    float m = __int_as_float(0xff800000);  // -inf; every row has at least one element
    for (int i = lane; i < n; i += 32) m = max_ignoring_nan(m, xr[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max_ignoring_nan(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    float acc = 0.0f;
    for (int i = lane; i < np; i += 32) {
      const float e = exp_correctly_rounded(__fsub_rn(xr[i], m));
      yr[i] = e;
      acc = __fadd_rn(acc, e);
    }
    float sum = avx_fold(acc);
    float tail = 0.0f;
    if (np + lane < n) {
      tail = exp_correctly_rounded(__fsub_rn(xr[np + lane], m));
      yr[np + lane] = tail;
    }
    for (int i = 0; i < n - np; ++i) sum = __fadd_rn(sum, __shfl_sync(0xFFFFFFFFu, tail, i));
    // each lane re-reads what it wrote itself
    for (int i = lane; i < n; i += 32) yr[i] = __fdiv_rn(yr[i], sum);
  }
}

// ---------------------------------------------------------------------------------------------
// softmax, f16 / bf16
// ---------------------------------------------------------------------------------------------
// T(expf(v)) for a T value v, see the head of the file.
template <int DT>
__device__ __forceinline__ float exp_rounded_to(float v) {
  if (v < -104.0f) return 0.0f;
  const float e = expf(v);
  const float lo = round_to<DT>(__fmul_rn(e, 0.99999905f)), hi = round_to<DT>(__fmul_rn(e, 1.00000095f));
  if (lo == hi && e >= 1e-36f) return lo;  // (the relative bracket does not hold for subnormal results)
  return round_to<DT>(exp_correctly_rounded(v));
}

// one T-rounded addition: the packed instruction on (a, 0) + (b, 0)
template <int DT>
__device__ __forceinline__ uint32_t add_t(uint32_t a16, uint32_t b16) {
  return add2_rn<DT>(a16, b16) & 0xFFFFu;
}

template <int DT>
__device__ __forceinline__ float widen16(uint32_t h) {
  if constexpr (DT == kDtBF16)
    return __uint_as_float(h << 16);
  else
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}
template <int DT>
__device__ __forceinline__ uint32_t narrow16(float v) {
  if constexpr (DT == kDtBF16)
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  else
    return __half_as_ushort(__float2half_rn(v));
}

constexpr int kSoftmax16Threads = 256;

// s = T(T(s + lo(w)) + hi(w)): two T-rounded additions on 16-bit registers.  The halves of `w` are
// named, not extracted -- the add instruction selects the half of a 32-bit register it reads -- so
// the dependent chain is the two additions and nothing else.
template <int DT>
__device__ __forceinline__ void add_pair_t(unsigned short& s, uint32_t w) {
  if constexpr (DT == kDtBF16)
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; add.rn.bf16 %0, %0, lo; add.rn.bf16 %0, %0, hi; }" : "+h"(s) : "r"(w));
  else
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; add.rn.f16 %0, %0, lo; add.rn.f16 %0, %0, hi; }" : "+h"(s) : "r"(w));
}

// e = T(exp(v)) for v = T(x - max) <= 0 depends on the 16 bits of v only, and only a few thousand
// magnitudes give anything but 1 (tiny |v|) or 0 (|v| beyond the underflow point): a table over those
// magnitudes, filled once per CTA with exp_rounded_to, replaces the evaluation per element.
//   bf16: |v| <= 2^-10 gives 1 (exp(v) > 1 - 2^-9, the midpoint below 1); |v| >= 105 gives 0.
//   f16:  |v| <= 2^-13 gives 1 (midpoint 1 - 2^-12);                      |v| >= 17.5 gives 0 (< 2^-25).
// The first and the last entry are those two constants, so clamping the magnitude into the table's
// range is all the lookup needs; both halves of a word are clamped at once.
template <int DT>
struct ExpLut {
  static constexpr uint32_t kLo = DT == kDtBF16 ? 0x3A80u : 0x0800u;   // bit pattern of 2^-10 / 2^-13
  static constexpr uint32_t kHi = DT == kDtBF16 ? 0x42D2u : 0x4C60u;   // bit pattern of 105 / 17.5: the entry is 0
  static constexpr uint32_t kInf = DT == kDtBF16 ? 0x7F80u : 0x7C00u;
  static constexpr uint32_t kNan = DT == kDtBF16 ? 0x7FC0u : 0x7E00u;
  // results below this pattern (2^-116 / never for f16) can make e / sum subnormal in T
  static constexpr uint32_t kTiny = DT == kDtBF16 ? 0x0580u : 0x0000u;
  static constexpr int kEntries = static_cast<int>(kHi - kLo + 1);
  static constexpr int kBytes = (kEntries * 2 + 15) & ~15;
};

template <int DT>
__device__ __forceinline__ void fill_exp_lut(uint16_t* lut) {
  for (int i = threadIdx.x; i < ExpLut<DT>::kEntries; i += blockDim.x) {
    const float v = -widen16<DT>(ExpLut<DT>::kLo + static_cast<uint32_t>(i));
    lut[i] = static_cast<uint16_t>(narrow16<DT>(exp_rounded_to<DT>(v)));
  }
}

// (T(exp(lo)), T(exp(hi))) for the two 16-bit patterns in `v2`, each <= 0 (or NaN).
template <int DT>
__device__ __forceinline__ uint32_t exp_lookup2(uint32_t v2, const uint16_t* lut) {
  constexpr uint32_t kLo2 = ExpLut<DT>::kLo * 0x00010001u, kHi2 = ExpLut<DT>::kHi * 0x00010001u,
                     kInf2 = ExpLut<DT>::kInf * 0x00010001u;
  const uint32_t mag2 = v2 & 0x7FFF7FFFu;
  const uint32_t idx2 = __vsub2(__vminu2(__vmaxu2(mag2, kLo2), kHi2), kLo2);
  uint32_t e2 = static_cast<uint32_t>(lut[idx2 & 0xFFFFu]) | (static_cast<uint32_t>(lut[idx2 >> 16]) << 16);
  if (__vcmpgtu2(mag2, kInf2) != 0u) {  // a NaN in one of the halves
    if ((mag2 & 0xFFFFu) > ExpLut<DT>::kInf) e2 = (e2 & 0xFFFF0000u) | ExpLut<DT>::kNan;
    if ((mag2 >> 16) > ExpLut<DT>::kInf) e2 = (e2 & 0x0000FFFFu) | (ExpLut<DT>::kNan << 16);
  }
  return e2;
}

// Persistent CTAs, tiles of R rows of V 16-byte vectors staged in shared memory at a pitch of an odd
// number of 16-byte units.  Per tile:
//   1. a warp per row: load, max (any order), e = T(exp(T(x - max))) through the table, in place;
//   2. warp 0 walks the rows sequentially, one lane per row -- the T-rounded sum is a chain of
//      dependent additions, and nothing but the addition itself is on the chain;
//   3. a warp per row: y = T(e / sum), stored with 16-byte accesses.
// Several CTAs share an SM, so one CTA's walk overlaps the other CTAs' loads and stores.
// Rows a warp loads together in phase 1: up to 16 vectors per lane in flight, at most 4 rows (a tile
// has at most 32 rows for 8 warps).
__host__ __device__ constexpr int softmax16_rows_per_batch(int vpl) { return vpl <= 0 ? 1 : (16 / vpl > 4 ? 4 : 16 / vpl); }

// VPL: 16-byte vectors per lane and row (V <= 32 VPL; 1, 2, 4, 8 or 16), or 0 for longer rows.
template <int DT, int VPL>
__global__ void __launch_bounds__(kSoftmax16Threads, 3) softmax16_staged_kernel(const uint4* __restrict__ x,
                                                                             uint4* __restrict__ y, int64_t rows,
                                                                             int V, int R, int pitch_vecs) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint16_t* lut = reinterpret_cast<uint16_t*>(smem_raw);
  uint4* buf = reinterpret_cast<uint4*>(smem_raw + ExpLut<DT>::kBytes);
  uint32_t* sums = reinterpret_cast<uint32_t*>(buf + static_cast<size_t>(R) * pitch_vecs);  // [R]
  int* tiny = reinterpret_cast<int*>(sums + R);                                              // [R]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kWarps = kSoftmax16Threads / 32;
  fill_exp_lut<DT>(lut);
  __syncthreads();
  const int64_t tiles = (rows + R - 1) / R;
  // -max, then e = T(exp(T(x - max))) in place for row r of the tile, whose max is m
  auto exp_row = [&](int r, float m) {
    uint4* br = buf + static_cast<size_t>(r) * pitch_vecs;
    // -max in both halves; x - max = x + (-max), rounded once to T by the packed add.  (A row of NaNs
    // only keeps max = -inf: x + inf is NaN for them, as x - (-inf) is.)
    const uint32_t nm16 = narrow16<DT>(-m);
    const uint32_t nm2 = nm16 | (nm16 << 16);
    uint32_t least = 0xFFFFFFFFu;  // per half: the smallest e - 1 (mod 2^16) seen, i.e. the smallest non-zero e
    for (int v = lane; v < V; v += 32) {  // each lane re-reads the vectors it staged itself
      const uint4 q = br[v];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        o[i] = exp_lookup2<DT>(add2_rn<DT>(w[i], nm2), lut);
        if (DT == kDtBF16) least = __vminu2(least, __vsub2(o[i], 0x00010001u));
      }
      br[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    if constexpr (DT == kDtBF16) {
      uint32_t t = min(least & 0xFFFFu, least >> 16);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xFFFFFFFFu, t, o));
      // a non-zero e under 2^-116: e / sum may be subnormal in bf16, where only the division is safe
      if (lane == 0) tiny[r] = (t + 1u < ExpLut<DT>::kTiny) ? 1 : 0;
    }
  };
  auto vec_max = [&](const uint4& q, float m) -> float {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack2<DT>(w[i]);
      m = max_ignoring_nan(m, max_ignoring_nan(f.x, f.y));
    }
    return m;
  };
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t row0 = tile * R;
    const int live = static_cast<int>(min(static_cast<int64_t>(R), rows - row0));
    // ---- 1: load, max (any order), then e in place ----
    if constexpr (VPL > 0) {
      // a warp takes RB rows at a time and has all their loads in flight before it uses the first
      constexpr int RB = softmax16_rows_per_batch(VPL);
      for (int rbase = warp * RB; rbase < live; rbase += kWarps * RB) {
        uint4 q[RB * VPL];
#pragma unroll
        for (int ri = 0; ri < RB; ++ri)
#pragma unroll
          for (int u = 0; u < VPL; ++u) {
            const int r = rbase + ri, v = lane + 32 * u;
            q[ri * VPL + u] = (r < live && v < V) ? ldg_stream(x + (row0 + r) * V + v) : make_uint4(0, 0, 0, 0);
          }
        float m[RB];
#pragma unroll
        for (int ri = 0; ri < RB; ++ri) {
          m[ri] = __int_as_float(0xff800000);
#pragma unroll
          for (int u = 0; u < VPL; ++u) {
            const int r = rbase + ri, v = lane + 32 * u;
            if (r < live && v < V) {
              buf[static_cast<size_t>(r) * pitch_vecs + v] = q[ri * VPL + u];
              m[ri] = vec_max(q[ri * VPL + u], m[ri]);
            }
          }
        }
#pragma unroll
        for (int ri = 0; ri < RB; ++ri) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) m[ri] = max_ignoring_nan(m[ri], __shfl_xor_sync(0xFFFFFFFFu, m[ri], o));
          if (rbase + ri < live) exp_row(rbase + ri, m[ri]);  // (warp-uniform)
        }
      }
    } else {
      for (int r = warp; r < live; r += kWarps) {
        const uint4* xr = x + (row0 + r) * V;
        uint4* br = buf + static_cast<size_t>(r) * pitch_vecs;
        float m = __int_as_float(0xff800000);
        constexpr int U = 8;
        for (int v0 = lane; v0 < V; v0 += 32 * U) {
          uint4 q[U];
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (v0 + 32 * u < V) q[u] = ldg_stream(xr + v0 + 32 * u);
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (v0 + 32 * u >= V) continue;
            br[v0 + 32 * u] = q[u];
            m = vec_max(q[u], m);
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = max_ignoring_nan(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        exp_row(r, m);
      }
    }
    __syncthreads();
    // ---- 2: the T-rounded sums, candle's order ----
    if (warp == 0 && lane < live) {
      const uint4* pr = buf + static_cast<size_t>(lane) * pitch_vecs;
      unsigned short s16 = 0;  // +0 in T
#pragma unroll 4
      for (int v = 0; v < V; ++v) {
        const uint4 q = pr[v];
        add_pair_t<DT>(s16, q.x);
        add_pair_t<DT>(s16, q.y);
        add_pair_t<DT>(s16, q.z);
        add_pair_t<DT>(s16, q.w);
      }
      sums[lane] = s16;
    }
    __syncthreads();
    // ---- 3: y = T(e / sum) ----
    for (int r = warp; r < live; r += kWarps) {
      const float sum = widen16<DT>(sums[r]);
      const RowDivisor dv = make_row_divisor(sum);
      // e is 0 or at least the smallest T value and the sum lies in [1, 2^12]: no intermediate of the
      // three-instruction division can be subnormal (f16).  For bf16 the quotient of two 8-bit
      // significands is never within 2^-17 of a rounding boundary, so T(e * (1 / sum)) is T(e / sum)
      // wherever the result is a normal number -- rows with a tiny non-zero e divide instead.
      const bool quick = dv.fast && (DT == kDtF16 || tiny[r] == 0);
      const uint4* br = buf + static_cast<size_t>(r) * pitch_vecs;
      uint4* yr = y + (row0 + r) * V;
      for (int v = lane; v < V; v += 32) {
        const uint4 q = br[v];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = unpack2<DT>(w[i]);
          if (!quick) {
            o[i] = pack2<DT>(__fdiv_rn(f.x, sum), __fdiv_rn(f.y, sum));
          } else if (DT == kDtBF16) {
            o[i] = pack2<DT>(__fmul_rn(f.x, dv.r), __fmul_rn(f.y, dv.r));
          } else {
            const float qx = __fmul_rn(f.x, dv.r), qy = __fmul_rn(f.y, dv.r);
            o[i] = pack2<DT>(__fmaf_rn(__fmaf_rn(-qx, sum, f.x), dv.r, qx), __fmaf_rn(__fmaf_rn(-qy, sum, f.y), dv.r, qy));
          }
        }
        stg_stream(yr + v, make_uint4(o[0], o[1], o[2], o[3]));
      }
    }
    __syncthreads();  // the tile buffer is refilled
  }
}

// Any row length and alignment: one warp per row on global memory; the T-rounded sum is walked by
// the whole warp in lockstep over values exchanged by shuffles (slow, correct).
template <int DT>
__global__ void __launch_bounds__(kSoftmaxThreads) softmax16_generic_kernel(const void* __restrict__ x,
                                                                            void* __restrict__ y, int64_t rows, int n) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t row = warp; row < rows; row += n_warps) {
    const int64_t base = row * n;
    float m = __int_as_float(0xff800000);
    for (int i = lane; i < n; i += 32) m = max_ignoring_nan(m, load_elem<DT>(x, base + i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max_ignoring_nan(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    uint32_t s = 0;
    for (int i0 = 0; i0 < n; i0 += 32) {
      uint32_t e16 = 0;
      if (i0 + lane < n) {
        const float e = exp_rounded_to<DT>(round_to<DT>(__fsub_rn(load_elem<DT>(x, base + i0 + lane), m)));
        store_elem<DT>(y, base + i0 + lane, e);
        e16 = narrow16<DT>(e);
      }
      const int cnt = min(32, n - i0);
      for (int j = 0; j < cnt; ++j) s = add_t<DT>(s, __shfl_sync(0xFFFFFFFFu, e16, j));
    }
    const float sum = widen16<DT>(s);
    for (int i = lane; i < n; i += 32) store_elem<DT>(y, base + i, __fdiv_rn(load_elem<DT>(y, base + i), sum));
  }
}

// ---------------------------------------------------------------------------------------------
// rotary embeddings: one thread per pair (x1, x2)
// ---------------------------------------------------------------------------------------------
constexpr int kRopeI = 0, kRope = 1, kRopeThd = 2;

template <int DT>
__device__ __forceinline__ void rope_pair(float x1, float x2, float c, float s, float& y1, float& y2) {
  y1 = round_to<DT>(__fsub_rn(round_to<DT>(__fmul_rn(x1, c)), round_to<DT>(__fmul_rn(x2, s))));
  y2 = round_to<DT>(__fadd_rn(round_to<DT>(__fmul_rn(x1, s)), round_to<DT>(__fmul_rn(x2, c))));
}

// Scalar form, any d (even): pair p of the flattened tensor.
template <int DT, int VARIANT>
__global__ void __launch_bounds__(256) rope_scalar_kernel(const void* __restrict__ src, const void* __restrict__ cos_,
                                                          const void* __restrict__ sin_, void* __restrict__ dst,
                                                          int64_t n_pairs, int h, int t, int d) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int hd = d / 2;
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
    const int64_t rowi = p / hd;  // row of d elements: (b, h, t) or (b, t, h)
    const int k = static_cast<int>(p - rowi * hd);
    const int it = VARIANT == kRopeThd ? static_cast<int>((rowi / h) % t) : static_cast<int>(rowi % t);
    const int64_t i1 = VARIANT == kRopeI ? rowi * d + 2 * k : rowi * d + k;
    const int64_t i2 = VARIANT == kRopeI ? i1 + 1 : i1 + hd;
    const int64_t ics = static_cast<int64_t>(it) * hd + k;
    float y1, y2;
    rope_pair<DT>(load_elem<DT>(src, i1), load_elem<DT>(src, i2), load_elem<DT>(cos_, ics), load_elem<DT>(sin_, ics),
                  y1, y2);
    store_elem<DT>(dst, i1, y1);
    store_elem<DT>(dst, i2, y2);
  }
}

// Vector forms.  16-bit types use the packed T-rounding instructions: mul.rn / add.rn on two values at
// a time round each product and each sum once to T, which is what candle's `half` arithmetic does
// (it widens to f32, where the product of two 16-bit values is exact and the double rounding of a
// sum is innocuous, then rounds to T).  x - y is computed as x + (-y), the same value.
template <int DT>
__device__ __forceinline__ uint32_t neg2(uint32_t a) { return a ^ 0x80008000u; }

// Half-split variants (rope, rope_thd): an item is one 16-byte vector of the first half of a row and
// its partner in the second half; cos / sin are the matching vector of row `it`.
template <int DT>
__device__ __forceinline__ void rope_split_item(const uint4& a, const uint4& b, const uint4& c, const uint4& s, uint4& r1,
                                                uint4& r2) {
  const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w}, wc[4] = {c.x, c.y, c.z, c.w},
                 ws[4] = {s.x, s.y, s.z, s.w};
  uint32_t o1[4], o2[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (DT == kDtF32) {
      float y1, y2;
      rope_pair<DT>(__uint_as_float(wa[i]), __uint_as_float(wb[i]), __uint_as_float(wc[i]), __uint_as_float(ws[i]), y1, y2);
      o1[i] = __float_as_uint(y1);
      o2[i] = __float_as_uint(y2);
    } else {
      o1[i] = add2_rn<DT>(mul2_rn<DT>(wa[i], wc[i]), neg2<DT>(mul2_rn<DT>(wb[i], ws[i])));
      o2[i] = add2_rn<DT>(mul2_rn<DT>(wa[i], ws[i]), mul2_rn<DT>(wb[i], wc[i]));
    }
  }
  r1 = make_uint4(o1[0], o1[1], o1[2], o1[3]);
  r2 = make_uint4(o2[0], o2[1], o2[2], o2[3]);
}

// Two items per thread and trip, all loads first.
template <int DT, int VARIANT>
__global__ void __launch_bounds__(256) rope_split_vec_kernel(const uint4* __restrict__ src, const uint4* __restrict__ cos_,
                                                             const uint4* __restrict__ sin_, uint4* __restrict__ dst,
                                                             int64_t n_items, int h, int t, int hv) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t p0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p0 < n_items; p0 += 2 * stride) {
    uint4 a[2], b[2], c[2], s[2];
    int64_t v1[2];
    bool live[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int64_t p = p0 + u * stride;
      live[u] = p < n_items;
      const int64_t pp = live[u] ? p : p0;
      const int64_t rowi = pp / hv;
      const int k = static_cast<int>(pp - rowi * hv);
      const int it = VARIANT == kRopeThd ? static_cast<int>((rowi / h) % t) : static_cast<int>(rowi % t);
      v1[u] = rowi * 2 * hv + k;
      a[u] = ldg_stream(src + v1[u]);
      b[u] = ldg_stream(src + v1[u] + hv);
      c[u] = __ldg(cos_ + static_cast<int64_t>(it) * hv + k);
      s[u] = __ldg(sin_ + static_cast<int64_t>(it) * hv + k);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (!live[u]) continue;
      uint4 r1, r2;
      rope_split_item<DT>(a[u], b[u], c[u], s[u], r1, r2);
      stg_stream(dst + v1[u], r1);
      stg_stream(dst + v1[u] + hv, r2);
    }
  }
}

// Interleaved variant (rope_i): an item is one 16-byte vector of a row, i.e. PV / 2 adjacent pairs
// (x1, x2); cos / sin contribute PV / 2 values, 8 bytes.  16-bit: a word is one pair; with cc = (c, c)
// and ss = (s, s), P = w * cc = (x1 c, x2 c), Q = w * ss = (x1 s, x2 s) and the result is
// (P.lo - Q.hi, P.hi + Q.lo) = P + (-Q.hi, Q.lo).
template <int DT>
__device__ __forceinline__ uint4 rope_interleaved_item(const uint4& x, const uint2& c, const uint2& s) {
  const uint32_t wx[4] = {x.x, x.y, x.z, x.w};
  uint32_t o[4];
  if constexpr (DT == kDtF32) {
    const uint32_t wc[2] = {c.x, c.y}, ws[2] = {s.x, s.y};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float y1, y2;
      rope_pair<DT>(__uint_as_float(wx[2 * i]), __uint_as_float(wx[2 * i + 1]), __uint_as_float(wc[i]),
                    __uint_as_float(ws[i]), y1, y2);
      o[2 * i] = __float_as_uint(y1);
      o[2 * i + 1] = __float_as_uint(y2);
    }
  } else {
    const uint32_t wc[2] = {c.x, c.y}, ws[2] = {s.x, s.y};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t sel = (i & 1) ? 0x3232u : 0x1010u;
      const uint32_t cc = __byte_perm(wc[i >> 1], 0u, sel), ss = __byte_perm(ws[i >> 1], 0u, sel);
      const uint32_t P = mul2_rn<DT>(wx[i], cc), Q = mul2_rn<DT>(wx[i], ss);
      o[i] = add2_rn<DT>(P, __byte_perm(Q, 0u, 0x1032u) ^ 0x00008000u);
    }
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

template <int DT>
__global__ void __launch_bounds__(256) rope_interleaved_vec_kernel(const uint4* __restrict__ src,
                                                                   const uint2* __restrict__ cos_,
                                                                   const uint2* __restrict__ sin_, uint4* __restrict__ dst,
                                                                   int64_t n_items, int t, int V) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t p0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p0 < n_items; p0 += 4 * stride) {
    uint4 x[4];
    uint2 c[4], s[4];
    bool live[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t p = p0 + u * stride;
      live[u] = p < n_items;
      const int64_t pp = live[u] ? p : p0;
      const int64_t rowi = pp / V;  // row of d elements: (b, h, t)
      const int k = static_cast<int>(pp - rowi * V);
      const int64_t ics = (rowi % t) * V + k;
      x[u] = ldg_stream(src + pp);
      c[u] = __ldg(cos_ + ics);
      s[u] = __ldg(sin_ + ics);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (live[u]) stg_stream(dst + p0 + u * stride, rope_interleaved_item<DT>(x[u], c[u], s[u]));
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int DT, int VARIANT>
cudaError_t launch_rope_t(const void* src, const void* cos_, const void* sin_, void* dst, int64_t b, int h, int t, int d,
                          cudaStream_t stream) {
  const int64_t n_pairs = b * h * t * (d / 2);
  if (n_pairs == 0) return cudaSuccess;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  constexpr int PV = Elem<DT>::kPerVec;
  const bool aligned = aligned16(src) && aligned16(cos_) && aligned16(sin_) && aligned16(dst);
  if (VARIANT != kRopeI && (d / 2) % PV == 0 && aligned) {
    const int hv = d / 2 / PV;
    const int64_t n_items = b * h * t * hv;
    int64_t grid = (n_items + 511) / 512;
    if (grid > cap) grid = cap;
    rope_split_vec_kernel<DT, VARIANT><<<static_cast<unsigned>(grid), 256, 0, stream>>>(
        static_cast<const uint4*>(src), static_cast<const uint4*>(cos_), static_cast<const uint4*>(sin_),
        static_cast<uint4*>(dst), n_items, h, t, hv);
    return cudaGetLastError();
  }
  if (VARIANT == kRopeI && d % PV == 0 && aligned) {
    const int V = d / PV;
    const int64_t n_items = b * h * t * V;
    int64_t grid = (n_items + 1023) / 1024;
    if (grid > cap) grid = cap;
    rope_interleaved_vec_kernel<DT><<<static_cast<unsigned>(grid), 256, 0, stream>>>(
        static_cast<const uint4*>(src), static_cast<const uint2*>(cos_), static_cast<const uint2*>(sin_),
        static_cast<uint4*>(dst), n_items, t, V);
    return cudaGetLastError();
  }
  int64_t grid = (n_pairs + 255) / 256;
  if (grid > cap) grid = cap;
  rope_scalar_kernel<DT, VARIANT><<<static_cast<unsigned>(grid), 256, 0, stream>>>(src, cos_, sin_, dst, n_pairs, h, t, d);
  return cudaGetLastError();
}

template <int DT>
cudaError_t launch_rope_dt(int variant, const void* src, const void* cos_, const void* sin_, void* dst, int64_t b, int h,
                           int t, int d, cudaStream_t stream) {
  switch (variant) {
    case kRopeI:
      return launch_rope_t<DT, kRopeI>(src, cos_, sin_, dst, b, h, t, d, stream);
    case kRope:
      return launch_rope_t<DT, kRope>(src, cos_, sin_, dst, b, h, t, d, stream);
    default:
      return launch_rope_t<DT, kRopeThd>(src, cos_, sin_, dst, b, h, t, d, stream);
  }
}

template <int DT>
cudaError_t launch_softmax16(const void* x, void* y, int64_t rows, int n, cudaStream_t stream) {
  const int64_t row_bytes = static_cast<int64_t>(n) * 2;
  constexpr int64_t kLut = ExpLut<DT>::kBytes;
  const int V = static_cast<int>(row_bytes / 16);
  const int pitch_vecs = V | 1;
  const int64_t pitch = static_cast<int64_t>(pitch_vecs) * 16;
  if (row_bytes % 16 == 0 && aligned16(x) && aligned16(y) && kLut + pitch + 64 <= 226 * 1024) {
    // three CTAs per SM where the rows allow it (their walks overlap the others' loads and stores),
    // up to 32 rows per tile (one per lane of the walking warp)
    const int64_t budget = 74 * 1024 - kLut;
    int R = static_cast<int>(budget > pitch ? budget / (pitch + 8) : 1);
    if (R > 32) R = 32;
    const int sms = sm_count();
    const int64_t spread = (rows + 3 * sms - 1) / (3 * sms);  // spread small problems over the device
    if (R > spread) R = static_cast<int>(spread);
    if (R < 1) R = 1;
    // whole batches per warp: phase 1 then takes one round of loads per tile
    const int vpl = V <= 32 ? 1 : (V <= 64 ? 2 : (V <= 128 ? 4 : (V <= 256 ? 8 : (V <= 512 ? 16 : 0))));
    const int round_rows = softmax16_rows_per_batch(vpl) * (kSoftmax16Threads / 32);
    if (R >= round_rows) R = R / round_rows * round_rows;
    const size_t smem = static_cast<size_t>(kLut) + static_cast<size_t>(R) * pitch + static_cast<size_t>(R) * 8 + 16;
    void (*kern)(const uint4*, uint4*, int64_t, int, int, int) = softmax16_staged_kernel<DT, 0>;
    switch (vpl) {
      case 1: kern = softmax16_staged_kernel<DT, 1>; break;
      case 2: kern = softmax16_staged_kernel<DT, 2>; break;
      case 4: kern = softmax16_staged_kernel<DT, 4>; break;
      case 8: kern = softmax16_staged_kernel<DT, 8>; break;
      case 16: kern = softmax16_staged_kernel<DT, 16>; break;
      default: break;
    }
    int per_sm = 1;
    const int want = smem * 3 + 3072 <= 227 * 1024 ? 3 : (smem * 2 + 2048 <= 227 * 1024 ? 2 : 1);
    cudaError_t e = kernel_launch_config(reinterpret_cast<const void*>(kern), kSoftmax16Threads, smem,
                                         static_cast<int>(((smem + 1024) * want * 100) / (228 * 1024) + 1), &per_sm);
    if (e != cudaSuccess) return e;
    const int64_t tiles = (rows + R - 1) / R;
    int64_t grid = static_cast<int64_t>(sms) * per_sm;
    if (grid > tiles) grid = tiles;
    kern<<<static_cast<unsigned>(grid), kSoftmax16Threads, smem, stream>>>(static_cast<const uint4*>(x),
                                                                         static_cast<uint4*>(y), rows, V, R, pitch_vecs);
    return cudaGetLastError();
  }
  int64_t grid = (rows + 7) / 8;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (grid > cap) grid = cap;
  softmax16_generic_kernel<DT><<<static_cast<unsigned>(grid), kSoftmaxThreads, 0, stream>>>(x, y, rows, n);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_softmax_last_dim(int dtype, const void* x, void* y, int64_t rows, int n, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  if (dtype == kDtF32) {
    const size_t row_bytes = static_cast<size_t>(n) * 4;
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0;
    if (aligned && row_bytes % 16 == 0 && row_bytes <= 96 * 1024) {
      int warps = static_cast<int>((200 * 1024) / row_bytes);
      if (warps > kSoftmaxStagedMaxWarps) warps = kSoftmaxStagedMaxWarps;
      const size_t smem = 256 + static_cast<size_t>(warps) * row_bytes;
      auto kern = softmax_f32_staged_kernel;
      int per_sm = 1;
      cudaError_t e = kernel_launch_config(reinterpret_cast<const void*>(kern), warps * 32, smem,
                                           static_cast<int>((2 * (smem + 1024) * 100) / (228 * 1024) + 1), &per_sm);
      if (e != cudaSuccess) return e;
      int64_t grid = (rows + warps - 1) / warps;
      const int64_t cap = static_cast<int64_t>(sm_count()) * per_sm;
      if (grid > cap) grid = cap;
      kern<<<static_cast<unsigned>(grid), warps * 32, smem, stream>>>(static_cast<const uint4*>(x), static_cast<uint4*>(y),
                                                                     rows, n, static_cast<int>(row_bytes));
      return cudaGetLastError();
    }
    int64_t grid = (rows + 7) / 8;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    if (grid > cap) grid = cap;
    softmax_f32_kernel<<<static_cast<unsigned>(grid), kSoftmaxThreads, 0, stream>>>(static_cast<const float*>(x),
                                                                                   static_cast<float*>(y), rows, n);
    return cudaGetLastError();
  }
  return dtype == kDtBF16 ? launch_softmax16<kDtBF16>(x, y, rows, n, stream) : launch_softmax16<kDtF16>(x, y, rows, n, stream);
}

cudaError_t launch_rope(int variant, int dtype, const void* src, const void* cos_, const void* sin_, void* dst, int64_t b,
                        int h, int t, int d, cudaStream_t stream) {
  switch (dtype) {
    case kDtF32:
      return launch_rope_dt<kDtF32>(variant, src, cos_, sin_, dst, b, h, t, d, stream);
    case kDtF16:
      return launch_rope_dt<kDtF16>(variant, src, cos_, sin_, dst, b, h, t, d, stream);
    default:
      return launch_rope_dt<kDtBF16>(variant, src, cos_, sin_, dst, b, h, t, d, stream);
  }
}

}  // namespace cb200
