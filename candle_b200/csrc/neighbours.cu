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

constexpr int kSoftmax16Threads = 128;

// R rows of V 16-byte vectors per CTA, staged in shared memory at a pitch of an odd number of
// 16-byte units (conflict-free when 32 lanes walk 32 rows).
template <int DT>
__global__ void __launch_bounds__(kSoftmax16Threads) softmax16_staged_kernel(const uint4* __restrict__ x,
                                                                             uint4* __restrict__ y, int64_t rows,
                                                                             int V, int R, int pitch_vecs) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* buf = reinterpret_cast<uint4*>(smem_raw);
  uint32_t* sums = reinterpret_cast<uint32_t*>(buf + static_cast<size_t>(R) * pitch_vecs);  // [R]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kWarps = kSoftmax16Threads / 32;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * R;
  const int live = static_cast<int>(min(static_cast<int64_t>(R), rows - row0));

  // phases 1 and 2: a warp per row -- max, then e = T(exp(T(x - max))) into shared memory
  for (int r = warp; r < live; r += kWarps) {
    const uint4* xr = x + (row0 + r) * V;
    uint4* br = buf + static_cast<size_t>(r) * pitch_vecs;
    float m = __int_as_float(0xff800000);
    for (int v = lane; v < V; v += 32) {
      const uint4 q = ldg_stream(xr + v);
      br[v] = q;
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2<DT>(w[i]);
        m = max_ignoring_nan(m, max_ignoring_nan(f.x, f.y));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max_ignoring_nan(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    for (int v = lane; v < V; v += 32) {  // each lane re-reads the vectors it staged itself
      const uint4 q = br[v];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2<DT>(w[i]);
        const float e0 = exp_rounded_to<DT>(round_to<DT>(__fsub_rn(f.x, m)));
        const float e1 = exp_rounded_to<DT>(round_to<DT>(__fsub_rn(f.y, m)));
        o[i] = pack2<DT>(e0, e1);
      }
      br[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  __syncthreads();
  // phase 3: one lane per row, the T-rounded sum in candle's order
  if (tid < live) {
    const uint4* br = buf + static_cast<size_t>(tid) * pitch_vecs;
    uint32_t s = 0;  // +0 in T
#pragma unroll 2
    for (int v = 0; v < V; ++v) {
      const uint4 q = br[v];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s = add_t<DT>(s, w[i] & 0xFFFFu);
        s = add_t<DT>(s, w[i] >> 16);
      }
    }
    sums[tid] = s;
  }
  __syncthreads();
  // phase 4: y = T(e / sum)
  for (int r = warp; r < live; r += kWarps) {
    const float sum = widen16<DT>(sums[r]);
    const uint4* br = buf + static_cast<size_t>(r) * pitch_vecs;
    uint4* yr = y + (row0 + r) * V;
    for (int v = lane; v < V; v += 32) {
      const uint4 q = br[v];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2<DT>(w[i]);
        o[i] = pack2<DT>(__fdiv_rn(f.x, sum), __fdiv_rn(f.y, sum));
      }
      stg_stream(yr + v, make_uint4(o[0], o[1], o[2], o[3]));
    }
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

// Vector form for the half-split variants (rope, rope_thd): a thread takes one 16-byte vector of the
// first half of a row and its partner in the second half.  Needs d/2 to be a whole number of vectors
// and 16-byte aligned tensors.
template <int DT, int VARIANT>
__global__ void __launch_bounds__(256) rope_split_vec_kernel(const uint4* __restrict__ src, const uint4* __restrict__ cos_,
                                                             const uint4* __restrict__ sin_, uint4* __restrict__ dst,
                                                             int64_t n_items, int h, int t, int hv) {
  constexpr int PV = Elem<DT>::kPerVec;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < n_items; p += stride) {
    const int64_t rowi = p / hv;
    const int k = static_cast<int>(p - rowi * hv);
    const int it = VARIANT == kRopeThd ? static_cast<int>((rowi / h) % t) : static_cast<int>(rowi % t);
    const int64_t v1 = rowi * 2 * hv + k, v2 = v1 + hv;
    const uint4 a = ldg_stream(src + v1), b = ldg_stream(src + v2);
    const uint4 c = __ldg(cos_ + static_cast<int64_t>(it) * hv + k), s = __ldg(sin_ + static_cast<int64_t>(it) * hv + k);
    float fa[PV], fb[PV], fc[PV], fs[PV], o1[PV], o2[PV];
    if constexpr (DT == kDtF32) {
      const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w}, wc[4] = {c.x, c.y, c.z, c.w},
                     ws[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        fa[i] = __uint_as_float(wa[i]);
        fb[i] = __uint_as_float(wb[i]);
        fc[i] = __uint_as_float(wc[i]);
        fs[i] = __uint_as_float(ws[i]);
      }
    } else {
      const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w}, wc[4] = {c.x, c.y, c.z, c.w},
                     ws[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 t2 = unpack2<DT>(wa[i]);
        fa[2 * i] = t2.x, fa[2 * i + 1] = t2.y;
        t2 = unpack2<DT>(wb[i]);
        fb[2 * i] = t2.x, fb[2 * i + 1] = t2.y;
        t2 = unpack2<DT>(wc[i]);
        fc[2 * i] = t2.x, fc[2 * i + 1] = t2.y;
        t2 = unpack2<DT>(ws[i]);
        fs[2 * i] = t2.x, fs[2 * i + 1] = t2.y;
      }
    }
#pragma unroll
    for (int i = 0; i < PV; ++i) rope_pair<DT>(fa[i], fb[i], fc[i], fs[i], o1[i], o2[i]);
    uint4 r1, r2;
    if constexpr (DT == kDtF32) {
      r1 = make_uint4(__float_as_uint(o1[0]), __float_as_uint(o1[1]), __float_as_uint(o1[2]), __float_as_uint(o1[3]));
      r2 = make_uint4(__float_as_uint(o2[0]), __float_as_uint(o2[1]), __float_as_uint(o2[2]), __float_as_uint(o2[3]));
    } else {
      r1 = make_uint4(pack2<DT>(o1[0], o1[1]), pack2<DT>(o1[2], o1[3]), pack2<DT>(o1[4], o1[5]), pack2<DT>(o1[6], o1[7]));
      r2 = make_uint4(pack2<DT>(o2[0], o2[1]), pack2<DT>(o2[2], o2[3]), pack2<DT>(o2[4], o2[5]), pack2<DT>(o2[6], o2[7]));
    }
    stg_stream(dst + v1, r1);
    stg_stream(dst + v2, r2);
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
  if (VARIANT != kRopeI && (d / 2) % PV == 0 && aligned16(src) && aligned16(cos_) && aligned16(sin_) && aligned16(dst)) {
    const int hv = d / 2 / PV;
    const int64_t n_items = b * h * t * hv;
    int64_t grid = (n_items + 255) / 256;
    if (grid > cap) grid = cap;
    rope_split_vec_kernel<DT, VARIANT><<<static_cast<unsigned>(grid), 256, 0, stream>>>(
        static_cast<const uint4*>(src), static_cast<const uint4*>(cos_), static_cast<const uint4*>(sin_),
        static_cast<uint4*>(dst), n_items, h, t, hv);
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
  constexpr int64_t kBudget = 56 * 1024;  // shared memory per CTA: four CTAs per SM
  if (row_bytes % 16 == 0 && aligned16(x) && aligned16(y) && row_bytes + 16 + 128 <= kBudget) {
    const int V = static_cast<int>(row_bytes / 16);
    const int pitch_vecs = V | 1;
    int R = static_cast<int>((kBudget - 128) / (static_cast<int64_t>(pitch_vecs) * 16));
    if (R > 32) R = 32;
    // spread small problems over the device
    const int64_t spread = (rows + 2 * sm_count() - 1) / (2 * sm_count());
    if (R > spread) R = static_cast<int>(spread);
    if (R < 1) R = 1;
    const size_t smem = static_cast<size_t>(R) * pitch_vecs * 16 + static_cast<size_t>(R) * 4;
    auto kern = softmax16_staged_kernel<DT>;
    cudaError_t e = kernel_launch_config(reinterpret_cast<const void*>(kern), kSoftmax16Threads, smem, -1, nullptr);
    if (e != cudaSuccess) return e;
    const int64_t grid = (rows + R - 1) / R;
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
