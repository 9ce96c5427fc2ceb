// candle's composite ("slow") norm as one kernel: what LayerNorm::forward computes when the fused
// op does not apply -- no bias, remove_mean == false, or a non-contiguous input -- and what
// ops::rms_norm_slow / layer_norm_slow compute (candle-nn/src/layer_norm.rs:115-135,
// candle-nn/src/ops.rs:628-639, 876-894).  The chain is f32 inside, rounds once to T and applies
// weight and bias in T:
//   x = f32(x); [mean = fl(fl(sum(x) * f32(1/n)) + 0); x = x - mean;]
//   norm = fl(fl(sum(x*x) * f32(1/n)) + 0); d = sqrt(fl(fl(norm * 1) + eps));
//   y = T(x / d) * weight [+ bias]
// (`Tensor / f64` and `Tensor + f64` are affine maps v * mul + add with both constants cast to f32,
// candle-core/src/tensor.rs:2653-2656, candle-core/src/cpu_backend/mod.rs:291-299.)
//
// The row sums are candle's `vec_sum` in its AVX form (candle-core/src/cpu/mod.rs:113-135,
// cpu/avx.rs:54-66): 32 partial sums, partial l taking elements l, l + 32, l + 64, ... in order,
// folded as ((p[l] + p[l+8]) + (p[l+16] + p[l+24])) for l < 8, then r[l] + r[l+4], then two
// horizontal adds, then the n % 32 leftover elements one by one.  That order maps onto a warp as it
// is -- lane l owns partial l, and the fold is a butterfly over lane distances 8, 16, 4, 1, 2 -- so
// the kernel reproduces the AVX build of candle bit for bit.  (A candle built without SIMD sums left
// to right instead; against such a build the results agree to rounding error only.)
#include "launch.h"
#include "rms_rowreg.cuh"

namespace cb200 {

namespace {

constexpr int kSlowThreads = 256;

__device__ __forceinline__ float avx_fold(float v) {
  v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 8));
  v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 16));
  v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 4));
  v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 1));
  v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 2));
  return v;
}

// Element i of a staged row / of a T array in shared memory.
template <int DT>
__device__ __forceinline__ float smem_elem(const unsigned char* buf, int i) {
  if constexpr (DT == kDtF32)
    return reinterpret_cast<const float*>(buf)[i];
  else if constexpr (DT == kDtBF16)
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(buf)[i]);
  else
    return __half2float(reinterpret_cast<const __half*>(buf)[i]);
}
template <int DT>
__device__ __forceinline__ void smem_put(unsigned char* buf, int i, float v) {
  if constexpr (DT == kDtF32)
    reinterpret_cast<float*>(buf)[i] = v;
  else if constexpr (DT == kDtBF16)
    reinterpret_cast<__nv_bfloat16*>(buf)[i] = __float2bfloat16_rn(v);
  else
    reinterpret_cast<__half*>(buf)[i] = __float2half_rn(v);
}

// Rows that are whole 16-byte vectors (16-byte aligned tensors): a warp per row, the row staged in
// the warp's own shared-memory buffer.  Global memory is touched by 16-byte accesses only -- all of a
// row's loads are issued before the first is used, and the finished row leaves the same way -- while
// the passes that need lane l to own elements l, l + 32, ... (the AVX order) run on shared memory,
// where that access pattern is conflict-free.  (weight and bias must be 16-byte aligned too.)
constexpr int kSlowStagedMaxWarps = 24;
template <int DT>
__global__ void __launch_bounds__(kSlowStagedMaxWarps * 32) norm_slow_staged_kernel(
    const uint4* __restrict__ x, const void* __restrict__ weight, const void* __restrict__ bias, uint4* __restrict__ y,
    int64_t rows, int n, float eps, int remove_mean, int pitch) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, warps = blockDim.x >> 5;
  unsigned char* buf = smem_raw + static_cast<size_t>(wib) * pitch;
  uint4* bufv = reinterpret_cast<uint4*>(buf);
  const int V = n * Elem<DT>::kBytes / 16;
  const int np = n & ~31;
  const float inv_n = static_cast<float>(1.0 / static_cast<double>(n));
  constexpr int U = 8;  // 16-byte loads per lane in flight
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * warps + wib; row < rows;
       row += static_cast<int64_t>(gridDim.x) * warps) {
    const uint4* xr = x + row * V;
    for (int v0 = lane; v0 < V; v0 += 32 * U) {
      uint4 q[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (v0 + 32 * u < V) q[u] = ldg_stream(xr + v0 + 32 * u);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (v0 + 32 * u < V) bufv[v0 + 32 * u] = q[u];
    }
    __syncwarp();
    float mean = 0.0f;
    if (remove_mean) {
      float acc = 0.0f;
#pragma unroll 4
      for (int i = lane; i < np; i += 32) acc = __fadd_rn(acc, smem_elem<DT>(buf, i));
      float s = avx_fold(acc);
      for (int i = np; i < n; ++i) s = __fadd_rn(s, smem_elem<DT>(buf, i));
      mean = __fadd_rn(__fmul_rn(s, inv_n), 0.0f);
    }
    float acc = 0.0f;
#pragma unroll 4
    for (int i = lane; i < np; i += 32) {
      float v = smem_elem<DT>(buf, i);
      if (remove_mean) v = __fsub_rn(v, mean);
      acc = __fadd_rn(acc, __fmul_rn(v, v));
    }
    float q = avx_fold(acc);
    for (int i = np; i < n; ++i) {
      float v = smem_elem<DT>(buf, i);
      if (remove_mean) v = __fsub_rn(v, mean);
      q = __fadd_rn(q, __fmul_rn(v, v));
    }
    const float norm = __fadd_rn(__fmul_rn(q, inv_n), 0.0f);
    const float d = __fsqrt_rn(__fadd_rn(__fmul_rn(norm, 1.0f), eps));
    // The last pass has no order to keep: 16 bytes per lane, the division by the row's d in its exact
    // three-instruction form, weight and bias applied with the packed T-rounding instructions.
    const RowDivisor dv = make_row_divisor(d);
    const uint4* wv = static_cast<const uint4*>(weight);
    const uint4* bv = static_cast<const uint4*>(bias);
    uint4* yr = y + row * V;
    constexpr int PV = Elem<DT>::kPerVec;
#pragma unroll 2
    for (int v = lane; v < V; v += 32) {
      float f[PV];
      vec_to_floats<DT>(bufv[v], f);
#pragma unroll
      for (int e = 0; e < PV; ++e) {
        if (remove_mean) f[e] = __fsub_rn(f[e], mean);
        f[e] = div_by_row(f[e], dv);
      }
      const uint4 w = __ldg(wv + v);
      uint4 o;
      if constexpr (DT == kDtF32) {
        float g[PV];
        vec_to_floats<DT>(w, g);
#pragma unroll
        for (int e = 0; e < PV; ++e) f[e] = __fmul_rn(f[e], g[e]);
        if (bv != nullptr) {
          vec_to_floats<DT>(__ldg(bv + v), g);
#pragma unroll
          for (int e = 0; e < PV; ++e) f[e] = __fadd_rn(f[e], g[e]);
        }
        o = floats_to_vec<DT>(f);
      } else {
        o = floats_to_vec<DT>(f);  // T(x / d)
        o = make_uint4(mul2_rn<DT>(o.x, w.x), mul2_rn<DT>(o.y, w.y), mul2_rn<DT>(o.z, w.z), mul2_rn<DT>(o.w, w.w));
        if (bv != nullptr) {
          const uint4 b = __ldg(bv + v);
          o = make_uint4(add2_rn<DT>(o.x, b.x), add2_rn<DT>(o.y, b.y), add2_rn<DT>(o.z, b.z), add2_rn<DT>(o.w, b.w));
        }
      }
      stg_stream(yr + v, o);
    }
    __syncwarp();  // the buffer is refilled by the next row's loads
  }
}

// Any shape and alignment: scalar accesses on global memory, same arithmetic.
template <int DT>
__global__ void __launch_bounds__(kSlowThreads) norm_slow_kernel(const void* __restrict__ x,
                                                                 const void* __restrict__ weight,
                                                                 const void* __restrict__ bias, void* __restrict__ y,
                                                                 int64_t rows, int n, float eps, int remove_mean) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int np = n & ~31;
  const float inv_n = static_cast<float>(1.0 / static_cast<double>(n));
  for (int64_t row = warp; row < rows; row += n_warps) {
    const int64_t base = row * n;
    float mean = 0.0f;
    if (remove_mean) {
      float acc = 0.0f;
      for (int i = lane; i < np; i += 32) acc = __fadd_rn(acc, load_elem<DT>(x, base + i));
      float s = avx_fold(acc);
      for (int i = np; i < n; ++i) s = __fadd_rn(s, load_elem<DT>(x, base + i));
      mean = __fadd_rn(__fmul_rn(s, inv_n), 0.0f);
    }
    float acc = 0.0f;
    for (int i = lane; i < np; i += 32) {
      float v = load_elem<DT>(x, base + i);
      if (remove_mean) v = __fsub_rn(v, mean);
      acc = __fadd_rn(acc, __fmul_rn(v, v));
    }
    float q = avx_fold(acc);
    for (int i = np; i < n; ++i) {
      float v = load_elem<DT>(x, base + i);
      if (remove_mean) v = __fsub_rn(v, mean);
      q = __fadd_rn(q, __fmul_rn(v, v));
    }
    const float norm = __fadd_rn(__fmul_rn(q, inv_n), 0.0f);
    const float d = __fsqrt_rn(__fadd_rn(__fmul_rn(norm, 1.0f), eps));
    for (int i = lane; i < n; i += 32) {
      float v = load_elem<DT>(x, base + i);
      if (remove_mean) v = __fsub_rn(v, mean);
      float t = round_to<DT>(__fdiv_rn(v, d));
      t = round_to<DT>(__fmul_rn(t, load_elem<DT>(weight, i)));
      if (bias != nullptr) t = round_to<DT>(__fadd_rn(t, load_elem<DT>(bias, i)));
      store_elem<DT>(y, base + i, t);
    }
  }
}

}  // namespace

template <int DT>
static cudaError_t launch_norm_slow_t(const void* x, const void* weight, const void* bias, void* y, int64_t rows, int n,
                                      float eps, int remove_mean, cudaStream_t stream) {
  const size_t row_bytes = static_cast<size_t>(n) * Elem<DT>::kBytes;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                         reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(bias)) & 15u) == 0;
  if (aligned && row_bytes % 16 == 0 && row_bytes <= 96 * 1024) {
    // as many warps (rows in flight) per CTA as 200 KB of row buffers allow
    const int pitch = static_cast<int>(row_bytes);
    int warps = static_cast<int>((200 * 1024) / row_bytes);
    if (warps > kSlowStagedMaxWarps) warps = kSlowStagedMaxWarps;
    if (warps < 1) warps = 1;
    const size_t smem = static_cast<size_t>(warps) * pitch;
    auto kern = norm_slow_staged_kernel<DT>;
    int per_sm = 1;
    cudaError_t e = kernel_launch_config(reinterpret_cast<const void*>(kern), warps * 32, smem,
                                         static_cast<int>((2 * (smem + 1024) * 100) / (228 * 1024) + 1), &per_sm);
    if (e != cudaSuccess) return e;
    int64_t grid = (rows + warps - 1) / warps;
    const int64_t cap = static_cast<int64_t>(sm_count()) * per_sm;
    if (grid > cap) grid = cap;
    kern<<<static_cast<unsigned>(grid), warps * 32, smem, stream>>>(static_cast<const uint4*>(x), weight, bias,
                                                                   static_cast<uint4*>(y), rows, n, eps, remove_mean, pitch);
    return cudaGetLastError();
  }
  const int rows_per_cta = kSlowThreads / 32;
  int64_t grid = (rows + rows_per_cta - 1) / rows_per_cta;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (grid > cap) grid = cap;
  norm_slow_kernel<DT><<<static_cast<unsigned>(grid), kSlowThreads, 0, stream>>>(x, weight, bias, y, rows, n, eps, remove_mean);
  return cudaGetLastError();
}

cudaError_t launch_norm_slow(int dtype, const void* x, const void* weight, const void* bias, void* y, int64_t rows,
                             int n, float eps, int remove_mean, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  switch (dtype) {
    case kDtF32:
      return launch_norm_slow_t<kDtF32>(x, weight, bias, y, rows, n, eps, remove_mean, stream);
    case kDtF16:
      return launch_norm_slow_t<kDtF16>(x, weight, bias, y, rows, n, eps, remove_mean, stream);
    default:
      return launch_norm_slow_t<kDtBF16>(x, weight, bias, y, rows, n, eps, remove_mean, stream);
  }
}

}  // namespace cb200
