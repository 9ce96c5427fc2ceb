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

cudaError_t launch_norm_slow(int dtype, const void* x, const void* weight, const void* bias, void* y, int64_t rows,
                             int n, float eps, int remove_mean, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  const int rows_per_cta = kSlowThreads / 32;
  int64_t grid = (rows + rows_per_cta - 1) / rows_per_cta;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (grid > cap) grid = cap;
  switch (dtype) {
    case kDtF32:
      norm_slow_kernel<kDtF32><<<static_cast<unsigned>(grid), kSlowThreads, 0, stream>>>(x, weight, bias, y, rows, n, eps, remove_mean);
      break;
    case kDtF16:
      norm_slow_kernel<kDtF16><<<static_cast<unsigned>(grid), kSlowThreads, 0, stream>>>(x, weight, bias, y, rows, n, eps, remove_mean);
      break;
    default:
      norm_slow_kernel<kDtBF16><<<static_cast<unsigned>(grid), kSlowThreads, 0, stream>>>(x, weight, bias, y, rows, n, eps, remove_mean);
      break;
  }
  return cudaGetLastError();
}

}  // namespace cb200
