// Shared device helpers: element traits, exact-rounding arithmetic, bulk-async copy and mbarrier
// wrappers (sm_100a inline PTX), block reductions and the device status record.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/candle_b200.h"

namespace cb200 {

constexpr int kDtF32 = CB200_DTYPE_F32;
constexpr int kDtF16 = CB200_DTYPE_F16;
constexpr int kDtBF16 = CB200_DTYPE_BF16;

// ---------------------------------------------------------------------------------------------
// Element traits.  Every conversion is IEEE round-to-nearest-even, which is what crate `half`
// does on candle's CPU path; products and sums that candle rounds separately are written with
// __fmul_rn/__fadd_rn/... so that nvcc never contracts them into an FMA.
// ---------------------------------------------------------------------------------------------
template <int DT>
struct Elem;

template <>
struct Elem<kDtF32> {
  using type = float;
  static constexpr int kBytes = 4;
  static constexpr int kPerVec = 4;  // elements per 16-byte vector
};
template <>
struct Elem<kDtF16> {
  using type = __half;
  static constexpr int kBytes = 2;
  static constexpr int kPerVec = 8;
};
template <>
struct Elem<kDtBF16> {
  using type = __nv_bfloat16;
  static constexpr int kBytes = 2;
  static constexpr int kPerVec = 8;
};

// Two 16-bit elements packed in a 32-bit word <-> two floats.
template <int DT>
__device__ __forceinline__ float2 unpack2(uint32_t w);
template <>
__device__ __forceinline__ float2 unpack2<kDtBF16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<kDtF16>(uint32_t w) {
  __half2 h = *reinterpret_cast<__half2*>(&w);
  return __half22float2(h);
}

template <int DT>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<kDtBF16>(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
template <>
__device__ __forceinline__ uint32_t pack2<kDtF16>(float lo, float hi) {
  __half2 p = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// One element rounded to T and widened again (the value a T-typed temporary holds on the CPU).
template <int DT>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<kDtF32>(float v) {
  return v;
}
template <>
__device__ __forceinline__ float round_to<kDtBF16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
template <>
__device__ __forceinline__ float round_to<kDtF16>(float v) {
  return __half2float(__float2half_rn(v));
}

template <int DT>
__device__ __forceinline__ float load_elem(const void* p, int64_t i);
template <>
__device__ __forceinline__ float load_elem<kDtF32>(const void* p, int64_t i) {
  return static_cast<const float*>(p)[i];
}
template <>
__device__ __forceinline__ float load_elem<kDtBF16>(const void* p, int64_t i) {
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
template <>
__device__ __forceinline__ float load_elem<kDtF16>(const void* p, int64_t i) {
  return __half2float(static_cast<const __half*>(p)[i]);
}

template <int DT>
__device__ __forceinline__ void store_elem(void* p, int64_t i, float v);
template <>
__device__ __forceinline__ void store_elem<kDtF32>(void* p, int64_t i, float v) {
  static_cast<float*>(p)[i] = v;
}
template <>
__device__ __forceinline__ void store_elem<kDtBF16>(void* p, int64_t i, float v) {
  static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ void store_elem<kDtF16>(void* p, int64_t i, float v) {
  static_cast<__half*>(p)[i] = __float2half_rn(v);
}

// One 16-byte vector <-> its elements widened to f32 (floats_to_vec rounds to T).
template <int DT>
__device__ __forceinline__ void vec_to_floats(const uint4& q, float (&f)[Elem<DT>::kPerVec]) {
  if constexpr (DT == kDtF32) {
    f[0] = __uint_as_float(q.x);
    f[1] = __uint_as_float(q.y);
    f[2] = __uint_as_float(q.z);
    f[3] = __uint_as_float(q.w);
  } else {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = unpack2<DT>(w[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}

template <int DT>
__device__ __forceinline__ uint4 floats_to_vec(const float (&f)[Elem<DT>::kPerVec]) {
  if constexpr (DT == kDtF32) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  } else {
    return make_uint4(pack2<DT>(f[0], f[1]), pack2<DT>(f[2], f[3]), pack2<DT>(f[4], f[5]), pack2<DT>(f[6], f[7]));
  }
}

// What a vocabulary shard writes for a row it does not own: zero BITS.  The shards' partial rows are
// combined by adding their bit patterns as unsigned integers (one non-zero contributor per element),
// which is exact for every value: -0.0, subnormals and NaN payloads come through unchanged, whatever a
// floating-point reduction would make of them.
__device__ __forceinline__ uint4 masked_row_vec() { return make_uint4(0, 0, 0, 0); }

// 16-byte global accesses.  Inputs are read once: bypass L1 allocation; outputs are streamed.
__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void stg_stream(uint4* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Two consecutive vectors (32 bytes, 32-byte aligned) in ONE store.  Where a lane owns 32 contiguous
// output bytes, two 16-byte stores make every warp instruction write the halves of 32-byte sectors, and
// both L2 and NVLink handle that badly: a kernel that only stores ran at 3.6 TB/s locally and 300 GB/s
// into a peer's memory that way, against 5.9 TB/s and 700 GB/s with the 256-bit store.
__device__ __forceinline__ void stg_stream32(uint4* p, uint4 lo, uint4 hi) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(lo.x), "r"(lo.y), "r"(lo.z),
               "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
               : "memory");
}
// The same 32 bytes for destinations that are only 16-byte aligned.
__device__ __forceinline__ void stg_stream_pair(uint4* p, uint4 lo, uint4 hi, bool wide) {
  if (wide) {
    stg_stream32(p, lo, hi);
  } else {
    stg_stream(p, lo);
    stg_stream(p + 1, hi);
  }
}

// ---------------------------------------------------------------------------------------------
// Device status record (mirrors cb200_status in the C header).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void report_status(cb200_status* st, int code, int64_t position, int64_t index,
                                              int64_t size) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, code) == 0) {  // keep the first report only
    st->position = position;
    st->index = index;
    st->size = size;
    __threadfence();
  }
}

// ids of any supported integer type, widened the way candle's IntDType::as_usize does
// (a negative i64 becomes a huge unsigned value and fails the bounds check).
__device__ __forceinline__ uint64_t read_id(const void* ids, int id_dtype, int64_t i) {
  switch (id_dtype) {
    case CB200_ID_U8:
      return static_cast<const uint8_t*>(ids)[i];
    case CB200_ID_U32:
      return static_cast<const uint32_t*>(ids)[i];
    default:
      return static_cast<uint64_t>(static_cast<const int64_t*>(ids)[i]);
  }
}

// ---------------------------------------------------------------------------------------------
// mbarrier + bulk async copy (the TMA engine's untiled form).  Addresses and sizes must be
// multiples of 16 bytes.  Every wait is bounded: after `spins` polls (kWaitSpins unless the host's
// self-test hook lowered it) it gives up and the caller reports CB200_STATUS_WAIT_TIMEOUT instead
// of spinning forever.
// ---------------------------------------------------------------------------------------------
constexpr uint32_t kWaitSpins = 1u << 22;

// How the kernels wait, as the launchers pass it to them.  Normally {kWaitSpins, 0}.  The library's
// self-test hook (cb200_selftest_wait_expiry) sets a small poll budget and makes every mbarrier
// expect `extra_tx` more bytes than its copies deliver, so that the waits run out and the give-up
// paths execute -- without any copy actually failing.
struct WaitTuning {
  uint32_t spins;
  uint32_t extra_tx;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Returns false if the phase did not complete within the spin budget.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t spins = kWaitSpins) {
  for (uint32_t i = 0; i < spins; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
// A CTA that gives up on a wait must not retire while bulk copies may still be writing its shared
// memory.  After the bounded second-chance waits it also pauses for about 0.1 ms (bounded), far longer
// than any copy that was issued takes to land.
__device__ __forceinline__ void drain_pause() {
  for (int i = 0; i < 64; ++i) __nanosleep(2000);
}
// global -> shared, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// shared -> global, tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Orders this thread's earlier generic-proxy view of shared memory before later async-proxy use.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 16-byte asynchronous global -> shared copy that bypasses registers and L1 (LDGSTS).  A thread
// may read what it copied itself after cp_async_wait_all(); other threads need a barrier.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
// Waits until at most `pending` (0..7) of this thread's most recent copy groups are unfinished.
__device__ __forceinline__ void cp_async_wait_pending(int pending) {
  switch (pending) {
    case 0:
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      break;
    case 1:
      asm volatile("cp.async.wait_group 1;" ::: "memory");
      break;
    case 2:
      asm volatile("cp.async.wait_group 2;" ::: "memory");
      break;
    case 3:
      asm volatile("cp.async.wait_group 3;" ::: "memory");
      break;
    case 4:
      asm volatile("cp.async.wait_group 4;" ::: "memory");
      break;
    case 5:
      asm volatile("cp.async.wait_group 5;" ::: "memory");
      break;
    case 6:
      asm volatile("cp.async.wait_group 6;" ::: "memory");
      break;
    default:
      asm volatile("cp.async.wait_group 7;" ::: "memory");
      break;
  }
}

// ---------------------------------------------------------------------------------------------
// Warp reductions.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// x / m, correctly rounded, for many x and one m.  With r = RN(1/m), q = RN(x r) is within one ulp
// of the quotient, rem = x - q m is then exact in an FMA, and RN(q + rem r) is the correctly rounded
// quotient (Markstein's theorem) -- three instructions instead of the full IEEE division sequence.
// It needs every intermediate to be a normal number, so it is used for 2^-60 <= |x|, m <= 2^60 only;
// anything else (zeros, tiny or huge values, NaN, infinity) takes the division instruction sequence.
struct RowDivisor {
  float m, r;
  bool fast;
};
__device__ __forceinline__ RowDivisor make_row_divisor(float m) {
  RowDivisor d;
  d.m = m;
  d.fast = (m >= 8.6736174e-19f) && (m <= 1.1529215e18f);
  d.r = d.fast ? __frcp_rn(m) : 0.0f;
  return d;
}
__device__ __forceinline__ float div_by_row(float x, const RowDivisor& d) {
  const float ax = fabsf(x);
  if (d.fast && ax >= 8.6736174e-19f && ax <= 1.1529215e18f) {
    const float q = __fmul_rn(x, d.r);
    const float rem = __fmaf_rn(-q, d.m, x);
    return __fmaf_rn(rem, d.r, q);
  }
  return __fdiv_rn(x, d.m);
}

// The f32 pipeline candle applies to a row's sum of squares (candle-nn/src/ops.rs:491):
// sqrt(sum2 / n + eps), every operation correctly rounded.
__device__ __forceinline__ float rms_from_sum(float sum2, float n, float eps) {
  return __fsqrt_rn(__fadd_rn(__fdiv_rn(sum2, n), eps));
}

}  // namespace cb200
