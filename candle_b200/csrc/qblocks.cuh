// Decoders for GGML blocks of 32 elements.
//   BlockQ4_0 { d: f16, qs: [u8; 16] }                  18 bytes   candle-core/src/quantized/k_quants.rs:42-48
//   BlockQ4_1 { d, m: f16, qs: [u8; 16] }               20 bytes   k_quants.rs:50-57
//   BlockQ5_0 { d: f16, qh: [u8; 4], qs: [u8; 16] }     22 bytes   k_quants.rs:59-66
//   BlockQ5_1 { d, m: f16, qh: [u8; 4], qs: [u8; 16] }  24 bytes   k_quants.rs:68-76
//   BlockQ8_0 { d: f16, qs: [i8; 32] }                  34 bytes   k_quants.rs:78-84
// Values follow GgmlType::to_float (k_quants.rs:163-183, 329-349, 428-452, 535-562, 568-584):
//   Q4_0: y[j] = ((qs[j] & 15) - 8) * d,  y[j + 16] = ((qs[j] >> 4) - 8) * d   (j < 16)
//   Q4_1: y[j] = (qs[j] & 15) * d + m,    y[j + 16] = (qs[j] >> 4) * d + m
//   Q5_0 / Q5_1: the same with a fifth bit per element, bit e of the little-endian word qh for
//         element e of the block (Q5_0 subtracts 16 and has no m)
//   Q8_0: y[j] = qs[j] * d
// The `* d` products are exact in f32; the `+ m` of Q4_1 / Q5_1 is a second, rounded f32 operation,
// as in the CPU code (no fused multiply-add).
// The products are exact in f32 (an 8-bit integer times an 11-bit significand), so the decoded
// f32 values, and their roundings to f16 / bf16, are bit-identical to the CPU's, including the
// sign of zero: the integer is converted to float first and multiplied by d, exactly as the CPU
// does, instead of the d*q + (-8d) form of the reference's CUDA kernel.
// Blocks are only 2-byte aligned inside a row, hence the 16-bit loads.
#pragma once

#include "common.cuh"

namespace cb200 {

template <int QT>
struct QBlock;
template <>
struct QBlock<CB200_QTYPE_Q4_0> {
  static constexpr int kBytes = 18;
};
template <>
struct QBlock<CB200_QTYPE_Q8_0> {
  static constexpr int kBytes = 34;
};
template <>
struct QBlock<CB200_QTYPE_Q4_1> {
  static constexpr int kBytes = 20;
};
template <>
struct QBlock<CB200_QTYPE_Q5_0> {
  static constexpr int kBytes = 22;
};
template <>
struct QBlock<CB200_QTYPE_Q5_1> {
  static constexpr int kBytes = 24;
};

// Internal pseudo-format: rows that already hold 16-bit elements of the output type (a dense f16 /
// bf16 table).  It lets the row-slot kernel, with its ring of bulk-copied rows, serve dense tables:
// a "block" is 32 elements = 64 bytes and decoding is a plain 16-byte load.  Never part of the ABI.
constexpr int kQTypeDense16 = 1000;
template <>
struct QBlock<kQTypeDense16> {
  static constexpr int kBytes = 64;
};

__host__ __device__ inline int qblock_bytes(int qtype) {
  switch (qtype) {
    case CB200_QTYPE_Q4_0:
      return 18;
    case CB200_QTYPE_Q4_1:
      return 20;
    case CB200_QTYPE_Q5_0:
      return 22;
    case CB200_QTYPE_Q5_1:
      return 24;
    case CB200_QTYPE_Q8_0:
      return 34;
    default:
      return 0;
  }
}

// Small integer held in byte `k` of `w` -> float, without the slow int-to-float conversion: the
// byte is spliced into the low mantissa bits of 2^23 (0x4B000000) and 2^23 + bias subtracted,
// which is exact.  For a signed byte the caller flips bit 7 first and passes bias = 128.
template <int K>
__device__ __forceinline__ float byte_to_float(uint32_t w, float magic_plus_bias) {
  return __fadd_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650 | K)), -magic_plus_bias);
}

// Decodes elements [8v, 8v+8) of a row of blocks starting at `row` (shared or global memory).
// `scale`, when given, receives the block's scale d.
template <int QT>
__device__ __forceinline__ void decode8(const unsigned char* row, int v, float (&out)[8], float* scale = nullptr) {
  constexpr bool kHasMin = QT == CB200_QTYPE_Q4_1 || QT == CB200_QTYPE_Q5_1;
  constexpr bool kFiveBits = QT == CB200_QTYPE_Q5_0 || QT == CB200_QTYPE_Q5_1;
  constexpr int kQsOffset = 2 + (kHasMin ? 2 : 0) + (kFiveBits ? 4 : 0);
  const int blk = v >> 2, sub = v & 3;
  const unsigned char* b = row + blk * QBlock<QT>::kBytes;
  const uint16_t* b16 = reinterpret_cast<const uint16_t*>(b);
  const float d = __half2float(*reinterpret_cast<const __half*>(b));
  if (scale != nullptr) *scale = d;
  uint32_t w0, w1;  // the eight source bytes
  {
    const uint16_t* q = reinterpret_cast<const uint16_t*>(b + kQsOffset + (QT == CB200_QTYPE_Q8_0 ? sub : (sub & 1)) * 8);
    w0 = static_cast<uint32_t>(q[0]) | (static_cast<uint32_t>(q[1]) << 16);
    w1 = static_cast<uint32_t>(q[2]) | (static_cast<uint32_t>(q[3]) << 16);
  }
  float bias;
  if (QT == CB200_QTYPE_Q8_0) {
    w0 ^= 0x80808080u;  // signed byte q -> unsigned q + 128
    w1 ^= 0x80808080u;
    bias = 8388608.0f + 128.0f;
  } else {
    const int shift = (sub >> 1) * 4;  // elements 0..15 are low nibbles, 16..31 high nibbles
    w0 = (w0 >> shift) & 0x0F0F0F0Fu;
    w1 = (w1 >> shift) & 0x0F0F0F0Fu;
    bias = 8388608.0f + (QT == CB200_QTYPE_Q4_0 ? 8.0f : (QT == CB200_QTYPE_Q5_0 ? 16.0f : 0.0f));
    if (kFiveBits) {
      // bits 8 sub .. 8 sub + 7 of qh are the fifth bits of these eight elements: one bit into bit 4
      // of each byte (x * 0x00204081 puts bit k of a 4-bit x at bit 8k; no two terms collide)
      const int qoff = kHasMin ? 2 : 1;  // qh sits after d (and m), 2-byte aligned
      const uint32_t qh = static_cast<uint32_t>(b16[qoff]) | (static_cast<uint32_t>(b16[qoff + 1]) << 16);
      const uint32_t bits = (qh >> (8 * sub)) & 0xFFu;
      w0 |= (((bits & 0xFu) * 0x00204081u) & 0x01010101u) << 4;
      w1 |= (((bits >> 4) * 0x00204081u) & 0x01010101u) << 4;
    }
  }
  out[0] = __fmul_rn(byte_to_float<0>(w0, bias), d);
  out[1] = __fmul_rn(byte_to_float<1>(w0, bias), d);
  out[2] = __fmul_rn(byte_to_float<2>(w0, bias), d);
  out[3] = __fmul_rn(byte_to_float<3>(w0, bias), d);
  out[4] = __fmul_rn(byte_to_float<0>(w1, bias), d);
  out[5] = __fmul_rn(byte_to_float<1>(w1, bias), d);
  out[6] = __fmul_rn(byte_to_float<2>(w1, bias), d);
  out[7] = __fmul_rn(byte_to_float<3>(w1, bias), d);
  if (kHasMin) {
    const float m = __half2float(*reinterpret_cast<const __half*>(b + 2));
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __fadd_rn(out[i], m);
  }
}

// Same, rounded to a 16-bit type and packed into one 16-byte vector.
template <int QT, int DT>
__device__ __forceinline__ uint4 decode_vec8(const unsigned char* row, int v, float* scale = nullptr) {
  if constexpr (QT == kQTypeDense16) {
    if (scale != nullptr) *scale = 1.0f;
    return reinterpret_cast<const uint4*>(row)[v];
  } else {
    float f[8];
    decode8<QT>(row, v, f, scale);
    return make_uint4(pack2<DT>(f[0], f[1]), pack2<DT>(f[2], f[3]), pack2<DT>(f[4], f[5]), pack2<DT>(f[6], f[7]));
  }
}

// Decodes the sixteen elements [16p, 16p+16) (half a block) of a row of blocks: two vectors that
// share one scale.  Q8_0: bytes 16*(p&1).. of the block; Q4_0: the low (p even) or high (p odd)
// nibbles of all sixteen bytes.
template <int QT, int DT>
__device__ __forceinline__ void decode_half_block(const unsigned char* row, int p, uint4& lo8, uint4& hi8, float& scale) {
  if constexpr (QT == kQTypeDense16) {
    lo8 = reinterpret_cast<const uint4*>(row)[2 * p];
    hi8 = reinterpret_cast<const uint4*>(row)[2 * p + 1];
    scale = 1.0f;
    return;
  } else {
    const unsigned char* b = row + (p >> 1) * QBlock<QT>::kBytes;
    const float d = __half2float(*reinterpret_cast<const __half*>(b));
    scale = d;
    const uint16_t* q = reinterpret_cast<const uint16_t*>(b + 2 + (QT == CB200_QTYPE_Q8_0 ? (p & 1) * 16 : 0));
    uint32_t w[4];
  #pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = static_cast<uint32_t>(q[2 * i]) | (static_cast<uint32_t>(q[2 * i + 1]) << 16);
    float bias;
    if (QT == CB200_QTYPE_Q8_0) {
  #pragma unroll
      for (int i = 0; i < 4; ++i) w[i] ^= 0x80808080u;
      bias = 8388608.0f + 128.0f;
    } else {
      const int shift = (p & 1) * 4;
  #pragma unroll
      for (int i = 0; i < 4; ++i) w[i] = (w[i] >> shift) & 0x0F0F0F0Fu;
      bias = 8388608.0f + 8.0f;
    }
    float f[16];
  #pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[4 * i] = __fmul_rn(byte_to_float<0>(w[i], bias), d);
      f[4 * i + 1] = __fmul_rn(byte_to_float<1>(w[i], bias), d);
      f[4 * i + 2] = __fmul_rn(byte_to_float<2>(w[i], bias), d);
      f[4 * i + 3] = __fmul_rn(byte_to_float<3>(w[i], bias), d);
    }
    lo8 = make_uint4(pack2<DT>(f[0], f[1]), pack2<DT>(f[2], f[3]), pack2<DT>(f[4], f[5]), pack2<DT>(f[6], f[7]));
    hi8 = make_uint4(pack2<DT>(f[8], f[9]), pack2<DT>(f[10], f[11]), pack2<DT>(f[12], f[13]), pack2<DT>(f[14], f[15]));
  }
}

}  // namespace cb200
