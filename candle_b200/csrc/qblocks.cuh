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
//
// K-quant super-blocks of 256 elements (k_quants.rs:96-154; decoders :834-871, 1095-1149, 1313-1342,
// 1528-1563, 1716-1746, 1827-1839):
//   BlockQ2K { scales: [u8; 16], qs: [u8; 64], d, dmin: f16 }                     84 bytes
//   BlockQ3K { hmask: [u8; 32], qs: [u8; 64], scales: [u8; 12], d: f16 }         110 bytes
//   BlockQ4K { d, dmin: f16, scales: [u8; 12], qs: [u8; 128] }                   144 bytes
//   BlockQ5K { d, dmin: f16, scales: [u8; 12], qh: [u8; 32], qs: [u8; 128] }     176 bytes
//   BlockQ6K { ql: [u8; 128], qh: [u8; 64], scales: [i8; 16], d: f16 }           210 bytes
//   BlockQ8K { d: f32, qs: [i8; 256], bsums: [i16; 16] }                         292 bytes
// Their values are NOT exact products: y = (d * sc) * q - (dmin * m) and the like round two or three
// times in f32, so the decoders below perform the same operations in the same order with
// __fmul_rn / __fsub_rn (no fused multiply-add).
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

template <>
struct QBlock<CB200_QTYPE_Q2K> {
  static constexpr int kBytes = 84;
};
template <>
struct QBlock<CB200_QTYPE_Q3K> {
  static constexpr int kBytes = 110;
};
template <>
struct QBlock<CB200_QTYPE_Q4K> {
  static constexpr int kBytes = 144;
};
template <>
struct QBlock<CB200_QTYPE_Q5K> {
  static constexpr int kBytes = 176;
};
template <>
struct QBlock<CB200_QTYPE_Q6K> {
  static constexpr int kBytes = 210;
};
template <>
struct QBlock<CB200_QTYPE_Q8K> {
  static constexpr int kBytes = 292;
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
    case CB200_QTYPE_Q2K:
      return 84;
    case CB200_QTYPE_Q3K:
      return 110;
    case CB200_QTYPE_Q4K:
      return 144;
    case CB200_QTYPE_Q5K:
      return 176;
    case CB200_QTYPE_Q6K:
      return 210;
    case CB200_QTYPE_Q8K:
      return 292;
    default:
      return 0;
  }
}

// Elements per block: 256 for the K-quant super-blocks, 32 for the others.
__host__ __device__ constexpr bool is_kquant(int qtype) { return qtype >= CB200_QTYPE_Q2K && qtype <= CB200_QTYPE_Q8K; }
__host__ __device__ constexpr int qblock_elems(int qtype) { return is_kquant(qtype) ? 256 : 32; }

__device__ __forceinline__ float half_at(const unsigned char* p) {
  return __half2float(*reinterpret_cast<const __half*>(p));
}

// Small integer held in byte `k` of `w` -> float, without the slow int-to-float conversion: the
// byte is spliced into the low mantissa bits of 2^23 (0x4B000000) and 2^23 + bias subtracted,
// which is exact.  For a signed byte the caller flips bit 7 first and passes bias = 128.
template <int K>
__device__ __forceinline__ float byte_to_float(uint32_t w, float magic_plus_bias) {
  return __fadd_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650 | K)), -magic_plus_bias);
}

// A small non-negative integer -> float the same way.
__device__ __forceinline__ float small_int_to_float(int v) {
  return __fadd_rn(__uint_as_float(0x4B000000u | static_cast<uint32_t>(v)), -8388608.0f);
}

// Eight consecutive bytes at a 2-byte aligned address as two words (four 16-bit loads), or with one
// 8-byte load where the caller knows the address is 8-byte aligned.
template <bool ALIGNED8>
__device__ __forceinline__ uint2 load8(const unsigned char* p) {
  if constexpr (ALIGNED8) {
    return *reinterpret_cast<const uint2*>(p);
  } else {
    const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
    return make_uint2(static_cast<uint32_t>(h[0]) | (static_cast<uint32_t>(h[1]) << 16),
                      static_cast<uint32_t>(h[2]) | (static_cast<uint32_t>(h[3]) << 16));
  }
}

// The 6-bit (scale, min) pair j of a Q4K / Q5K block (get_scale_min_k4, quantized/utils.rs:49-59).
__device__ __forceinline__ void scale_min_k4(int j, const unsigned char* q, float& sc, float& mn) {
  int d, m;
  if (j < 4) {
    d = q[j] & 63;
    m = q[j + 4] & 63;
  } else {
    d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
  sc = small_int_to_float(d);
  mn = small_int_to_float(m);
}

// Elements [8s, 8s+8) of ONE super-block `b` (s = 0..31), with candle's operation order.  The eight
// source bytes are consecutive: they are fetched as two words and turned into floats four at a time
// (byte_to_float), so that neither byte loads nor integer-to-float conversions are on the path.
// ALIGNED16: `b` is 16-byte aligned (blocks of 144 and 176 bytes in a 16-byte aligned row).
template <int QT, bool ALIGNED16 = false>
__device__ __forceinline__ void decode8_kquant(const unsigned char* b, int s, float (&out)[8]) {
  const int e0 = 8 * s;
  if constexpr (QT == CB200_QTYPE_Q4K || QT == CB200_QTYPE_Q5K) {
    constexpr bool kFive = QT == CB200_QTYPE_Q5K;
    const float d = half_at(b), dmin = half_at(b + 2);
    const int g = e0 >> 6, idx = e0 & 63, hi = idx >> 5, l0 = idx & 31;
    float sc, mn;
    scale_min_k4(2 * g + hi, b + 4, sc, mn);
    const float dl = __fmul_rn(d, sc), ml = __fmul_rn(dmin, mn);
    uint2 w = load8<ALIGNED16>(b + (kFive ? 48 : 16) + 32 * g + l0);
    const int shift = 4 * hi;  // low nibbles are elements 0..31 of the group, high nibbles 32..63
    w.x = (w.x >> shift) & 0x0F0F0F0Fu;
    w.y = (w.y >> shift) & 0x0F0F0F0Fu;
    if (kFive) {
      const uint2 h = load8<ALIGNED16>(b + 16 + l0);
      const int bit = 2 * g + hi;
      w.x |= ((h.x >> bit) & 0x01010101u) << 4;
      w.y |= ((h.y >> bit) & 0x01010101u) << 4;
    }
    const float v[8] = {byte_to_float<0>(w.x, 8388608.0f), byte_to_float<1>(w.x, 8388608.0f),
                        byte_to_float<2>(w.x, 8388608.0f), byte_to_float<3>(w.x, 8388608.0f),
                        byte_to_float<0>(w.y, 8388608.0f), byte_to_float<1>(w.y, 8388608.0f),
                        byte_to_float<2>(w.y, 8388608.0f), byte_to_float<3>(w.y, 8388608.0f)};
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __fsub_rn(__fmul_rn(dl, v[i]), ml);
  } else if constexpr (QT == CB200_QTYPE_Q6K) {
    const float d = half_at(b + 208);
    const int n = e0 >> 7, r = e0 & 127, j = r >> 5, l0 = r & 31, is = l0 >> 4;
    uint2 lo = load8<false>(b + 64 * n + ((j & 1) ? 32 : 0) + l0);  // blocks of 210 bytes: 2-byte aligned only
    const uint2 hq = load8<false>(b + 128 + 32 * n + l0);
    const float sc = static_cast<float>(static_cast<signed char>(b[192 + 8 * n + is + 2 * j]));
    const float ds = __fmul_rn(d, sc);
    const int shift = (j & 2) ? 4 : 0;
    lo.x = ((lo.x >> shift) & 0x0F0F0F0Fu) | (((hq.x >> (2 * j)) & 0x03030303u) << 4);
    lo.y = ((lo.y >> shift) & 0x0F0F0F0Fu) | (((hq.y >> (2 * j)) & 0x03030303u) << 4);
    constexpr float kBias = 8388608.0f + 32.0f;  // the six-bit value minus 32, exactly
    const float v[8] = {byte_to_float<0>(lo.x, kBias), byte_to_float<1>(lo.x, kBias), byte_to_float<2>(lo.x, kBias),
                        byte_to_float<3>(lo.x, kBias), byte_to_float<0>(lo.y, kBias), byte_to_float<1>(lo.y, kBias),
                        byte_to_float<2>(lo.y, kBias), byte_to_float<3>(lo.y, kBias)};
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __fmul_rn(ds, v[i]);
  } else if constexpr (QT == CB200_QTYPE_Q8K) {
    // d is an f32 at a 2-byte aligned address: read it as two halves
    const uint16_t* d16 = reinterpret_cast<const uint16_t*>(b);
    const float d = __uint_as_float(static_cast<uint32_t>(d16[0]) | (static_cast<uint32_t>(d16[1]) << 16));
#pragma unroll
    for (int i = 0; i < 8; ++i)
      out[i] = __fmul_rn(d, static_cast<float>(static_cast<signed char>(b[4 + e0 + i])));
  } else if constexpr (QT == CB200_QTYPE_Q2K) {
    const float d = half_at(b + 80), dmin = half_at(b + 82);
    const int n = e0 >> 7, r = e0 & 127, j = r >> 5, half = (r & 31) >> 4, l0 = r & 15;
    const int sc = b[8 * n + 2 * j + half];
    const float dl = __fmul_rn(d, static_cast<float>(sc & 0xF)), ml = __fmul_rn(dmin, static_cast<float>(sc >> 4));
    const unsigned char* q = b + 16 + 32 * n + 16 * half + l0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      out[i] = __fsub_rn(__fmul_rn(dl, static_cast<float>((q[i] >> (2 * j)) & 3)), ml);
  } else {  // Q3K
    const float d_all = half_at(b + 108);
    const int n = e0 >> 7, r = e0 & 127, j = r >> 5, half = (r & 31) >> 4, l0 = r & 15;
    const int js = 8 * n + 2 * j + half;  // which of the sixteen 6-bit scales
    const unsigned char* s12 = b + 96;
    const int lo = js < 8 ? (s12[js] & 0xF) : (s12[js - 8] >> 4);
    const int sc = (lo | (((s12[8 + (js & 3)] >> (2 * (js >> 2))) & 3) << 4)) - 32;
    const float dl = __fmul_rn(d_all, static_cast<float>(sc));
    const unsigned char* q = b + 32 + 32 * n + 16 * half + l0;
    const unsigned char* hm = b + 16 * half + l0;
    const int mbit = 4 * n + j;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int v = ((q[i] >> (2 * j)) & 3) - (((hm[i] >> mbit) & 1) ? 0 : 4);
      out[i] = __fmul_rn(dl, static_cast<float>(v));
    }
  }
}

// Decodes elements [8v, 8v+8) of a row of blocks starting at `row` (shared or global memory).
// `scale`, when given, receives the block's scale d.
// ALIGNED16: `row` is 16-byte aligned (a staged row buffer).
template <int QT, bool ALIGNED16 = false>
__device__ __forceinline__ void decode8(const unsigned char* row, int v, float (&out)[8], float* scale = nullptr) {
  if constexpr (is_kquant(QT)) {
    if (scale != nullptr) *scale = 1.0f;
    decode8_kquant<QT, ALIGNED16>(row + (v >> 5) * QBlock<QT>::kBytes, v & 31, out);
    return;
  }
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
    // The sixteen quant bytes start 2 bytes into a block of 18 or 34 bytes, so they are 4-byte aligned
    // in every other block only.  Five aligned words cover them either way; a funnel shift by 0 or 16
    // bits re-aligns them (five wide loads and four shifts instead of eight 16-bit loads).
    // (`row` is 16-byte aligned: a staged row buffer)
    const int qoff = (p >> 1) * QBlock<QT>::kBytes + 2 + (QT == CB200_QTYPE_Q8_0 ? (p & 1) * 16 : 0);
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(row) + (qoff >> 2);
    const uint32_t sh = (static_cast<uint32_t>(qoff) & 2u) * 8u;
    uint32_t raw[5];
  #pragma unroll
    for (int i = 0; i < 5; ++i) raw[i] = wp[i];
    uint32_t w[4];
  #pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = __funnelshift_r(raw[i], raw[i + 1], sh);
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
