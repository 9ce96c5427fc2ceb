/*
 * CPU oracle: a plain-C restatement of the arithmetic candle's CPU backend performs on the
 * normalisation + embedding path.  TEST INFRASTRUCTURE ONLY: it is the checker the CUDA path is
 * compared against and the timed CPU baseline; the library never links or calls it.
 *
 * Parity pinning: the restatement is checked against the golden vectors held by candle's own
 * tests (candle-nn/tests/ops.rs:55-125, candle-nn/tests/layer_norm.rs:11-55,
 * candle-nn/src/layer_norm.rs:7-28, candle-core/tests/tensor_tests.rs:817-896,
 * candle-core/tests/quantized_tests.rs:222-254, and for the K-quant super-blocks :437-716, see
 * candle_cpu_kquants.h).  candle pins only f32 norms, gather and the quantise->dequantise round trips; bf16/f16 norm results and Q8_0 dequant values have no
 * golden vector in candle, so for those the oracle is "parity unpinned" by the reference and is
 * anchored on the restated `half` crate semantics (cross-checked against torch CPU casts).
 *
 * Third-party arithmetic restated here: crate `half` (>= 2.3.1, < 3): bf16/f16 <-> f32
 * conversion is IEEE round-to-nearest-even with NaNs kept (quiet bit forced); every bf16/f16
 * binary operator converts both operands to f32, applies the f32 operator and rounds back.
 *
 * Must be compiled with -ffp-contract=off and without -ffast-math: Rust never contracts a*b+c
 * into an FMA and never re-associates float sums, and the results below depend on both.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_F32 0
#define ORACLE_F16 1
#define ORACLE_BF16 2

#define ORACLE_U8 0
#define ORACLE_U32 1
#define ORACLE_I64 2

#define ORACLE_Q4_0 2 /* ggml type ids, candle-core/src/quantized/mod.rs:152-171 */
#define ORACLE_Q8_0 8

#define ORACLE_OK 0
#define ORACLE_E_DTYPE -1
#define ORACLE_E_INVALID_INDEX -2
#define ORACLE_E_SHAPE -3

static inline uint32_t f32_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static inline float bits_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* half::bf16::from_f32 / to_f32 (software path of crate `half`, bfloat/convert.rs). */
static inline uint16_t bf16_from_f32(float f) {
  uint32_t x = f32_bits(f);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u);
  uint32_t round_bit = 0x00008000u;
  if ((x & round_bit) != 0 && (x & (3 * round_bit - 1)) != 0) return (uint16_t)((x >> 16) + 1);
  return (uint16_t)(x >> 16);
}
static inline float bf16_to_f32(uint16_t h) {
  if ((h & 0x7FFFu) > 0x7F80u) return bits_f32(((uint32_t)h | 0x0040u) << 16);
  return bits_f32((uint32_t)h << 16);
}

/* half::f16::from_f32 / to_f32 (binary16/arch.rs f32_to_f16_fallback / f16_to_f32_fallback). */
static inline uint16_t f16_from_f32(float f) {
  uint32_t x = f32_bits(f);
  uint32_t sign = x & 0x80000000u;
  uint32_t exp = x & 0x7F800000u;
  uint32_t man = x & 0x007FFFFFu;
  if (exp == 0x7F800000u) {
    uint32_t nan_bit = (man == 0) ? 0 : 0x0200u;
    return (uint16_t)((sign >> 16) | 0x7C00u | nan_bit | (man >> 13));
  }
  uint32_t half_sign = sign >> 16;
  int32_t unbiased_exp = (int32_t)(exp >> 23) - 127;
  int32_t half_exp = unbiased_exp + 15;
  if (half_exp >= 0x1F) return (uint16_t)(half_sign | 0x7C00u);
  if (half_exp <= 0) {
    if (14 - half_exp > 24) return (uint16_t)half_sign;
    man |= 0x00800000u;
    uint32_t half_man = man >> (14 - half_exp);
    uint32_t round_bit = 1u << (13 - half_exp);
    if ((man & round_bit) != 0 && (man & (3 * round_bit - 1)) != 0) half_man += 1;
    return (uint16_t)(half_sign | half_man);
  }
  uint32_t half_exp_bits = (uint32_t)half_exp << 10;
  uint32_t half_man = man >> 13;
  uint32_t round_bit = 0x00001000u;
  if ((man & round_bit) != 0 && (man & (3 * round_bit - 1)) != 0)
    return (uint16_t)((half_sign | half_exp_bits | half_man) + 1);
  return (uint16_t)(half_sign | half_exp_bits | half_man);
}
static inline float f16_to_f32(uint16_t h) {
  uint32_t i = h;
  if ((i & 0x7FFFu) == 0) return bits_f32(i << 16);
  uint32_t half_sign = i & 0x8000u;
  uint32_t half_exp = i & 0x7C00u;
  uint32_t half_man = i & 0x03FFu;
  if (half_exp == 0x7C00u) {
    if (half_man == 0) return bits_f32((half_sign << 16) | 0x7F800000u);
    return bits_f32((half_sign << 16) | 0x7FC00000u | (half_man << 13));
  }
  uint32_t sign = half_sign << 16;
  int32_t unbiased_exp = ((int32_t)half_exp >> 10) - 15;
  if (half_exp == 0) {
    /* subnormal: normalise */
    uint32_t e = 0;
    uint32_t m = half_man;
    while ((m & 0x0400u) == 0) {
      m <<= 1;
      e++;
    }
    /* value = m * 2^-24 * 2^-e with m in [2^10, 2^11) */
    uint32_t exp = (uint32_t)(127 - 14 - e) << 23;
    uint32_t man = (m & 0x03FFu) << 13;
    return bits_f32(sign | exp | man);
  }
  uint32_t exp = (uint32_t)(unbiased_exp + 127) << 23;
  uint32_t man = half_man << 13;
  return bits_f32(sign | exp | man);
}

/* Exposed scalar converters (the tests cross-check them against torch's CPU casts). */
uint16_t oracle_bf16_from_f32(float f) { return bf16_from_f32(f); }
float oracle_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
uint16_t oracle_f16_from_f32(float f) { return f16_from_f32(f); }
float oracle_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

static int resolve_threads(int threads) {
#ifdef _OPENMP
  if (threads <= 0) return omp_get_max_threads();
  return threads;
#else
  (void)threads;
  return 1;
#endif
}

int oracle_max_threads(void) { return resolve_threads(0); }

/* f32 -> {f32,f16,bf16} element-wise cast: candle-core/src/cpu_backend/mod.rs:1669-1672 (bf16),
 * :1697-1700 (f16).  candle's unary_map is sequential; `threads` > 1 is a courtesy variant. */
int oracle_cast_from_f32(int dtype, const float* x, void* y, int64_t n, int threads) {
  int nt = resolve_threads(threads);
  (void)nt;
  if (dtype == ORACLE_F32) {
    memcpy(y, x, (size_t)n * 4);
    return ORACLE_OK;
  }
  if (dtype != ORACLE_F16 && dtype != ORACLE_BF16) return ORACLE_E_DTYPE;
  uint16_t* o = (uint16_t*)y;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t i = 0; i < n; i++) o[i] = dtype == ORACLE_BF16 ? bf16_from_f32(x[i]) : f16_from_f32(x[i]);
  return ORACLE_OK;
}

/* {f16,bf16} -> f32: half::{f16,bf16}::to_f32. */
int oracle_cast_to_f32(int dtype, const void* x, float* y, int64_t n, int threads) {
  int nt = resolve_threads(threads);
  (void)nt;
  if (dtype == ORACLE_F32) {
    memcpy(y, x, (size_t)n * 4);
    return ORACLE_OK;
  }
  if (dtype != ORACLE_F16 && dtype != ORACLE_BF16) return ORACLE_E_DTYPE;
  const uint16_t* in = (const uint16_t*)x;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t i = 0; i < n; i++) y[i] = dtype == ORACLE_BF16 ? bf16_to_f32(in[i]) : f16_to_f32(in[i]);
  return ORACLE_OK;
}

/* Element-wise add rounded to T: candle-core/src/op.rs:330 (`|v1, v2| v1 + v2` on T) applied by
 * binary_map, candle-core/src/cpu_backend/utils.rs:84-96 (a sequential iterator). */
int oracle_add(int dtype, const void* a, const void* b, void* out, int64_t n, int threads) {
  int nt = resolve_threads(threads);
  (void)nt;
  if (dtype == ORACLE_F32) {
    const float *pa = (const float*)a, *pb = (const float*)b;
    float* po = (float*)out;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
    for (int64_t i = 0; i < n; i++) po[i] = pa[i] + pb[i];
    return ORACLE_OK;
  }
  if (dtype != ORACLE_F16 && dtype != ORACLE_BF16) return ORACLE_E_DTYPE;
  const uint16_t *pa = (const uint16_t*)a, *pb = (const uint16_t*)b;
  uint16_t* po = (uint16_t*)out;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t i = 0; i < n; i++) {
    if (dtype == ORACLE_BF16)
      po[i] = bf16_from_f32(bf16_to_f32(pa[i]) + bf16_to_f32(pb[i]));
    else
      po[i] = f16_from_f32(f16_to_f32(pa[i]) + f16_to_f32(pb[i]));
  }
  return ORACLE_OK;
}

/* RmsNorm::cpu_fwd, candle-nn/src/ops.rs:447-508.  Per row (one rayon task per row, :481):
 *   sum2 = sum over the row, left to right in f32, of f32(v)*f32(v)          (:484-490)
 *   m    = sqrt(sum2 / n + eps) in f32, then converted to T                   (:491-492)
 *   y    = x / m * alpha evaluated in T: two T operations, each rounding      (:493-495)
 */
#define RMS_ROW_HALF(TO_F32, FROM_F32)                                   \
  do {                                                                   \
    const uint16_t* src = (const uint16_t*)x + r * cols;                 \
    uint16_t* dst = (uint16_t*)y + r * cols;                             \
    const uint16_t* al = (const uint16_t*)alpha;                         \
    float sum2 = 0.0f;                                                   \
    for (int64_t c = 0; c < cols; c++) {                                 \
      float v = TO_F32(src[c]);                                          \
      float p = v * v;                                                   \
      sum2 = sum2 + p;                                                   \
    }                                                                    \
    float m = sqrtf(sum2 / (float)cols + eps);                           \
    float mt = TO_F32(FROM_F32(m));                                      \
    for (int64_t c = 0; c < cols; c++) {                                 \
      float q = TO_F32(FROM_F32(TO_F32(src[c]) / mt));                   \
      dst[c] = FROM_F32(q * TO_F32(al[c]));                              \
    }                                                                    \
  } while (0)

int oracle_rms_norm(int dtype, const void* x, const void* alpha, void* y, int64_t rows, int64_t cols,
                    float eps, int threads) {
  int nt = resolve_threads(threads);
  (void)nt;
  if (dtype != ORACLE_F32 && dtype != ORACLE_F16 && dtype != ORACLE_BF16) return ORACLE_E_DTYPE;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t r = 0; r < rows; r++) {
    if (dtype == ORACLE_F32) {
      const float* src = (const float*)x + r * cols;
      float* dst = (float*)y + r * cols;
      const float* al = (const float*)alpha;
      float sum2 = 0.0f;
      for (int64_t c = 0; c < cols; c++) {
        float p = src[c] * src[c];
        sum2 = sum2 + p;
      }
      float m = sqrtf(sum2 / (float)cols + eps);
      for (int64_t c = 0; c < cols; c++) {
        float q = src[c] / m;
        dst[c] = q * al[c];
      }
    } else if (dtype == ORACLE_BF16) {
      RMS_ROW_HALF(bf16_to_f32, bf16_from_f32);
    } else {
      RMS_ROW_HALF(f16_to_f32, f16_from_f32);
    }
  }
  return ORACLE_OK;
}

/* LayerNorm::cpu_fwd, candle-nn/src/ops.rs:664-741.  Per row:
 *   sum += v; sum2 += v*v  (both f32, left to right, :709-715)
 *   mean = sum/n; var = sum2/n - mean*mean; inv_std = 1/sqrt(var+eps)          (:716-718)
 *   y = T((f32(x) - mean) * inv_std * f32(alpha) + f32(beta)), one rounding    (:719-726)
 */
#define LN_ROW(LOAD, STORE, TIN, TOUT)                                            \
  do {                                                                            \
    const TIN* src = (const TIN*)x + r * cols;                                    \
    TOUT* dst = (TOUT*)y + r * cols;                                              \
    const TIN* ga = (const TIN*)gamma;                                            \
    const TIN* be = (const TIN*)beta;                                             \
    float sum = 0.0f, sum2 = 0.0f;                                                \
    for (int64_t c = 0; c < cols; c++) {                                          \
      float v = LOAD(src[c]);                                                     \
      sum = sum + v;                                                              \
      float p = v * v;                                                            \
      sum2 = sum2 + p;                                                            \
    }                                                                             \
    float mean = sum / (float)cols;                                               \
    float mm = mean * mean;                                                       \
    float var = sum2 / (float)cols - mm;                                          \
    float inv_std = 1.0f / sqrtf(var + eps);                                      \
    for (int64_t c = 0; c < cols; c++) {                                          \
      float t0 = LOAD(src[c]) - mean;                                             \
      float t1 = t0 * inv_std;                                                    \
      float t2 = t1 * LOAD(ga[c]);                                                \
      float t3 = t2 + LOAD(be[c]);                                                \
      dst[c] = STORE(t3);                                                         \
    }                                                                             \
  } while (0)
#define ID_F32(v) (v)

int oracle_layer_norm(int dtype, const void* x, const void* gamma, const void* beta, void* y,
                      int64_t rows, int64_t cols, float eps, int threads) {
  int nt = resolve_threads(threads);
  (void)nt;
  if (dtype != ORACLE_F32 && dtype != ORACLE_F16 && dtype != ORACLE_BF16) return ORACLE_E_DTYPE;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t r = 0; r < rows; r++) {
    if (dtype == ORACLE_F32)
      LN_ROW(ID_F32, ID_F32, float, float);
    else if (dtype == ORACLE_BF16)
      LN_ROW(bf16_to_f32, bf16_from_f32, uint16_t, uint16_t);
    else
      LN_ROW(f16_to_f32, f16_from_f32, uint16_t, uint16_t);
  }
  return ORACLE_OK;
}

static inline int read_id(int id_dtype, const void* ids, int64_t pos, uint64_t* out) {
  switch (id_dtype) {
    case ORACLE_U8:
      *out = ((const uint8_t*)ids)[pos];
      return 0;
    case ORACLE_U32:
      *out = ((const uint32_t*)ids)[pos];
      return 0;
    case ORACLE_I64:
      /* IntDType::as_usize for i64 is `self as usize`: a negative id wraps to a huge index and
       * fails the bounds check (candle-core/src/dtype.rs, impl IntDType for i64). */
      *out = (uint64_t)((const int64_t*)ids)[pos];
      return 0;
    default:
      return -1;
  }
}

/* IndexSelect::f, candle-core/src/cpu_backend/mod.rs:510-555: a single-threaded loop over
 * (left, i) copying `right` elements; ids may be strided (:526,538); an id >= src_dim is
 * Error::InvalidIndex{index,size,op:"index-select"} (:539-546) -- reported through *bad_index. */
int oracle_index_select(int64_t elem_size, int id_dtype, const void* src, const void* ids,
                        int64_t ids_stride, void* dst, int64_t left, int64_t src_dim, int64_t right,
                        int64_t n_ids, int64_t* bad_index) {
  const char* s = (const char*)src;
  char* d = (char*)dst;
  for (int64_t l = 0; l < left; l++) {
    int64_t start_src = l * right * src_dim;
    int64_t start_dst = l * right * n_ids;
    for (int64_t i = 0; i < n_ids; i++) {
      uint64_t index;
      if (read_id(id_dtype, ids, ids_stride * i, &index)) return ORACLE_E_DTYPE;
      if (index >= (uint64_t)src_dim) {
        if (bad_index) *bad_index = (int64_t)index;
        return ORACLE_E_INVALID_INDEX;
      }
      memcpy(d + (size_t)(start_dst + i * right) * elem_size,
             s + (size_t)(start_src + (int64_t)index * right) * elem_size, (size_t)(right * elem_size));
    }
  }
  return ORACLE_OK;
}

/* Block layouts: BlockQ4_0 {d: f16, qs: [u8; 16]} = 18 bytes, BlockQ8_0 {d: f16, qs: [i8; 32]} =
 * 34 bytes, #[repr(C)], candle-core/src/quantized/k_quants.rs:42-48, 78-84. */
#define QK 32
#define Q4_0_BYTES 18
#define Q8_0_BYTES 34
/* BlockQ4_1 {d, m: f16, qs: [u8; 16]} = 20 bytes, BlockQ5_0 {d: f16, qh: [u8; 4], qs: [u8; 16]} = 22,
 * BlockQ5_1 {d, m: f16, qh: [u8; 4], qs: [u8; 16]} = 24 (k_quants.rs:50-76). */
#define ORACLE_Q4_1 3
#define ORACLE_Q5_0 6
#define ORACLE_Q5_1 7
#define Q4_1_BYTES 20
#define Q5_0_BYTES 22
#define Q5_1_BYTES 24

static inline uint32_t read_u32_le(const uint8_t* p) {
  return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

#include "candle_cpu_kquants.h"

/* elements per block: 32 for the Q4_0 .. Q8_0 family, 256 for the K-quant super-blocks */
int64_t oracle_block_elems(int qtype) { return kq_block_bytes(qtype) > 0 ? QK_K : QK; }

int64_t oracle_block_bytes(int qtype) {
  if (kq_block_bytes(qtype) > 0) return kq_block_bytes(qtype);
  if (qtype == ORACLE_Q4_0) return Q4_0_BYTES;
  if (qtype == ORACLE_Q8_0) return Q8_0_BYTES;
  if (qtype == ORACLE_Q4_1) return Q4_1_BYTES;
  if (qtype == ORACLE_Q5_0) return Q5_0_BYTES;
  if (qtype == ORACLE_Q5_1) return Q5_1_BYTES;
  return ORACLE_E_DTYPE;
}

/* GgmlType::to_float: Q4_0 k_quants.rs:163-183, Q8_0 k_quants.rs:568-584 (sequential in candle). */
int oracle_dequantize(int qtype, const void* blocks, float* y, int64_t k, int threads) {
  int nt = resolve_threads(threads);
  (void)nt;
  if (kq_block_bytes(qtype) > 0) return kq_dequantize(qtype, (const uint8_t*)blocks, y, k, nt);
  if (k % QK != 0) return ORACLE_E_SHAPE;
  int64_t nb = k / QK;
  const uint8_t* b = (const uint8_t*)blocks;
  if (qtype == ORACLE_Q4_0) {
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
    for (int64_t i = 0; i < nb; i++) {
      const uint8_t* blk = b + i * Q4_0_BYTES;
      uint16_t dh;
      memcpy(&dh, blk, 2);
      float d = f16_to_f32(dh);
      const uint8_t* qs = blk + 2;
      for (int j = 0; j < QK / 2; j++) {
        int16_t x0 = (int16_t)(qs[j] & 0x0F) - 8;
        int16_t x1 = (int16_t)(qs[j] >> 4) - 8;
        y[i * QK + j] = (float)x0 * d;
        y[i * QK + j + QK / 2] = (float)x1 * d;
      }
    }
    return ORACLE_OK;
  }
  if (qtype == ORACLE_Q8_0) {
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
    for (int64_t i = 0; i < nb; i++) {
      const uint8_t* blk = b + i * Q8_0_BYTES;
      uint16_t dh;
      memcpy(&dh, blk, 2);
      float d = f16_to_f32(dh);
      const int8_t* qs = (const int8_t*)(blk + 2);
      for (int j = 0; j < QK; j++) y[i * QK + j] = (float)qs[j] * d;
    }
    return ORACLE_OK;
  }
  if (qtype == ORACLE_Q4_1) { /* k_quants.rs:329-349: (x as f32) * d + m, two roundings */
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
    for (int64_t i = 0; i < nb; i++) {
      const uint8_t* blk = b + i * Q4_1_BYTES;
      uint16_t dh, mh;
      memcpy(&dh, blk, 2);
      memcpy(&mh, blk + 2, 2);
      float d = f16_to_f32(dh), m = f16_to_f32(mh);
      const uint8_t* qs = blk + 4;
      for (int j = 0; j < QK / 2; j++) {
        uint8_t x0 = qs[j] & 0x0F, x1 = qs[j] >> 4;
        float p0 = (float)x0 * d, p1 = (float)x1 * d;
        y[i * QK + j] = p0 + m;
        y[i * QK + j + QK / 2] = p1 + m;
      }
    }
    return ORACLE_OK;
  }
  if (qtype == ORACLE_Q5_0) { /* k_quants.rs:428-452 */
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
    for (int64_t i = 0; i < nb; i++) {
      const uint8_t* blk = b + i * Q5_0_BYTES;
      uint16_t dh;
      memcpy(&dh, blk, 2);
      float d = f16_to_f32(dh);
      uint32_t qh = read_u32_le(blk + 2);
      const uint8_t* qs = blk + 6;
      for (int j = 0; j < QK / 2; j++) {
        uint8_t xh0 = (uint8_t)(((qh >> j) << 4) & 0x10);
        uint8_t xh1 = (uint8_t)((qh >> (j + 12)) & 0x10);
        int32_t x0 = (int32_t)((qs[j] & 0x0F) | xh0) - 16;
        int32_t x1 = (int32_t)((qs[j] >> 4) | xh1) - 16;
        y[i * QK + j] = (float)x0 * d;
        y[i * QK + j + QK / 2] = (float)x1 * d;
      }
    }
    return ORACLE_OK;
  }
  if (qtype == ORACLE_Q5_1) { /* k_quants.rs:535-562 */
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
    for (int64_t i = 0; i < nb; i++) {
      const uint8_t* blk = b + i * Q5_1_BYTES;
      uint16_t dh, mh;
      memcpy(&dh, blk, 2);
      memcpy(&mh, blk + 2, 2);
      float d = f16_to_f32(dh), m = f16_to_f32(mh);
      uint32_t qh = read_u32_le(blk + 4);
      const uint8_t* qs = blk + 8;
      for (int j = 0; j < QK / 2; j++) {
        uint8_t xh0 = (uint8_t)(((qh >> j) << 4) & 0x10);
        uint8_t xh1 = (uint8_t)((qh >> (j + 12)) & 0x10);
        uint8_t x0 = (uint8_t)((qs[j] & 0x0F) | xh0), x1 = (uint8_t)((qs[j] >> 4) | xh1);
        float p0 = (float)x0 * d, p1 = (float)x1 * d;
        y[i * QK + j] = p0 + m;
        y[i * QK + j + QK / 2] = p1 + m;
      }
    }
    return ORACLE_OK;
  }
  return ORACLE_E_DTYPE;
}

/* GgmlType::from_float (the writer of the format the lookup reads): Q4_0 k_quants.rs:185-220,
 * Q8_0 k_quants.rs:586-615.  Rust's `as u8` on a float saturates; `f32::round` rounds half away
 * from zero (roundf). */
static inline uint8_t sat_u8(float v) {
  if (!(v > 0.0f)) return 0; /* also NaN -> 0 */
  if (v >= 255.0f) return 255;
  return (uint8_t)v;
}
static inline int8_t sat_i8(float v) {
  if (v != v) return 0;
  if (v <= -128.0f) return -128;
  if (v >= 127.0f) return 127;
  return (int8_t)v;
}

int oracle_quantize(int qtype, const float* x, void* blocks, int64_t k) {
  if (kq_block_bytes(qtype) > 0) return kq_quantize(qtype, x, (uint8_t*)blocks, k);
  if (k % QK != 0) return ORACLE_E_SHAPE;
  int64_t nb = k / QK;
  uint8_t* b = (uint8_t*)blocks;
  if (qtype == ORACLE_Q4_0) {
    for (int64_t i = 0; i < nb; i++) {
      const float* xs = x + i * QK;
      float amax = 0.0f, max = 0.0f;
      for (int j = 0; j < QK; j++) {
        if (amax < fabsf(xs[j])) {
          amax = fabsf(xs[j]);
          max = xs[j];
        }
      }
      float d = max / -8.0f;
      float id = d != 0.0f ? 1.0f / d : 0.0f;
      uint16_t dh = f16_from_f32(d);
      uint8_t* blk = b + i * Q4_0_BYTES;
      memcpy(blk, &dh, 2);
      for (int j = 0; j < QK / 2; j++) {
        float x0 = xs[j] * id;
        float x1 = xs[QK / 2 + j] * id;
        uint8_t xi0 = sat_u8(x0 + 8.5f);
        uint8_t xi1 = sat_u8(x1 + 8.5f);
        if (xi0 > 15) xi0 = 15;
        if (xi1 > 15) xi1 = 15;
        blk[2 + j] = (uint8_t)(xi0 | (xi1 << 4));
      }
    }
    return ORACLE_OK;
  }
  if (qtype == ORACLE_Q8_0) {
    for (int64_t i = 0; i < nb; i++) {
      const float* xs = x + i * QK;
      float amax = 0.0f;
      for (int j = 0; j < QK; j++) amax = fmaxf(amax, fabsf(xs[j]));
      float d = amax / 127.0f;
      float id = d != 0.0f ? 1.0f / d : 0.0f;
      uint16_t dh = f16_from_f32(d);
      uint8_t* blk = b + i * Q8_0_BYTES;
      memcpy(blk, &dh, 2);
      for (int j = 0; j < QK; j++) blk[2 + j] = (uint8_t)sat_i8(roundf(xs[j] * id));
    }
    return ORACLE_OK;
  }
  if (qtype == ORACLE_Q4_1 || qtype == ORACLE_Q5_1) { /* k_quants.rs:295-326, 496-532 */
    const int bits5 = qtype == ORACLE_Q5_1;
    const int bb = bits5 ? Q5_1_BYTES : Q4_1_BYTES;
    for (int64_t i = 0; i < nb; i++) {
      const float* xs = x + i * QK;
      float min = INFINITY, max = -INFINITY;
      for (int j = 0; j < QK; j++) { /* f32::min / f32::max ignore a NaN operand, like fminf / fmaxf */
        min = fminf(xs[j], min);
        max = fmaxf(xs[j], max);
      }
      float d = (max - min) / (float)((bits5 ? 32 : 16) - 1);
      float id = d != 0.0f ? 1.0f / d : 0.0f;
      uint16_t dh = f16_from_f32(d), mh = f16_from_f32(min);
      uint8_t* blk = b + i * bb;
      memcpy(blk, &dh, 2);
      memcpy(blk + 2, &mh, 2);
      uint32_t qh = 0;
      uint8_t* qs = blk + (bits5 ? 8 : 4);
      for (int j = 0; j < QK / 2; j++) {
        float x0 = (xs[j] - min) * id;
        float x1 = (xs[QK / 2 + j] - min) * id;
        uint8_t xi0 = sat_u8(x0 + 0.5f), xi1 = sat_u8(x1 + 0.5f);
        if (!bits5) {
          if (xi0 > 15) xi0 = 15;
          if (xi1 > 15) xi1 = 15;
          qs[j] = (uint8_t)(xi0 | (xi1 << 4));
        } else {
          qs[j] = (uint8_t)((xi0 & 0x0F) | ((xi1 & 0x0F) << 4));
          qh |= (((uint32_t)xi0 & 0x10u) >> 4) << j;
          qh |= (((uint32_t)xi1 & 0x10u) >> 4) << (j + QK / 2);
        }
      }
      if (bits5) {
        blk[4] = (uint8_t)qh;
        blk[5] = (uint8_t)(qh >> 8);
        blk[6] = (uint8_t)(qh >> 16);
        blk[7] = (uint8_t)(qh >> 24);
      }
    }
    return ORACLE_OK;
  }
  if (qtype == ORACLE_Q5_0) { /* k_quants.rs:392-425 */
    for (int64_t i = 0; i < nb; i++) {
      const float* xs = x + i * QK;
      float amax = 0.0f, max = 0.0f;
      for (int j = 0; j < QK; j++) {
        if (amax < fabsf(xs[j])) {
          amax = fabsf(xs[j]);
          max = xs[j];
        }
      }
      float d = max / -16.0f;
      float id = d != 0.0f ? 1.0f / d : 0.0f;
      uint16_t dh = f16_from_f32(d);
      uint8_t* blk = b + i * Q5_0_BYTES;
      memcpy(blk, &dh, 2);
      uint32_t qh = 0;
      for (int j = 0; j < QK / 2; j++) {
        float x0 = xs[j] * id;
        float x1 = xs[j + QK / 2] * id;
        int8_t s0 = sat_i8(x0 + 16.5f), s1 = sat_i8(x1 + 16.5f); /* `as i8` saturates */
        uint8_t xi0 = (uint8_t)(s0 < 31 ? s0 : 31), xi1 = (uint8_t)(s1 < 31 ? s1 : 31);
        blk[6 + j] = (uint8_t)((xi0 & 0x0F) | ((xi1 & 0x0F) << 4));
        qh |= (((uint32_t)xi0 & 0x10u) >> 4) << j;
        qh |= (((uint32_t)xi1 & 0x10u) >> 4) << (j + QK / 2);
      }
      blk[2] = (uint8_t)qh;
      blk[3] = (uint8_t)(qh >> 8);
      blk[4] = (uint8_t)(qh >> 16);
      blk[5] = (uint8_t)(qh >> 24);
    }
    return ORACLE_OK;
  }
  return ORACLE_E_DTYPE;
}

/* Row lookup out of a quantised [vocab, hidden] table as candle's models compose it:
 * QTensor::dequantize (whole table -> f32, quantized/mod.rs:361-365, as done at load in
 * candle-transformers/src/models/quantized_llama.rs:378-379), optional to_dtype(T)
 * (cpu_backend/mod.rs:1669-1672,1697-1700), then Embedding::forward = index_select on dim 0
 * (candle-nn/src/embedding.rs:29-36).  Dequantisation and the cast are element-wise, so decoding
 * only the selected rows yields the same bytes as decoding the whole table and then gathering;
 * this function does the former so that full-size tables do not need a multi-GB f32 copy. */
int oracle_qembedding(int qtype, int out_dtype, int id_dtype, const void* qtable, const void* ids,
                      void* out, int64_t vocab, int64_t hidden, int64_t n_ids, int64_t* bad_index,
                      int threads) {
  int nt = resolve_threads(threads);
  (void)nt;
  int64_t bb = oracle_block_bytes(qtype);
  if (bb < 0) return ORACLE_E_DTYPE;
  const int64_t be = oracle_block_elems(qtype);
  if (hidden % be != 0) return ORACLE_E_SHAPE;
  if (out_dtype != ORACLE_F32 && out_dtype != ORACLE_F16 && out_dtype != ORACLE_BF16) return ORACLE_E_DTYPE;
  int64_t row_bytes = hidden / be * bb;
  for (int64_t i = 0; i < n_ids; i++) {
    uint64_t index;
    if (read_id(id_dtype, ids, i, &index)) return ORACLE_E_DTYPE;
    if (index >= (uint64_t)vocab) {
      if (bad_index) *bad_index = (int64_t)index;
      return ORACLE_E_INVALID_INDEX;
    }
  }
  int rc = ORACLE_OK;
#pragma omp parallel num_threads(nt) if (nt > 1)
  {
    float* tmp = (float*)__builtin_alloca((size_t)QK_K * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t i = 0; i < n_ids; i++) {
      uint64_t index = 0;
      read_id(id_dtype, ids, i, &index);
      const uint8_t* row = (const uint8_t*)qtable + (size_t)index * row_bytes;
      for (int64_t blk = 0; blk < hidden / be; blk++) {
        oracle_dequantize(qtype, row + blk * bb, tmp, be, 1);
        size_t o = (size_t)i * hidden + blk * be;
        if (out_dtype == ORACLE_F32)
          memcpy((float*)out + o, tmp, be * sizeof(float));
        else
          oracle_cast_from_f32(out_dtype, tmp, (uint16_t*)out + o, be, 1);
      }
    }
  }
  return rc;
}

/* ------------------------------------------------------------------------------------------------
 * The composite ("slow") norm: LayerNorm::forward when the fused op does not apply
 * (candle-nn/src/layer_norm.rs:108-136; the same chain as ops::rms_norm_slow / layer_norm_slow,
 * candle-nn/src/ops.rs:628-639, 876-894).  Each line is one candle tensor op on f32 data:
 *   x      = to_dtype(F32)
 *   mean   = sum_keepdim(x) / n       -> `Tensor / f64` is affine(1/n, 0): fl(fl(s * f32(1/n)) + 0)
 *                                        (candle-core/src/tensor.rs:2656, cpu_backend/mod.rs:291-299)
 *   x      = x - mean                 (only when remove_mean)
 *   norm   = sum_keepdim(x*x) / n     (same affine)
 *   d      = sqrt(norm + eps)         -> `Tensor + f64` is affine(1, eps): fl(fl(v * 1) + f32(eps))
 *   y      = T(x / d) * weight [+ bias]   (the product and the sum are T operations, each rounding)
 * sum_keepdim over the last dimension of a contiguous f32 tensor is ReduceSum -> vec_reduce_sum ->
 * vec_sum (candle-core/src/cpu_backend/mod.rs:213-260, candle-core/src/cpu/kernels.rs:79-81).  With
 * AVX (candle builds with target-cpu=native, .cargo/config.toml) vec_sum keeps four 8-lane
 * accumulators -- accumulator j lane l takes elements 32 i + 8 j + l in increasing i -- and folds
 * them as (a0 + a1) + (a2 + a3), then low half + high half, then two horizontal adds; the k % 32
 * leftovers are added one by one (candle-core/src/cpu/mod.rs:113-135, cpu/avx.rs:54-66).  That AVX
 * order is what is restated here; a build without SIMD would add left to right instead.
 */
static float avx_vec_sum(const float* row, int64_t k) {
  float acc[32];
  for (int i = 0; i < 32; i++) acc[i] = 0.0f;
  int64_t np = k & ~(int64_t)31;
  for (int64_t i = 0; i < np; i += 32)
    for (int l = 0; l < 32; l++) acc[l] = acc[l] + row[i + l];
  float r8[8], t0[4];
  for (int l = 0; l < 8; l++) {
    float a01 = acc[l] + acc[8 + l];
    float a23 = acc[16 + l] + acc[24 + l];
    r8[l] = a01 + a23;
  }
  for (int l = 0; l < 4; l++) t0[l] = r8[l] + r8[l + 4];
  float h0 = t0[0] + t0[1], h1 = t0[2] + t0[3];
  float b = h0 + h1;
  for (int64_t i = np; i < k; i++) b = b + row[i];
  return b;
}

float oracle_avx_vec_sum(const float* row, int64_t k) { return avx_vec_sum(row, k); }

int oracle_norm_slow(int dtype, const void* x, const void* weight, const void* bias, void* y, int64_t rows,
                     int64_t cols, double eps, int remove_mean, int threads) {
  int nt = resolve_threads(threads);
  (void)nt;
  if (dtype != ORACLE_F32 && dtype != ORACLE_F16 && dtype != ORACLE_BF16) return ORACLE_E_DTYPE;
  const float inv_n = (float)(1.0 / (double)cols); /* T::from_f64(1. / rhs) */
  const float eps32 = (float)eps;
  int rc = ORACLE_OK;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t r = 0; r < rows; r++) {
    float stack_buf[2048];
    float* xf = cols <= 1024 ? stack_buf : (float*)malloc((size_t)cols * 2 * sizeof(float));
    if (xf == NULL) {
      rc = ORACLE_E_SHAPE;
      continue;
    }
    float* sq = xf + cols;
    for (int64_t c = 0; c < cols; c++) {
      if (dtype == ORACLE_F32)
        xf[c] = ((const float*)x)[r * cols + c];
      else if (dtype == ORACLE_BF16)
        xf[c] = bf16_to_f32(((const uint16_t*)x)[r * cols + c]);
      else
        xf[c] = f16_to_f32(((const uint16_t*)x)[r * cols + c]);
    }
    if (remove_mean) {
      float s = avx_vec_sum(xf, cols);
      float sm = s * inv_n;
      float mean = sm + 0.0f;
      for (int64_t c = 0; c < cols; c++) xf[c] = xf[c] - mean;
    }
    for (int64_t c = 0; c < cols; c++) sq[c] = xf[c] * xf[c];
    float q = avx_vec_sum(sq, cols);
    float qm = q * inv_n;
    float norm = qm + 0.0f;
    float n1 = norm * 1.0f;
    float d = sqrtf(n1 + eps32);
    for (int64_t c = 0; c < cols; c++) {
      float xn = xf[c] / d;
      if (dtype == ORACLE_F32) {
        float t = xn * ((const float*)weight)[c];
        if (bias != NULL) t = t + ((const float*)bias)[c];
        ((float*)y)[r * cols + c] = t;
      } else if (dtype == ORACLE_BF16) {
        uint16_t t = bf16_from_f32(xn);
        t = bf16_from_f32(bf16_to_f32(t) * bf16_to_f32(((const uint16_t*)weight)[c]));
        if (bias != NULL) t = bf16_from_f32(bf16_to_f32(t) + bf16_to_f32(((const uint16_t*)bias)[c]));
        ((uint16_t*)y)[r * cols + c] = t;
      } else {
        uint16_t t = f16_from_f32(xn);
        t = f16_from_f32(f16_to_f32(t) * f16_to_f32(((const uint16_t*)weight)[c]));
        if (bias != NULL) t = f16_from_f32(f16_to_f32(t) + f16_to_f32(((const uint16_t*)bias)[c]));
        ((uint16_t*)y)[r * cols + c] = t;
      }
    }
    if (xf != stack_buf) free(xf);
  }
  return rc;
}

/* ------------------------------------------------------------------------------------------------
 * softmax over the last dimension: SoftmaxLastDim::cpu_fwd, candle-nn/src/ops.rs:296-333.  Per row
 * (a rayon task), everything in T:
 *   max = vec_reduce_max(row)                 (f32::max / half's max: a NaN operand is ignored)
 *   d[i] = (x[i] - max).exp()                 (T subtraction; exp of half types = T(expf(f32(v))))
 *   sum = vec_reduce_sum(d)                   (f32: the AVX-ordered vec_sum above; f16 / bf16: the
 *                                              default `*res += x`, i.e. a T-rounded add per element,
 *                                              candle-core/src/cpu/kernels.rs:26-31, 84-123)
 *   d[i] /= sum                               (T division)
 * expf is the platform's libm, as it is for candle (Rust's f32::exp calls it).
 */
#define SOFTMAX_ROW_HALF(TO_F32, FROM_F32)                                                   \
  do {                                                                                       \
    const uint16_t* src = (const uint16_t*)x + r * cols;                                     \
    uint16_t* dst = (uint16_t*)y + r * cols;                                                 \
    float max = TO_F32(src[0]);                                                              \
    for (int64_t c = 1; c < cols; c++) max = fmaxf(max, TO_F32(src[c]));                     \
    for (int64_t c = 0; c < cols; c++) {                                                     \
      float dlt = TO_F32(FROM_F32(TO_F32(src[c]) - max));                                    \
      dst[c] = FROM_F32(expf(dlt));                                                          \
    }                                                                                        \
    uint16_t sum = FROM_F32(0.0f);                                                           \
    for (int64_t c = 0; c < cols; c++) sum = FROM_F32(TO_F32(sum) + TO_F32(dst[c]));         \
    for (int64_t c = 0; c < cols; c++) dst[c] = FROM_F32(TO_F32(dst[c]) / TO_F32(sum));      \
  } while (0)

int oracle_softmax_last_dim(int dtype, const void* x, void* y, int64_t rows, int64_t cols, int threads) {
  int nt = resolve_threads(threads);
  (void)nt;
  if (dtype != ORACLE_F32 && dtype != ORACLE_F16 && dtype != ORACLE_BF16) return ORACLE_E_DTYPE;
  if (cols <= 0) return rows == 0 ? ORACLE_OK : ORACLE_E_SHAPE;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t r = 0; r < rows; r++) {
    if (dtype == ORACLE_F32) {
      const float* src = (const float*)x + r * cols;
      float* dst = (float*)y + r * cols;
      float max = src[0];
      for (int64_t c = 1; c < cols; c++) max = fmaxf(max, src[c]);
      for (int64_t c = 0; c < cols; c++) {
        float dlt = src[c] - max;
        dst[c] = expf(dlt);
      }
      float sum = avx_vec_sum(dst, cols);
      for (int64_t c = 0; c < cols; c++) dst[c] = dst[c] / sum;
    } else if (dtype == ORACLE_BF16) {
      SOFTMAX_ROW_HALF(bf16_to_f32, bf16_from_f32);
    } else {
      SOFTMAX_ROW_HALF(f16_to_f32, f16_from_f32);
    }
  }
  return ORACLE_OK;
}

/* ------------------------------------------------------------------------------------------------
 * Rotary embeddings, the three fused forms of candle-nn/src/rotary_emb.rs, all arithmetic in T with
 * every product and the sum / difference rounded separately (Rust never fuses them):
 *   variant 0  rope_i   (:47-60)   src [b, h, t, d], pairs interleaved: (x[2k], x[2k+1]) with cos/sin[i_t, k]
 *   variant 1  rope     (:288-305) src [b, h, t, d], pairs (x[k], x[k + d/2])
 *   variant 2  rope_thd (:540-558) src [b, t, h, d], pairs (x[k], x[k + d/2])
 *   y1 = x1 * cos - x2 * sin;  y2 = x1 * sin + x2 * cos;   cos, sin: [t, d/2] (more rows are allowed)
 */
#define ROPE_PAIR(LOAD, STORE, T)                                                    \
  do {                                                                               \
    const T* s = (const T*)src;                                                      \
    T* o = (T*)dst;                                                                  \
    float x1 = LOAD(s[i1]), x2 = LOAD(s[i2]);                                        \
    float c = LOAD(((const T*)cos_)[ics]), sn = LOAD(((const T*)sin_)[ics]);         \
    float p1 = LOAD(STORE(x1 * c)), p2 = LOAD(STORE(x2 * sn));                       \
    float p3 = LOAD(STORE(x1 * sn)), p4 = LOAD(STORE(x2 * c));                       \
    o[i1] = STORE(p1 - p2);                                                          \
    o[i2] = STORE(p3 + p4);                                                          \
  } while (0)

int oracle_rope(int variant, int dtype, const void* src, const void* cos_, const void* sin_, void* dst, int64_t b,
                int64_t h, int64_t t, int64_t d, int threads) {
  int nt = resolve_threads(threads);
  (void)nt;
  if (dtype != ORACLE_F32 && dtype != ORACLE_F16 && dtype != ORACLE_BF16) return ORACLE_E_DTYPE;
  if (variant < 0 || variant > 2 || d % 2 != 0) return ORACLE_E_SHAPE;
  const int64_t outer = variant == 2 ? b : b * h; /* one rayon task per [t, d] (rope, rope_i) or [t, h, d] slab */
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t ob = 0; ob < outer; ob++) {
    const int64_t base = ob * (variant == 2 ? t * h * d : t * d);
    for (int64_t it = 0; it < t; it++) {
      for (int64_t id = 0; id < d / 2; id++) {
        const int64_t ics = it * (d / 2) + id;
        for (int64_t ih = 0; ih < (variant == 2 ? h : 1); ih++) {
          int64_t i1, i2;
          if (variant == 0) {
            i1 = base + it * d + 2 * id;
            i2 = i1 + 1;
          } else if (variant == 1) {
            i1 = base + it * d + id;
            i2 = i1 + d / 2;
          } else {
            i1 = base + it * h * d + ih * d + id;
            i2 = i1 + d / 2;
          }
          if (dtype == ORACLE_F32)
            ROPE_PAIR(ID_F32, ID_F32, float);
          else if (dtype == ORACLE_BF16)
            ROPE_PAIR(bf16_to_f32, bf16_from_f32, uint16_t);
          else
            ROPE_PAIR(f16_to_f32, f16_from_f32, uint16_t);
        }
      }
    }
  }
  return ORACLE_OK;
}
