/*
 * CPU oracle, part 2: the 256-element "K-quant" super-blocks of candle-core/src/quantized/k_quants.rs,
 * decoders (GgmlType::to_float) and writers (GgmlType::from_float), restated in plain C.  Included by
 * candle_cpu_oracle.c after its f16 helpers.  TEST INFRASTRUCTURE ONLY.
 *
 * Parity pinning: candle's tests quantise a known ramp with from_float, decode it with to_float and
 * compare six of the values (rounded to three decimals) plus error bounds over the whole vector
 * (candle-core/tests/quantized_tests.rs:437-716, quantize_q2k .. quantize_q8k); the restated writers
 * and decoders reproduce those values (tests/test_kquants.py).  Block layouts (#[repr(C)], little
 * endian, k_quants.rs:96-154):
 *   BlockQ2K { scales: [u8; 16], qs: [u8; 64], d: f16, dmin: f16 }                        84 bytes
 *   BlockQ3K { hmask: [u8; 32], qs: [u8; 64], scales: [u8; 12], d: f16 }                 110 bytes
 *   BlockQ4K { d: f16, dmin: f16, scales: [u8; 12], qs: [u8; 128] }                      144 bytes
 *   BlockQ5K { d: f16, dmin: f16, scales: [u8; 12], qh: [u8; 32], qs: [u8; 128] }        176 bytes
 *   BlockQ6K { ql: [u8; 128], qh: [u8; 64], scales: [i8; 16], d: f16 }                   210 bytes
 *   BlockQ8K { d: f32, qs: [i8; 256], bsums: [i16; 16] }                                 292 bytes
 */
#define QK_K 256
#define ORACLE_Q2K 10 /* ggml type ids, candle-core/src/quantized/mod.rs:152-171 */
#define ORACLE_Q3K 11
#define ORACLE_Q4K 12
#define ORACLE_Q5K 13
#define ORACLE_Q6K 14
#define ORACLE_Q8K 15
#define Q2K_BYTES 84
#define Q3K_BYTES 110
#define Q4K_BYTES 144
#define Q5K_BYTES 176
#define Q6K_BYTES 210
#define Q8K_BYTES 292

static int64_t kq_block_bytes(int qtype) {
  switch (qtype) {
    case ORACLE_Q2K: return Q2K_BYTES;
    case ORACLE_Q3K: return Q3K_BYTES;
    case ORACLE_Q4K: return Q4K_BYTES;
    case ORACLE_Q5K: return Q5K_BYTES;
    case ORACLE_Q6K: return Q6K_BYTES;
    case ORACLE_Q8K: return Q8K_BYTES;
    default: return -1;
  }
}

static inline float load_f16(const uint8_t* p) {
  uint16_t h;
  memcpy(&h, p, 2);
  return f16_to_f32(h);
}
static inline void store_f16(uint8_t* p, float v) {
  uint16_t h = f16_from_f32(v);
  memcpy(p, &h, 2);
}

/* utils.rs:49-59 */
static inline void get_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) {
    *d = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

/* ---- decoders ---------------------------------------------------------------------------------- */

/* BlockQ2K::to_float, k_quants.rs:834-871: y = dl * q - ml with dl = d * (sc & 15), ml = min * (sc >> 4) */
static void kq_dequant_q2k(const uint8_t* b, float* y) {
  const uint8_t *scales = b, *qs = b + 16;
  const float d = load_f16(b + 80), min = load_f16(b + 82);
  int is = 0;
  for (int n = 0; n < 2; n++) {
    const uint8_t* q = qs + 32 * n;
    float* yb = y + 128 * n;
    int idx = 0;
    for (int shift = 0; shift < 8; shift += 2) {
      for (int half = 0; half < 2; half++) {
        const uint8_t sc = scales[is++];
        const float dl = d * (float)(sc & 0xF);
        const float ml = min * (float)(sc >> 4);
        for (int l = 0; l < 16; l++) {
          const float p = dl * (float)((q[16 * half + l] >> shift) & 3);
          yb[idx++] = p - ml;
        }
      }
    }
  }
}

/* BlockQ3K::to_float, k_quants.rs:1095-1149 */
static void kq_dequant_q3k(const uint8_t* b, float* y) {
  const uint8_t *hmask = b, *qs = b + 32, *sc12 = b + 96;
  const float d_all = load_f16(b + 108);
  const uint32_t kmask1 = 0x03030303u, kmask2 = 0x0f0f0f0fu;
  uint32_t aux[4];
  for (int i = 0; i < 3; i++) aux[i] = read_u32_le(sc12 + 4 * i);
  const uint32_t tmp = aux[2];
  aux[2] = ((aux[0] >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4);
  aux[3] = ((aux[1] >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4);
  aux[0] = (aux[0] & kmask2) | (((tmp) & kmask1) << 4);
  aux[1] = (aux[1] & kmask2) | (((tmp >> 2) & kmask1) << 4);
  int8_t scales[16];
  for (int i = 0; i < 16; i++) scales[i] = (int8_t)((aux[i / 4] >> (8 * (i % 4))) & 0xFF);
  uint8_t m = 1;
  int is = 0;
  for (int n = 0; n < 2; n++) {
    const uint8_t* q = qs + 32 * n;
    float* yb = y + 128 * n;
    for (int shift = 0, j = 0; j < 4; j++, shift += 2) {
      for (int half = 0; half < 2; half++) {
        const float dl = d_all * ((float)scales[is] - 32.0f);
        for (int i = 0; i < 16; i++) {
          const int8_t lo = (int8_t)((q[i + 16 * half] >> shift) & 3);
          const int8_t v = (int8_t)(lo - ((hmask[i + 16 * half] & m) == 0 ? 4 : 0));
          yb[32 * j + 16 * half + i] = dl * (float)v;
        }
        is++;
      }
      m = (uint8_t)(m << 1);
    }
  }
}

/* BlockQ4K::to_float, k_quants.rs:1313-1342: y = d1 * q - m1 */
static void kq_dequant_q4k(const uint8_t* b, float* y) {
  const float d = load_f16(b), min = load_f16(b + 2);
  const uint8_t *scales = b + 4, *qs = b + 16;
  int is = 0, idx = 0;
  for (int j = 0; j < QK_K; j += 64) {
    const uint8_t* q = qs + j / 2;
    uint8_t sc, m;
    get_scale_min_k4(is, scales, &sc, &m);
    const float d1 = d * (float)sc, m1 = min * (float)m;
    get_scale_min_k4(is + 1, scales, &sc, &m);
    const float d2 = d * (float)sc, m2 = min * (float)m;
    for (int l = 0; l < 32; l++) {
      const float p = d1 * (float)(q[l] & 0xF);
      y[idx++] = p - m1;
    }
    for (int l = 0; l < 32; l++) {
      const float p = d2 * (float)(q[l] >> 4);
      y[idx++] = p - m2;
    }
    is += 2;
  }
}

/* BlockQ5K::to_float, k_quants.rs:1528-1563: y = d1 * ((ql & 15) + (qh bit ? 16 : 0)) - m1 */
static void kq_dequant_q5k(const uint8_t* b, float* y) {
  const float d = load_f16(b), min = load_f16(b + 2);
  const uint8_t *scales = b + 4, *qh = b + 16, *qs = b + 48;
  int is = 0, idx = 0;
  uint8_t u1 = 1, u2 = 2;
  for (int j = 0; j < QK_K; j += 64) {
    const uint8_t* ql = qs + j / 2;
    uint8_t sc, m;
    get_scale_min_k4(is, scales, &sc, &m);
    const float d1 = d * (float)sc, m1 = min * (float)m;
    get_scale_min_k4(is + 1, scales, &sc, &m);
    const float d2 = d * (float)sc, m2 = min * (float)m;
    for (int l = 0; l < 32; l++) {
      const float q = (float)(ql[l] & 0xF) + ((qh[l] & u1) != 0 ? 16.0f : 0.0f);
      const float p = d1 * q;
      y[idx++] = p - m1;
    }
    for (int l = 0; l < 32; l++) {
      const float q = (float)(ql[l] >> 4) + ((qh[l] & u2) != 0 ? 16.0f : 0.0f);
      const float p = d2 * q;
      y[idx++] = p - m2;
    }
    is += 2;
    u1 = (uint8_t)(u1 << 2);
    u2 = (uint8_t)(u2 << 2);
  }
}

/* BlockQ6K::to_float, k_quants.rs:1716-1746: y = (d * sc) * q, two roundings */
static void kq_dequant_q6k(const uint8_t* b, float* y) {
  const uint8_t *ql0 = b, *qh0 = b + 128;
  const int8_t* sc0 = (const int8_t*)(b + 192);
  const float d = load_f16(b + 208);
  for (int n = 0; n < QK_K; n += 128) {
    const int idx = n / 128;
    float* ys = y + n;
    const int8_t* sc = sc0 + 8 * idx;
    const uint8_t *ql = ql0 + 64 * idx, *qh = qh0 + 32 * idx;
    for (int l = 0; l < 32; l++) {
      const int is = l / 16;
      const int8_t q1 = (int8_t)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
      const int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
      const int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      const float s1 = d * (float)sc[is], s2 = d * (float)sc[is + 2], s3 = d * (float)sc[is + 4],
                  s4 = d * (float)sc[is + 6];
      ys[l] = s1 * (float)q1;
      ys[l + 32] = s2 * (float)q2;
      ys[l + 64] = s3 * (float)q3;
      ys[l + 96] = s4 * (float)q4;
    }
  }
}

/* BlockQ8K::to_float, k_quants.rs:1827-1839 */
static void kq_dequant_q8k(const uint8_t* b, float* y) {
  float d;
  memcpy(&d, b, 4);
  const int8_t* qs = (const int8_t*)(b + 4);
  for (int j = 0; j < QK_K; j++) y[j] = d * (float)qs[j];
}

static int kq_dequantize(int qtype, const uint8_t* blocks, float* y, int64_t k, int nt) {
  const int64_t bb = kq_block_bytes(qtype);
  if (bb < 0) return ORACLE_E_DTYPE;
  if (k % QK_K != 0) return ORACLE_E_SHAPE;
  const int64_t nb = k / QK_K;
  (void)nt;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t i = 0; i < nb; i++) {
    const uint8_t* b = blocks + i * bb;
    float* yo = y + i * QK_K;
    switch (qtype) {
      case ORACLE_Q2K: kq_dequant_q2k(b, yo); break;
      case ORACLE_Q3K: kq_dequant_q3k(b, yo); break;
      case ORACLE_Q4K: kq_dequant_q4k(b, yo); break;
      case ORACLE_Q5K: kq_dequant_q5k(b, yo); break;
      case ORACLE_Q6K: kq_dequant_q6k(b, yo); break;
      default: kq_dequant_q8k(b, yo); break;
    }
  }
  return ORACLE_OK;
}

/* ---- writers ----------------------------------------------------------------------------------- */

/* Rust `as i32` on a float saturates and maps NaN to 0; f32::round rounds half away from zero. */
static inline int32_t nearest_int(float v) { /* utils.rs:3-5 */
  const float r = roundf(v);
  if (r != r) return 0;
  if (r >= 2147483648.0f) return INT32_MAX;
  if (r <= -2147483648.0f) return INT32_MIN;
  return (int32_t)r;
}
static inline int32_t clampi(int32_t v, int32_t lo, int32_t hi) { return v < lo ? lo : (v > hi ? hi : v); }
/* f32::max / f32::min: a NaN operand is ignored (fmaxf / fminf semantics) */

/* utils.rs:61-211 */
static float make_qx_quants(int n, int nmax, const float* x, int8_t* ls, int rmse_type) {
  float max = 0.0f, amax = 0.0f;
  for (int i = 0; i < n; i++) {
    const float ax = fabsf(x[i]);
    if (ax > amax) {
      amax = ax;
      max = x[i];
    }
  }
  if (amax == 0.0f) {
    for (int i = 0; i < n; i++) ls[i] = 0;
    return 0.0f;
  }
  float iscale = -(float)nmax / max;
  if (rmse_type == 0) {
    for (int i = 0; i < n; i++) ls[i] = (int8_t)(nmax + clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1));
    return 1.0f / iscale;
  }
  const int weight_type = rmse_type % 2;
  float sumlx = 0.0f, suml2 = 0.0f;
  for (int i = 0; i < n; i++) {
    const int l = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
    ls[i] = (int8_t)(l + nmax);
    const float w = weight_type == 1 ? x[i] * x[i] : 1.0f;
    const float lf = (float)l;
    const float wx = w * x[i], wl = w * lf;
    sumlx += wx * lf;
    suml2 += wl * lf;
  }
  float scale = sumlx / suml2;
  float best = scale * sumlx;
  for (int itry = 0; itry < 3; itry++) {
    const float is2 = 1.0f / scale;
    float slx = 0.0f, sl2 = 0.0f;
    int changed = 0;
    for (int i = 0; i < n; i++) {
      const int l = clampi(nearest_int(is2 * x[i]), -nmax, nmax - 1);
      if (l + nmax != (int)ls[i]) changed = 1;
      const float w = weight_type == 1 ? x[i] * x[i] : 1.0f;
      const float lf = (float)l;
      const float wx = w * x[i], wl = w * lf;
      slx += wx * lf;
      sl2 += wl * lf;
    }
    if (!changed || sl2 == 0.0f || slx * slx <= best * sl2) break;
    for (int i = 0; i < n; i++) ls[i] = (int8_t)(nmax + clampi(nearest_int(is2 * x[i]), -nmax, nmax - 1));
    sumlx = slx;
    suml2 = sl2;
    scale = sumlx / suml2;
    best = scale * sumlx;
  }
  for (int itry = 0; itry < 5; itry++) {
    int n_changed = 0;
    for (int i = 0; i < n; i++) {
      const float w = weight_type == 1 ? x[i] * x[i] : 1.0f;
      const int l = (int)ls[i] - nmax;
      const float wx = w * x[i];
      float slx = sumlx - wx * (float)l;
      if (slx > 0.0f) {
        const float wl = w * (float)l;
        float sl2 = suml2 - wl * (float)l;
        const float xs = x[i] * sl2;
        const int new_l = clampi(nearest_int(xs / slx), -nmax, nmax - 1);
        if (new_l != l) {
          slx += wx * (float)new_l;
          const float wn = w * (float)new_l;
          sl2 += wn * (float)new_l;
          const float lhs = (slx * slx) * suml2, rhs = (sumlx * sumlx) * sl2;
          if (sl2 > 0.0f && lhs > rhs) {
            ls[i] = (int8_t)(nmax + new_l);
            sumlx = slx;
            suml2 = sl2;
            scale = sumlx / suml2;
            best = scale * sumlx;
            n_changed++;
          }
        }
      }
    }
    if (n_changed == 0) break;
  }
  if (rmse_type < 3) return scale;
  for (int is = -4; is < 4; is++) {
    if (is == 0) continue;
    const float t = 0.1f * (float)is;
    iscale = -((float)nmax + t) / max;
    float slx = 0.0f, sl2 = 0.0f;
    for (int i = 0; i < n; i++) {
      const int l = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
      const float w = weight_type == 1 ? x[i] * x[i] : 1.0f;
      const float lf = (float)l;
      const float wx = w * x[i], wl = w * lf;
      slx += wx * lf;
      sl2 += wl * lf;
    }
    if (sl2 > 0.0f && slx * slx > best * sl2) {
      for (int i = 0; i < n; i++) ls[i] = (int8_t)(nmax + clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1));
      scale = slx / sl2;
      best = scale * slx;
    }
  }
  return scale;
}

/* utils.rs:214-267: returns (scale, -min) */
static void make_qkx1_quants(int nmax, int ntry, const float* x, int n, float* scale_out, float* min_out) {
  uint8_t l[QK_K];
  memset(l, 0, sizeof(l));
  float min = x[0], max = x[0];
  for (int i = 1; i < n; i++) { /* total_cmp order; ties are bit-identical values */
    if (x[i] < min) min = x[i];
    if (x[i] > max) max = x[i];
  }
  if (max == min) {
    *scale_out = 0.0f;
    *min_out = 0.0f;
    return;
  }
  min = fminf(min, 0.0f);
  float iscale = (float)nmax / (max - min);
  float scale = 1.0f / iscale;
  for (int t = 0; t < ntry; t++) {
    float sumlx = 0.0f;
    int32_t suml2 = 0;
    int did_change = 0;
    for (int i = 0; i < n; i++) {
      const float v = x[i] - min;
      const int32_t li = clampi(nearest_int(iscale * v), 0, nmax);
      if ((uint8_t)li != l[i]) {
        l[i] = (uint8_t)li;
        did_change = 1;
      }
      sumlx += v * (float)li;
      suml2 += li * li;
    }
    scale = sumlx / (float)suml2;
    float sum = 0.0f;
    for (int i = 0; i < n; i++) {
      const float p = scale * (float)l[i];
      sum += x[i] - p;
    }
    min = sum / (float)n;
    if (min > 0.0f) min = 0.0f;
    iscale = 1.0f / scale;
    if (!did_change) break;
  }
  *scale_out = scale;
  *min_out = -min;
}

/* utils.rs:270-329 with do_rmse == true (the only use, k_quants.rs:1015) */
static float make_q3_quants(const float* x, int n, int nmax) {
  int8_t l[QK_K];
  memset(l, 0, sizeof(l));
  float max = 0.0f, amax = 0.0f;
  for (int i = 0; i < n; i++) {
    const float ax = fabsf(x[i]);
    if (ax > amax) {
      amax = ax;
      max = x[i];
    }
  }
  if (amax == 0.0f) return 0.0f;
  const float iscale = -(float)nmax / max;
  float sumlx = 0.0f, suml2 = 0.0f;
  for (int i = 0; i < n; i++) {
    const int32_t li = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
    l[i] = (int8_t)li;
    const float w = x[i] * x[i];
    const float wx = w * x[i];
    sumlx += wx * (float)li;
    suml2 += w * (float)(li * li);
  }
  for (int t = 0; t < 5; t++) {
    int n_changed = 0;
    for (int i = 0; i < n; i++) {
      const float w = x[i] * x[i];
      const float wx = w * x[i];
      float slx = sumlx - wx * (float)l[i];
      if (slx > 0.0f) {
        float sl2 = suml2 - w * (float)((int32_t)l[i] * (int32_t)l[i]);
        const float xs = x[i] * sl2;
        const int32_t new_l = clampi(nearest_int(xs / slx), -nmax, nmax - 1);
        if (new_l != (int32_t)l[i]) {
          slx += wx * (float)new_l;
          sl2 += w * (float)(new_l * new_l);
          const float lhs = (slx * slx) * suml2, rhs = (sumlx * sumlx) * sl2;
          if (sl2 > 0.0f && lhs > rhs) {
            l[i] = (int8_t)new_l;
            sumlx = slx;
            suml2 = sl2;
            n_changed++;
          }
        }
      }
    }
    if (n_changed == 0) break;
  }
  return sumlx / suml2;
}

static inline float fold_max0(const float* v, int n) { /* iter().fold(0.0, |max, &val| val.max(max)) */
  float m = 0.0f;
  for (int i = 0; i < n; i++) m = fmaxf(v[i], m);
  return m;
}

/* the 6-bit scale / min packing shared by Q4K and Q5K, k_quants.rs:1272-1284, 1470-1482 */
static void pack_scales_k4(const float* scales, const float* mins, float max_scale, float max_min, uint8_t* out) {
  const float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
  const float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
  memset(out, 0, 12);
  for (int j = 0; j < QK_K / 32; j++) {
    int32_t a = nearest_int(inv_scale * scales[j]), c = nearest_int(inv_min * mins[j]);
    const uint8_t ls = (uint8_t)(a < 63 ? a : 63), lm = (uint8_t)(c < 63 ? c : 63);
    if (j < 4) {
      out[j] = ls;
      out[j + 4] = lm;
    } else {
      out[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
      out[j - 4] |= (uint8_t)((ls >> 4) << 6);
      out[j] |= (uint8_t)((lm >> 4) << 6);
    }
  }
}

/* BlockQ2K::from_float, k_quants.rs:769-832 */
static void kq_quant_q2k(const float* x, uint8_t* b) {
  uint8_t *bscales = b, *qs = b + 16;
  float mins[16], scales[16];
  for (int j = 0; j < 16; j++) make_qkx1_quants(3, 5, x + 16 * j, 16, &scales[j], &mins[j]);
  const float max_scale = fold_max0(scales, 16), max_min = fold_max0(mins, 16);
  if (max_scale > 0.0f) {
    const float iscale = 15.0f / max_scale;
    for (int j = 0; j < 16; j++) bscales[j] = (uint8_t)nearest_int(iscale * scales[j]);
    store_f16(b + 80, max_scale / 15.0f);
  } else {
    memset(bscales, 0, 16);
    store_f16(b + 80, 0.0f);
  }
  if (max_min > 0.0f) {
    const float iscale = 15.0f / max_min;
    for (int j = 0; j < 16; j++) bscales[j] |= (uint8_t)((uint8_t)nearest_int(iscale * mins[j]) << 4);
    store_f16(b + 82, max_min / 15.0f);
  } else {
    store_f16(b + 82, 0.0f);
  }
  uint8_t big_l[QK_K];
  memset(big_l, 0, sizeof(big_l));
  const float bd = load_f16(b + 80), bdmin = load_f16(b + 82);
  for (int j = 0; j < 16; j++) {
    const float d = bd * (float)(bscales[j] & 0xF);
    if (d == 0.0f) continue;
    const float dm = bdmin * (float)(bscales[j] >> 4);
    for (int ii = 0; ii < 16; ii++) {
      const float v = x[16 * j + ii] + dm;
      big_l[16 * j + ii] = (uint8_t)clampi(nearest_int(v / d), 0, 3);
    }
  }
  for (int j = 0; j < QK_K; j += 128)
    for (int ll = 0; ll < 32; ll++)
      qs[j / 4 + ll] = (uint8_t)(big_l[j + ll] | (big_l[j + ll + 32] << 2) | (big_l[j + ll + 64] << 4) |
                                 (big_l[j + ll + 96] << 6));
}

/* BlockQ3K::from_float, k_quants.rs:1011-1093 */
static void kq_quant_q3k(const float* x, uint8_t* b) {
  uint8_t *hmask = b, *qs = b + 32, *bscales = b + 96;
  float scales[16];
  for (int j = 0; j < 16; j++) scales[j] = make_q3_quants(x + 16 * j, 16, 4);
  float max_scale = 0.0f;
  for (int j = 0; j < 16; j++)
    if (fabsf(scales[j]) > fabsf(max_scale)) max_scale = scales[j];
  memset(bscales, 0, 12);
  if (max_scale != 0.0f) {
    const float iscale = -32.0f / max_scale;
    for (int j = 0; j < 16; j++) {
      int32_t l_val = clampi(nearest_int(iscale * scales[j]), -32, 31) + 32;
      if (j < 8)
        bscales[j] = (uint8_t)(l_val & 0xF);
      else
        bscales[j - 8] |= (uint8_t)((l_val & 0xF) << 4);
      l_val >>= 4;
      bscales[j % 4 + 8] |= (uint8_t)(l_val << (2 * (j / 4)));
    }
    store_f16(b + 108, 1.0f / iscale);
  } else {
    store_f16(b + 108, 0.0f);
  }
  int8_t l[QK_K];
  memset(l, 0, sizeof(l));
  const float bd = load_f16(b + 108);
  for (int j = 0; j < 16; j++) {
    uint8_t sc = j < 8 ? (uint8_t)(bscales[j] & 0xF) : (uint8_t)(bscales[j - 8] >> 4);
    const int8_t scs = (int8_t)((int8_t)(sc | (((bscales[8 + j % 4] >> (2 * (j / 4))) & 3) << 4)) - 32);
    const float d = bd * (float)scs;
    if (d != 0.0f)
      for (int ii = 0; ii < 16; ii++) l[16 * j + ii] = (int8_t)(clampi(nearest_int(x[16 * j + ii] / d), -4, 3) + 4);
  }
  memset(hmask, 0, 32);
  int m = 0;
  uint8_t hm = 1;
  for (int i = 0; i < QK_K; i++) {
    if (l[i] > 3) {
      hmask[m] |= hm;
      l[i] = (int8_t)(l[i] - 4);
    }
    if (++m == QK_K / 8) {
      m = 0;
      hm = (uint8_t)(hm << 1);
    }
  }
  for (int j = 0; j < QK_K; j += 128)
    for (int lv = 0; lv < 32; lv++)
      qs[j / 4 + lv] = (uint8_t)(l[j + lv] | (l[j + lv + 32] << 2) | (l[j + lv + 64] << 4) | (l[j + lv + 96] << 6));
}

/* BlockQ4K::from_float (k_quants.rs:1252-1310) and BlockQ5K::from_float (:1450-1526) */
static void kq_quant_q4k_q5k(const float* x, uint8_t* b, int five) {
  uint8_t* bscales = b + 4;
  float mins[8], scales[8];
  for (int j = 0; j < 8; j++) make_qkx1_quants(five ? 31 : 15, 5, x + 32 * j, 32, &scales[j], &mins[j]);
  const float max_scale = fold_max0(scales, 8), max_min = fold_max0(mins, 8);
  pack_scales_k4(scales, mins, max_scale, max_min, bscales);
  store_f16(b, max_scale / 63.0f);
  store_f16(b + 2, max_min / 63.0f);
  uint8_t l[QK_K];
  memset(l, 0, sizeof(l));
  const float bd = load_f16(b), bdmin = load_f16(b + 2);
  for (int j = 0; j < 8; j++) {
    uint8_t sc, m;
    get_scale_min_k4(j, bscales, &sc, &m);
    const float d = bd * (float)sc;
    if (d == 0.0f) continue;
    const float dm = bdmin * (float)m;
    for (int ii = 0; ii < 32; ii++) {
      const float v = x[32 * j + ii] + dm;
      l[32 * j + ii] = (uint8_t)clampi(nearest_int(v / d), 0, five ? 31 : 15);
    }
  }
  if (!five) {
    uint8_t* q = b + 16;
    for (int j = 0; j < QK_K; j += 64)
      for (int lv = 0; lv < 32; lv++) q[(j / 64) * 32 + lv] = (uint8_t)(l[j + lv] | (l[j + lv + 32] << 4));
    return;
  }
  uint8_t *qh = b + 16, *ql = b + 48;
  memset(qh, 0, 32);
  uint8_t m1 = 1, m2 = 2;
  for (int n = 0; n < QK_K; n += 64) {
    const int offset = (n / 64) * 32;
    for (int j = 0; j < 32; j++) {
      uint8_t l1 = l[n + j], l2 = l[n + j + 32];
      if (l1 > 15) {
        l1 = (uint8_t)(l1 - 16);
        qh[j] |= m1;
      }
      if (l2 > 15) {
        l2 = (uint8_t)(l2 - 16);
        qh[j] |= m2;
      }
      ql[offset + j] = (uint8_t)(l1 | (l2 << 4));
    }
    m1 = (uint8_t)(m1 << 2);
    m2 = (uint8_t)(m2 << 2);
  }
}

/* BlockQ6K::from_float, k_quants.rs:1643-1714 */
static void kq_quant_q6k(const float* x, uint8_t* b) {
  uint8_t *ql = b, *qh = b + 128;
  int8_t* bscales = (int8_t*)(b + 192);
  int8_t l[QK_K];
  float scales[16];
  memset(l, 0, sizeof(l));
  float max_scale = 0.0f, max_abs_scale = 0.0f;
  for (int ib = 0; ib < 16; ib++) {
    const float scale = make_qx_quants(16, 32, x + 16 * ib, l + 16 * ib, 1);
    scales[ib] = scale;
    if (fabsf(scale) > max_abs_scale) {
      max_abs_scale = fabsf(scale);
      max_scale = scale;
    }
  }
  const float iscale = -128.0f / max_scale;
  store_f16(b + 208, 1.0f / iscale);
  for (int j = 0; j < 16; j++) {
    const int32_t v = nearest_int(iscale * scales[j]);
    const int32_t c = v < 127 ? v : 127;
    bscales[j] = (int8_t)(c < -128 ? -128 : c); /* `as i8` saturates */
  }
  const float bd = load_f16(b + 208);
  for (int j = 0; j < 16; j++) {
    const float d = bd * (float)bscales[j];
    if (d == 0.0f) continue;
    for (int ii = 0; ii < 16; ii++) l[16 * j + ii] = (int8_t)(clampi(nearest_int(x[16 * j + ii] / d), -32, 31) + 32);
  }
  for (int j = 0; j < QK_K; j += 128) {
    for (int li = 0; li < 32; li++) {
      const int8_t q1 = l[j + li] & 0xF, q2 = l[j + li + 32] & 0xF, q3 = l[j + li + 64] & 0xF, q4 = l[j + li + 96] & 0xF;
      ql[li] = (uint8_t)(q1 | (q3 << 4));
      ql[li + 32] = (uint8_t)(q2 | (q4 << 4));
      qh[li] = (uint8_t)((l[j + li] >> 4) | ((l[j + li + 32] >> 4) << 2) | ((l[j + li + 64] >> 4) << 4) |
                         ((l[j + li + 96] >> 4) << 6));
    }
    ql += 64;
    qh += 32;
  }
}

/* BlockQ8K::from_float, k_quants.rs:1788-1825 */
static void kq_quant_q8k(const float* x, uint8_t* b) {
  int8_t* qs = (int8_t*)(b + 4);
  float max = 0.0f, amax = 0.0f;
  for (int j = 0; j < QK_K; j++)
    if (amax < fabsf(x[j])) {
      amax = fabsf(x[j]);
      max = x[j];
    }
  if (amax == 0.0f) {
    memset(b, 0, Q8K_BYTES); /* d = 0, qs = 0 (bsums keep the zero they were created with) */
    return;
  }
  const float iscale = -128.0f / max;
  for (int j = 0; j < QK_K; j++) {
    const float v = fminf(roundf(iscale * x[j]), 127.0f);
    qs[j] = v != v ? 0 : (v <= -128.0f ? -128 : (int8_t)v);
  }
  for (int j = 0; j < QK_K / 16; j++) {
    int32_t sum = 0;
    for (int ii = 0; ii < 16; ii++) sum += qs[j * 16 + ii];
    const int16_t s16 = (int16_t)sum;
    memcpy(b + 4 + QK_K + 2 * j, &s16, 2);
  }
  const float d = 1.0f / iscale;
  memcpy(b, &d, 4);
}

static int kq_quantize(int qtype, const float* x, uint8_t* blocks, int64_t k) {
  const int64_t bb = kq_block_bytes(qtype);
  if (bb < 0) return ORACLE_E_DTYPE;
  if (k % QK_K != 0) return ORACLE_E_SHAPE;
  for (int64_t i = 0; i < k / QK_K; i++) {
    const float* xs = x + i * QK_K;
    uint8_t* b = blocks + i * bb;
    switch (qtype) {
      case ORACLE_Q2K: kq_quant_q2k(xs, b); break;
      case ORACLE_Q3K: kq_quant_q3k(xs, b); break;
      case ORACLE_Q4K: kq_quant_q4k_q5k(xs, b, 0); break;
      case ORACLE_Q5K: kq_quant_q4k_q5k(xs, b, 1); break;
      case ORACLE_Q6K: kq_quant_q6k(xs, b); break;
      default: kq_quant_q8k(xs, b); break;
    }
  }
  return ORACLE_OK;
}
