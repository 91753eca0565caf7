/* CPU oracle for the quantized linear-layer path: TEST INFRASTRUCTURE ONLY (see b200q_oracle.h).
 * Compile with -O2 -ffp-contract=off -pthread: the activation quantizer depends on every
 * float32 operation being rounded once, so fused multiply-adds must not be formed. */
#include "b200q_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ---- scalar formats ------------------------------------------------------------------------ */

static const double kE2m1[8] = {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0};

double orc_e2m1_decode(uint8_t nibble) {
  const double m = kE2m1[nibble & 7u];
  return (nibble & 8u) ? -m : m;
}

double orc_e4m3_decode(uint8_t byte) {
  const int e = (byte >> 3) & 15;
  const int m = byte & 7;
  double v;
  if (e == 0) {
    v = ldexp((double)m, -9);
  } else if (e == 15 && m == 7) {
    v = NAN;
  } else {
    v = ldexp(1.0 + (double)m / 8.0, e - 7);
  }
  return (byte & 0x80u) ? -v : v;
}

/* Round-to-nearest-even onto the E4M3FN grid, saturating at 448; NaN gives the positive NaN
 * word 0x7F. The grid below 2^-6 is the subnormal one with spacing 2^-9. */
uint8_t orc_e4m3_encode_satfinite(float v) {
  if (isnan(v)) return 0x7F;
  const uint8_t sign = signbit(v) ? 0x80u : 0u;
  double a = fabs((double)v);
  if (a >= 448.0) return sign | 0x7Eu; /* includes infinities */
  int e;
  double q; /* spacing of the grid around a */
  if (a < ldexp(1.0, -6)) {
    q = ldexp(1.0, -9);
  } else {
    (void)frexp(a, &e);          /* a = f * 2^e, f in [0.5, 1) -> exponent of a is e - 1 */
    q = ldexp(1.0, (e - 1) - 3); /* three mantissa bits */
  }
  const double steps = nearbyint(a / q); /* default rounding mode: ties to even; a / q is exact */
  const double r = steps * q;
  if (r >= 448.0 + 1e-9) return sign | 0x7Eu;
  if (r == 0.0) return sign;
  /* re-encode r (it may have carried into the next binade) */
  if (r < ldexp(1.0, -6)) return sign | (uint8_t)(r / ldexp(1.0, -9));
  double f = frexp(r, &e); /* r = f 2^e, f in [0.5,1) */
  const int exp_field = (e - 1) + 7;
  const int man = (int)((f * 2.0 - 1.0) * 8.0);
  return sign | (uint8_t)((exp_field << 3) | man);
}

/* Saturating round-to-nearest-even onto {0,.5,1,1.5,2,3,4,6}: boundaries 0.25 down, 0.75 up,
 * 1.25 down, 1.75 up, 2.5 down, 3.5 up, 5.0 down (tools/27b-nvfp4-converter/encode.py:29-30).
 * NaN maps to the positive maximum, as the hardware conversion does. */
uint8_t orc_e2m1_encode_satfinite(float v) {
  static const float bound[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
  static const int tie_up[7] = {0, 1, 0, 1, 0, 1, 0};
  if (isnan(v)) return 0x7;
  const uint8_t sign = signbit(v) ? 8u : 0u;
  const float a = fabsf(v);
  uint8_t code = 0;
  for (int i = 0; i < 7; ++i) {
    if (a > bound[i] || (a == bound[i] && tie_up[i])) ++code;
  }
  return sign | code;
}

float orc_bf16_to_f32(uint16_t h) {
  const uint32_t b = (uint32_t)h << 16;
  float v;
  memcpy(&v, &b, 4);
  return v;
}

uint16_t orc_f32_to_bf16(float v) {
  uint32_t b;
  memcpy(&b, &v, 4);
  if ((b & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((b >> 16) | 0x40u); /* quiet NaN */
  b += 0x7FFFu + ((b >> 16) & 1u);
  return (uint16_t)(b >> 16);
}

float orc_f16_to_f32(uint16_t h) {
  const int s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023;
  float v;
  if (e == 0) {
    v = ldexpf((float)m, -24);
  } else if (e == 31) {
    v = m ? NAN : INFINITY;
  } else {
    v = ldexpf(1.0f + (float)m / 1024.0f, e - 15);
  }
  return s ? -v : v;
}

uint16_t orc_f32_to_f16(float v) {
  if (isnan(v)) return 0x7E00;
  const uint16_t sign = signbit(v) ? 0x8000u : 0u;
  const double a = fabs((double)v);
  if (a >= 65520.0) return sign | 0x7C00u; /* rounds to infinity */
  if (a < ldexp(1.0, -14)) {               /* subnormal grid 2^-24 */
    return sign | (uint16_t)nearbyint(a / ldexp(1.0, -24));
  }
  int e;
  (void)frexp(a, &e);
  const double q = ldexp(1.0, (e - 1) - 10);
  const double r = nearbyint(a / q) * q;
  int e2;
  const double f = frexp(r, &e2);
  const int exp_field = (e2 - 1) + 15;
  const int man = (int)((f * 2.0 - 1.0) * 1024.0);
  return sign | (uint16_t)((exp_field << 10) | man);
}

/* ---- tiny thread pool helper ------------------------------------------------------------- */

typedef void (*range_fn)(void *ctx, int64_t begin, int64_t end);
typedef struct {
  range_fn fn;
  void *ctx;
  int64_t begin, end;
} range_job;

static void *range_thread(void *p) {
  range_job *j = (range_job *)p;
  j->fn(j->ctx, j->begin, j->end);
  return NULL;
}

/* Splits [0, n) over `threads` workers exactly as the reference's oracle splits its rows:
 * worker i takes [n i / T, n (i + 1) / T). */
static void parallel_ranges(int64_t n, int32_t threads, range_fn fn, void *ctx) {
  if (threads < 1) threads = 1;
  if (threads > n) threads = (int32_t)(n > 0 ? n : 1);
  if (threads == 1) {
    fn(ctx, 0, n);
    return;
  }
  pthread_t *tid = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
  range_job *jobs = (range_job *)malloc(sizeof(range_job) * (size_t)threads);
  for (int32_t i = 0; i < threads; ++i) {
    jobs[i].fn = fn;
    jobs[i].ctx = ctx;
    jobs[i].begin = n * i / threads;
    jobs[i].end = n * (i + 1) / threads;
    pthread_create(&tid[i], NULL, range_thread, &jobs[i]);
  }
  for (int32_t i = 0; i < threads; ++i) pthread_join(tid[i], NULL);
  free(jobs);
  free(tid);
}

/* ---- NVFP4 ------------------------------------------------------------------------------- */

int64_t orc_nvfp4_scale_offset(int32_t row, int32_t group, int32_t k) {
  const int32_t m_tile = row / 128, inner = row % 128;
  return ((int64_t)m_tile * (k / 64) + group / 4) * 512 + (inner % 32) * 16 + (inner / 32) * 4 + group % 4;
}

void orc_nvfp4_patterned(int32_t n, int32_t k, uint32_t seed, uint8_t *codes, uint8_t *scales) {
  static const uint8_t words[8] = {0x00, 0x04, 0x08, 0x0b, 0x10, 0x13, 0x18, 0x1d};
  for (int32_t r = 0; r < n; ++r) {
    for (int32_t c = 0; c < k; c += 2) {
      const uint8_t lo = (uint8_t)(((uint32_t)r * 13u + (uint32_t)c * 7u + seed) & 15u);
      const uint8_t hi = (uint8_t)(((uint32_t)r * 13u + (uint32_t)(c + 1) * 7u + seed) & 15u);
      codes[(size_t)r * k / 2 + c / 2] = (uint8_t)(lo | (hi << 4));
    }
    for (int32_t g = 0; g < k / 16; ++g) {
      scales[orc_nvfp4_scale_offset(r, g, k)] = words[((uint32_t)r * 5u + (uint32_t)g * 3u + seed) & 7u];
    }
  }
}

void orc_nvfp4_dequant(const uint8_t *codes, const uint8_t *scales, int32_t n, int32_t k, float d_w,
                       int32_t row0, int32_t row1, float *out) {
  (void)n;
  for (int32_t r = row0; r < row1; ++r) {
    float *dst = out + (size_t)(r - row0) * k;
    for (int32_t c = 0; c < k; ++c) {
      const uint8_t packed = codes[(size_t)r * k / 2 + c / 2];
      const uint8_t code = (c & 1) ? (uint8_t)(packed >> 4) : (uint8_t)(packed & 15u);
      const double s = orc_e4m3_decode(scales[orc_nvfp4_scale_offset(r, c / 16, k)]);
      dst[c] = (float)(orc_e2m1_decode(code) * s / (double)d_w);
    }
  }
}

typedef struct {
  const float *w, *x;
  double *out;
  int32_t n, k, t;
} gemm_ctx;

static void gemm_rows(void *p, int64_t begin, int64_t end) {
  const gemm_ctx *c = (const gemm_ctx *)p;
  for (int64_t row = begin; row < end; ++row) {
    const float *wr = c->w + (size_t)row * c->k;
    for (int32_t t0 = 0; t0 < c->t; t0 += 8) {
      const int32_t active = c->t - t0 < 8 ? c->t - t0 : 8;
      double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int32_t col = 0; col < c->k; ++col) {
        const double wv = (double)wr[col];
        for (int32_t j = 0; j < active; ++j) acc[j] += wv * (double)c->x[(size_t)(t0 + j) * c->k + col];
      }
      for (int32_t j = 0; j < active; ++j) c->out[(size_t)(t0 + j) * c->n + row] = acc[j];
    }
  }
}

void orc_gemm_f64(const float *w, const float *x, double *out, int32_t n, int32_t k, int32_t t,
                  int32_t threads) {
  gemm_ctx c = {w, x, out, n, k, t};
  parallel_ranges(n, threads, gemm_rows, &c);
}

void orc_nvfp4_quantize_act(const uint16_t *x_bf16, int32_t t, int32_t k, float d_in, uint8_t *codes,
                            uint8_t *scales) {
  for (int32_t tok = 0; tok < t; ++tok) {
    for (int32_t g = 0; g < k / 16; ++g) {
      float v[16];
      float amax = 0.0f;
      for (int i = 0; i < 16; ++i) {
        v[i] = orc_bf16_to_f32(x_bf16[(size_t)tok * k + g * 16 + i]);
        amax = fmaxf(amax, fabsf(v[i]));
      }
      volatile float scaled = d_in * amax; /* one rounding */
      volatile float unencoded = scaled / 6.0f;
      const uint8_t s = orc_e4m3_encode_satfinite(unencoded);
      scales[(size_t)tok * (k / 16) + g] = s;
      uint8_t *dst = codes + (size_t)tok * (k / 2) + g * 8;
      if (s == 0) {
        memset(dst, 0, 8);
        continue;
      }
      const float dec = (float)orc_e4m3_decode(s);
      for (int i = 0; i < 16; i += 2) {
        volatile float a0 = v[i] * d_in, a1 = v[i + 1] * d_in;
        volatile float q0 = a0 / dec, q1 = a1 / dec;
        dst[i / 2] = (uint8_t)(orc_e2m1_encode_satfinite(q0) | (orc_e2m1_encode_satfinite(q1) << 4));
      }
    }
  }
}

typedef struct {
  const uint8_t *wc, *ws, *ac, *as;
  int32_t n, k, t;
  double alpha;
  double *out;
} w4a4_ctx;

static void w4a4_rows(void *p, int64_t begin, int64_t end) {
  const w4a4_ctx *c = (const w4a4_ctx *)p;
  const int32_t groups = c->k / 16;
  for (int64_t row = begin; row < end; ++row) {
    for (int32_t tok = 0; tok < c->t; ++tok) {
      double acc = 0.0;
      for (int32_t g = 0; g < groups; ++g) {
        const double sw = orc_e4m3_decode(c->ws[orc_nvfp4_scale_offset((int32_t)row, g, c->k)]);
        const double sa = orc_e4m3_decode(c->as[(size_t)tok * groups + g]);
        const uint8_t *wb = c->wc + (size_t)row * c->k / 2 + g * 8;
        const uint8_t *ab = c->ac + (size_t)tok * c->k / 2 + g * 8;
        double dot = 0.0; /* exact: sums of products of quarter-integers */
        for (int i = 0; i < 8; ++i) {
          dot += orc_e2m1_decode(wb[i] & 15u) * orc_e2m1_decode(ab[i] & 15u);
          dot += orc_e2m1_decode(wb[i] >> 4) * orc_e2m1_decode(ab[i] >> 4);
        }
        acc += sw * sa * dot;
      }
      c->out[(size_t)tok * c->n + row] = c->alpha * acc;
    }
  }
}

void orc_nvfp4_w4a4_gemm(const uint8_t *w_codes, const uint8_t *w_scales, int32_t n, int32_t k, float d_w,
                         const uint8_t *a_codes, const uint8_t *a_scales, int32_t t, float d_in,
                         double *out, int32_t threads) {
  /* alpha is formed in float32 as the reference does (1.0f / (d_in * d_w)) */
  volatile float prod = d_in * d_w;
  volatile float alpha = 1.0f / prod;
  w4a4_ctx c = {w_codes, w_scales, a_codes, a_scales, n, k, t, (double)alpha, out};
  parallel_ranges(n, threads, w4a4_rows, &c);
}

/* ---- trellis ----------------------------------------------------------------------------- */

uint32_t orc_lowbias32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}

uint32_t orc_hash_u32(uint32_t stream, uint64_t i) {
  return orc_lowbias32((uint32_t)i * 0x9E3779B9u + stream * 0x85EBCA6Bu);
}

float orc_hash_uniform(uint32_t stream, uint64_t i, float amplitude) {
  volatile float u = (float)(orc_hash_u32(stream, i) >> 8) * 0x1p-23f - 1.0f;
  return u * amplitude;
}

void orc_hash_trellis_words(uint32_t stream, int32_t in, int32_t out, uint32_t k2, uint16_t *words) {
  const size_t n = (size_t)(in / 16) * (size_t)(out / 16) * 8u * k2;
  for (size_t i = 0; i < n; ++i) words[i] = (uint16_t)(orc_hash_u32(stream, i) & 0xFFFFu);
}

uint16_t orc_mul1_f16_bits(uint32_t state) {
  const uint32_t prod = state * 0x83DCD12Du;
  const uint32_t bsum = (prod & 255u) + ((prod >> 8) & 255u) + ((prod >> 16) & 255u) + (prod >> 24);
  const float k_inv = orc_f16_to_f32(0x1EEE);
  const float k_bias = orc_f16_to_f32(0xC931);
  /* (1024 + bsum) * k_inv is exact in float32 (11 x 11 significant bits); the sum with k_bias is
   * computed in double so the only rounding is the conversion to fp16. */
  const double exact = (double)(1024.0f + (float)bsum) * (double)k_inv + (double)k_bias;
  return orc_f32_to_f16((float)exact);
}

static int step_bits(uint32_t k2, int p) { return k2 == 5 ? ((p & 1) ? 3 : 2) : (int)(k2 / 2); }

typedef struct {
  const uint16_t *words;
  uint32_t k2;
  int32_t in, out, tile_stride;
  uint16_t *inner;
  const uint16_t *lut; /* state -> fp16 bits */
} decode_ctx;

static void decode_tile_rows(void *p, int64_t begin, int64_t end) {
  const decode_ctx *c = (const decode_ctx *)p;
  const int tn = c->out / 16;
  const int w16 = 8 * (int)c->k2;
  const int bits = w16 * 16;
  int perm[256], endb[256];
  for (int t = 0; t < 32; ++t) {
    const int r0 = (t % 4) * 2, c0 = t / 4;
    const int rows[4] = {r0, r0 + 1, r0 + 8, r0 + 9};
    for (int j = 0; j < 8; ++j) perm[t * 8 + j] = rows[j % 4] * 16 + c0 + (j >= 4 ? 8 : 0);
  }
  for (int q = 0, e = 0; q < 256; ++q) {
    e += step_bits(c->k2, q);
    endb[q] = e;
  }
  uint8_t *stream = (uint8_t *)malloc((size_t)bits);
  for (int64_t tk = begin; tk < end; ++tk) {
    for (int tc = 0; tc < tn; ++tc) {
      const uint16_t *tile = c->words + ((size_t)tk * c->tile_stride + tc) * w16;
      for (int b = 0; b < bits; ++b) {
        const uint32_t u32 = tile[2 * (b / 32)] | ((uint32_t)tile[2 * (b / 32) + 1] << 16);
        stream[b] = (uint8_t)((u32 >> (31 - (b % 32))) & 1u);
      }
      for (int q = 0; q < 256; ++q) {
        uint32_t state = 0;
        for (int j = 0; j < 16; ++j) {
          int b = endb[q] - 16 + j;
          b = ((b % bits) + bits) % bits;
          state = (state << 1) | stream[b];
        }
        const int r = perm[q] / 16, col = perm[q] % 16;
        c->inner[(size_t)(tk * 16 + r) * c->out + tc * 16 + col] = c->lut[state];
      }
    }
  }
  free(stream);
}

void orc_trellis_decode(const uint16_t *words, uint32_t k2, int32_t in, int32_t out, int32_t tile_stride,
                        uint16_t *inner, int32_t threads) {
  uint16_t *lut = (uint16_t *)malloc(65536 * sizeof(uint16_t));
  for (uint32_t s = 0; s < 65536; ++s) lut[s] = orc_mul1_f16_bits(s);
  decode_ctx c = {words, k2, in, out, tile_stride ? tile_stride : out / 16, inner, lut};
  parallel_ranges(in / 16, threads, decode_tile_rows, &c);
  free(lut);
}

uint64_t orc_checksum_u16(const uint16_t *v, uint64_t n) {
  uint64_t s = 0;
  for (uint64_t i = 0; i < n; ++i) s += (uint64_t)v[i] * (uint64_t)(orc_lowbias32((uint32_t)i) | 1u);
  return s;
}

void orc_hadamard128(double *v, int64_t n) {
  const double norm = sqrt(128.0);
  for (int64_t b = 0; b < n; b += 128) {
    for (int h = 1; h < 128; h <<= 1) {
      for (int i = 0; i < 128; i += 2 * h) {
        for (int j = i; j < i + h; ++j) {
          const double a = v[b + j], c = v[b + j + h];
          v[b + j] = a + c;
          v[b + j + h] = a - c;
        }
      }
    }
    for (int i = 0; i < 128; ++i) v[b + i] /= norm;
  }
}

static double f16_lut_value(uint16_t h) { return (double)orc_f16_to_f32(h); }

void orc_trellis_project(const uint16_t *inner, const uint16_t *suh, const uint16_t *svh, int32_t in,
                         int32_t out, const double *x, double *y) {
  double *xs = (double *)malloc(sizeof(double) * (size_t)in);
  for (int32_t k = 0; k < in; ++k) xs[k] = x[k] * f16_lut_value(suh[k]);
  orc_hadamard128(xs, in);
  for (int32_t n = 0; n < out; ++n) y[n] = 0.0;
  for (int32_t k = 0; k < in; ++k) {
    const uint16_t *row = inner + (size_t)k * out;
    const double a = xs[k];
    for (int32_t n = 0; n < out; ++n) y[n] += a * f16_lut_value(row[n]);
  }
  orc_hadamard128(y, out);
  for (int32_t n = 0; n < out; ++n) y[n] *= f16_lut_value(svh[n]);
  free(xs);
}

typedef struct {
  const uint16_t *inner, *suh, *svh;
  int32_t in, out;
  const double *x;
  double *y;
} project_ctx;

static void project_tokens(void *p, int64_t begin, int64_t end) {
  const project_ctx *c = (const project_ctx *)p;
  for (int64_t t = begin; t < end; ++t) {
    orc_trellis_project(c->inner, c->suh, c->svh, c->in, c->out, c->x + (size_t)t * c->in,
                        c->y + (size_t)t * c->out);
  }
}

void orc_trellis_project_tokens(const uint16_t *inner, const uint16_t *suh, const uint16_t *svh, int32_t in,
                                int32_t out, const double *x, int32_t t, double *y, int32_t threads) {
  project_ctx c = {inner, suh, svh, in, out, x, y};
  parallel_ranges(t, threads, project_tokens, &c);
}

/* ---- routed experts ---------------------------------------------------------------------- */

void orc_moe_expert(const uint16_t *gu_inner, const uint16_t *gu_suh, const uint16_t *gu_svh,
                    const uint16_t *dn_inner, const uint16_t *dn_suh, const uint16_t *dn_svh, int32_t hidden,
                    int32_t inter, const double *x, double *y) {
  double *gu = (double *)malloc(sizeof(double) * (size_t)inter * 2);
  double *h = (double *)malloc(sizeof(double) * (size_t)inter);
  orc_trellis_project(gu_inner, gu_suh, gu_svh, hidden, 2 * inter, x, gu);
  for (int32_t j = 0; j < inter; ++j) h[j] = gu[j] / (1.0 + exp(-gu[j])) * gu[inter + j];
  orc_trellis_project(dn_inner, dn_suh, dn_svh, inter, hidden, h, y);
  free(h);
  free(gu);
}
