/* CPU oracle for the quantized linear-layer path: TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference's own host-side dequantizers and fp64 products.
 * Nothing the library ships links, loads or calls it: only the tests, the smoke check and the
 * CPU-baseline / reference legs of the benchmark do, and only as the checker or as the thing
 * timed on the host cores. Each function names the reference code it follows (paths are relative
 * to the reference project's root).
 *
 * Parity is pinned: the trellis decoder reproduces the recorded exllamav3 `reconstruct` tensors
 * and the real-shape checksums the reference's fixtures hold, and the NVFP4 dequantizer agrees
 * with the reference's own `logical_weight_fp64` compiled from its source (see tests/).
 */
#ifndef B200Q_ORACLE_H
#define B200Q_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar formats ---------------------------------------------------------------------- */
double orc_e2m1_decode(uint8_t nibble);          /* kernel/vendor/tests/ops/quantized_weight.h:122-126 */
double orc_e4m3_decode(uint8_t byte);            /* quantized_weight.h:128-143; NaN words give NaN */
uint8_t orc_e4m3_encode_satfinite(float v);      /* cvt.rn.satfinite.e4m3x2.f32 semantics */
uint8_t orc_e2m1_encode_satfinite(float v);      /* cvt.rn.satfinite.e2m1x2.f32; ties per encode.py:29-30 */
float orc_bf16_to_f32(uint16_t h);
uint16_t orc_f32_to_bf16(float v);               /* round to nearest even */
float orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float v);                /* round to nearest even */

/* ---- NVFP4 `blockscale-k16-m128x4-v1` ------------------------------------------------------ */
/* Byte offset of the scale of (row, group = k / 16) inside the swizzled scale plane.
 * kernel/vendor/src/ops/linear/nvfp4/nvfp4_codec.cuh:32-42 */
int64_t orc_nvfp4_scale_offset(int32_t row, int32_t group, int32_t k);

/* Patterned weight of the reference's linear tests: codes (13 row + 7 col + seed) & 15, scales
 * from eight fixed E4M3 words by (5 row + 3 group + seed) & 7. quantized_weight.h:413-456 */
void orc_nvfp4_patterned(int32_t n, int32_t k, uint32_t seed, uint8_t *codes, uint8_t *scales);

/* w[row][col] = float(E2M1(code) * E4M3(scale) / d_w), the logical weight. rows [row0, row1).
 * quantized_weight.h:642-690 (logical_weight_fp64, NVFP4 branch) */
void orc_nvfp4_dequant(const uint8_t *codes, const uint8_t *scales, int32_t n, int32_t k, float d_w,
                       int32_t row0, int32_t row1, float *out);

/* out[t][row] = sum_k w[row][k] * x[t][k] in fp64, rows split over `threads` workers, tokens in
 * blocks of 8. kernel/vendor/tests/ops/linear/linear_test_common.cpp:246-287 */
void orc_gemm_f64(const float *w, const float *x, double *out, int32_t n, int32_t k, int32_t t,
                  int32_t threads);

/* Activation block quantizer: per token and 16 values along K.
 * kernel/vendor/src/ops/linear/nvfp4/nvfp4_codec.cuh:81-110; token-major outputs
 * codes [t][k/2] (even k in the low nibble), scales [t][k/16]. */
void orc_nvfp4_quantize_act(const uint16_t *x_bf16, int32_t t, int32_t k, float d_in,
                            uint8_t *codes, uint8_t *scales);

/* W4A4 product: out[t][row] = (1 / (d_in d_w)) * sum over groups of
 * E4M3(sa) E4M3(sw) sum_16 E2M1(a) E2M1(w), fp64 accumulate.
 * kernel/vendor/src/ops/linear/nvfp4/nvfp4_w4a4.cu:37, nvfp4_w4a4_mma.cuh:342-358 */
void orc_nvfp4_w4a4_gemm(const uint8_t *w_codes, const uint8_t *w_scales, int32_t n, int32_t k,
                         float d_w, const uint8_t *a_codes, const uint8_t *a_scales, int32_t t,
                         float d_in, double *out, int32_t threads);

/* ---- trellis `trellis-tile16-v1` ----------------------------------------------------------- */
uint32_t orc_lowbias32(uint32_t x);                         /* kernel/tests/moe_fixture.h:129-136 */
uint32_t orc_hash_u32(uint32_t stream, uint64_t i);         /* moe_fixture.h:138-140 */
float orc_hash_uniform(uint32_t stream, uint64_t i, float amplitude); /* moe_fixture.h:143-146 */
void orc_hash_trellis_words(uint32_t stream, int32_t in, int32_t out, uint32_t k2, uint16_t *words);
                                                            /* moe_fixture.h:321-325 */
uint16_t orc_mul1_f16_bits(uint32_t state);                 /* moe_fixture.h:264-270 */
/* inner[in][out] fp16 bits from words [in/16][tile_stride][16K]; tile_stride 0 means out/16.
 * moe_fixture.h:274-309 (host_trellis_decode) */
void orc_trellis_decode(const uint16_t *words, uint32_t k2, int32_t in, int32_t out,
                        int32_t tile_stride, uint16_t *inner, int32_t threads);
uint64_t orc_checksum_u16(const uint16_t *v, uint64_t n);   /* moe_fixture.h:312-318 */
void orc_hadamard128(double *v, int64_t n);                 /* moe_fixture.h:331-345 */
/* y[out] = had(had(x o suh) . inner) o svh for one token. moe_fixture.h:348-361 */
void orc_trellis_project(const uint16_t *inner, const uint16_t *suh, const uint16_t *svh,
                         int32_t in, int32_t out, const double *x, double *y);
/* tokens in parallel over `threads` workers; x [t][in], y [t][out] */
void orc_trellis_project_tokens(const uint16_t *inner, const uint16_t *suh, const uint16_t *svh,
                                int32_t in, int32_t out, const double *x, int32_t t, double *y,
                                int32_t threads);

/* ---- routed experts ------------------------------------------------------------------------ */
/* One expert on one token: y[hidden] = down(silu(gate(x)) * up(x)); gate_up inner is
 * [hidden][2 inter] (gate columns first), down inner [inter][hidden].
 * kernel/tests/moe_experts_common.h:142-164 (project, expert_f64), geometry made a parameter. */
void orc_moe_expert(const uint16_t *gu_inner, const uint16_t *gu_suh, const uint16_t *gu_svh,
                    const uint16_t *dn_inner, const uint16_t *dn_suh, const uint16_t *dn_svh,
                    int32_t hidden, int32_t inter, const double *x, double *y);

#ifdef __cplusplus
}
#endif
#endif
