/* Dense trellis linear layers for B200 (sm_100a): the reference's C ABI, re-implemented.
 *
 * Every declaration below replaces the one of the same name in the reference's
 * kernel/include/ignis_trellis_linear.h:81-145 (struct layouts pinned by its Rust mirror,
 * crates/core/src/trellis.rs:53-82, :229-234): same names, argument order, units and error
 * behaviour, so the callers (kernel/src/trellis_body.cu and the Rust bindings) link unchanged.
 *
 * A trellis weight is one EXL3 tensor (`trellis-tile16-v1`, docs/formats/flash-next-layout.md:73-146):
 * the inner matrix `inner` [in][out] as 16 x 16 tiles, tile (tk, tn) the 16 K int16 words at word
 * (tk * tile_stride + tn) * 16 K of `trellis`, K = k2 / 2 bits per weight, and
 *     W = diag(suh) H inner H diag(svh)              (in x out)
 * with H the block-diagonal 128-wide Sylvester Hadamard / sqrt(128), suh [in] and svh [out] fp16.
 * A call computes y[t] = x[t] W for each token.
 *
 * How this implementation differs inside (results stay within the reference's stated tolerance,
 * |y - Y| <= 2^-8 |Y| + 2^-9 s against the fp64 product, ignis_trellis_linear.h:32-44):
 * - one kernel per call: the input rotation is fused into the multiply's prologue, the split of
 *   the inputs is reduced through a thread-block cluster's distributed shared memory, so the
 *   workspace holds nothing (the query still returns a small non-zero size and init still zeroes
 *   it, for callers that reserve and initialise it);
 * - fp16 operands with fp32 accumulation (the reference accumulates in fp16 and folds every 32
 *   inputs); a power-of-two scale per token and 128-input block keeps the rotated activations in
 *   fp16 range whatever the input;
 * - up to 64 tokens a call shares every decoded tile among token tiles of 8; beyond 64 tokens, given
 *   the workspace ignis_trellis_workspace_bytes asks for, a call takes the tensor-core route: the
 *   activations rotated once into the workspace (fp16 rows, one power-of-two scale per token), the
 *   trellis tiles decoded into shared memory and multiplied by tcgen05 with fp32 accumulation in
 *   tensor memory; SwiGLU stores the gate in BF16 between its two products there, as the
 *   reference's prefill route does (ignis_trellis_linear.h:43-44). Without that workspace a wide
 *   call runs as passes of 64 tokens.
 *
 * Conventions (unchanged): activations device-resident token-major BF16 x [tokens][in], 16-byte
 * aligned; outputs BF16 [tokens][ldy], ldy a multiple of 4, y 8-byte aligned; `in` and `out`
 * positive multiples of 128, `out` at most IGNIS_TRELLIS_MAX_OUT; trellis 16-byte aligned, suh and
 * svh 8-byte aligned. Calls enqueue on `stream`, allocate nothing, never synchronize the host.
 * Results are deterministic run to run. Return 0 on success, -1 otherwise with the reason in
 * ignis_trellis_last_error().
 */
#ifndef IGNIS_TRELLIS_LINEAR_H
#define IGNIS_TRELLIS_LINEAR_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IGNIS_TRELLIS_DECODE_MAX_TOKENS 64 /* reference: ignis_trellis_linear.h:83 */
#define IGNIS_TRELLIS_MAX_OUT 524288       /* reference: ignis_trellis_linear.h:89 */

/* reference: ignis_trellis_linear.h:91-102 (40 bytes) */
typedef struct ignis_trellis_weight {
  const void *trellis; /* int16 tiles */
  const void *suh;     /* fp16 [in] */
  const void *svh;     /* fp16 [out] */
  uint32_t k2;         /* 2 K: 4, 5, 6, 8, 10 or 12 */
  uint32_t in;
  uint32_t out;
  uint32_t tile_stride; /* tiles per stored row; 0 for out / 16. A column view [c, c + out) of a
                           wider plane passes trellis advanced by c / 16 tiles, svh by c, and the
                           plane's out / 16 here (c a multiple of 128). */
} ignis_trellis_weight;

/* reference: ignis_trellis_linear.h:104-107 (16 bytes) */
typedef struct ignis_trellis_workspace {
  void *base;     /* device, 256-byte aligned */
  uint64_t bytes; /* at least what ignis_trellis_workspace_bytes asked for */
} ignis_trellis_workspace;

/* Prepares the current device (kernel attributes, SM count, IGNIS_TRELLIS_SM_CAP). Once per
 * device at load, outside any stream capture. reference: ignis_trellis_linear.h:112 */
int32_t ignis_trellis_prepare(void);

/* The SM cap the device was prepared with, 0 for none. reference: ignis_trellis_linear.h:115 */
uint32_t ignis_trellis_sm_cap(void);

/* Workspace bytes of a call; 0 for a shape the ops refuse or an unprepared device.
 * reference: ignis_trellis_linear.h:121 */
uint64_t ignis_trellis_workspace_bytes(uint32_t in, uint32_t out, uint32_t weights, uint32_t tokens);

/* Zeroes the workspace once after it is reserved. reference: ignis_trellis_linear.h:124 */
int32_t ignis_trellis_workspace_init(const ignis_trellis_workspace *workspace, void *stream);

#define IGNIS_TRELLIS_STORE 0 /* y[t][c] = BF16(v) */
#define IGNIS_TRELLIS_ADD 1   /* y[t][c] = BF16(y[t][c] + v), one rounding */

/* y = x W through `epilogue`. reference: ignis_trellis_linear.h:131-133 */
int32_t ignis_trellis_linear(const ignis_trellis_weight *w, const void *x, uint32_t tokens, void *y,
                             uint32_t ldy, uint32_t epilogue, const ignis_trellis_workspace *workspace,
                             void *stream);

/* h[t][c] = BF16(silu(x[t] G)[c] * (x[t] U)[c]), one rounding from fp32.
 * reference: ignis_trellis_linear.h:137-140 */
int32_t ignis_trellis_linear_swiglu(const ignis_trellis_weight *gate, const ignis_trellis_weight *up,
                                    const void *x, uint32_t tokens, void *h, uint32_t ldh,
                                    const ignis_trellis_workspace *workspace, void *stream);

/* Not in the reference's ABI: up to 4 weights of the same `in` applied to the same x in one launch,
 * weight i writing y[i][t][..ldy[i]] (q | k | v and the like: a narrow weight alone cannot fill
 * the device, and every launch has a fixed cost). Same arithmetic and bits as `count` separate
 * ignis_trellis_linear calls; STORE or ADD. Needs no workspace. */
int32_t b200q_trellis_linear_group(const ignis_trellis_weight *const *w, uint32_t count, const void *x,
                                   uint32_t tokens, void *const *y, const uint32_t *ldy, uint32_t epilogue,
                                   void *stream);

/* `inner` decoded to fp16 [in][out] row-major, bit for bit exllamav3's `reconstruct`.
 * reference: ignis_trellis_linear.h:145 */
int32_t ignis_trellis_reconstruct(const ignis_trellis_weight *w, void *w_f16, void *stream);

/* Not in the reference's ABI (its kernels trap or spin instead): the status word of the tensor-core
 * route's bounded device-side waits, copied to *status after `stream` has finished. 0 unless a wait
 * ran out (bit 0 producer, 1 MMA issuer, 2 epilogue, 3 decoder), in which case that call's output
 * is not valid. Per device, sticky. */
int32_t b200q_trellis_device_status(void *stream, uint32_t *status);

/* Thread-local message of the most recent failed call. Never NULL.
 * reference: ignis_trellis_linear.h:148 */
const char *ignis_trellis_last_error(void);

#ifdef __cplusplus
}
#endif

#endif /* IGNIS_TRELLIS_LINEAR_H */
