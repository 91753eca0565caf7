/* Flash-Next mixture-of-experts ops for B200 (sm_100a): the reference's C ABI, re-implemented.
 *
 * Every declaration below replaces the one of the same name in the reference's
 * kernel/include/ignis_moe.h:65-215 (Rust mirror crates/core/src/moe.rs:47-170, struct layouts
 * pinned by its tests :355-388): same names, argument order and meaning. One addition,
 * b200q_moe_set_geometry, lifts the reference's compile-time geometry (2560 / 640 / 512 experts /
 * top 10, "the ops refuse anything else", ignis_moe.h:41-45) to a process-wide setting whose
 * default is that geometry.
 *
 * The block, per token: a router picks top_k of `experts` experts from a BF16 router weight; each
 * selected expert is a SwiGLU MLP hidden -> inter -> hidden stored as two trellis records (fused
 * gate/up plane (hidden, 2 inter): columns [0, inter) gate, [inter, 2 inter) up; down plane
 * (inter, hidden); docs/formats/flash-next-layout.md section 3), each at its own k2 in {4, 5, 6,
 * 8}; a shared expert (FP8 row-scale, gated by a sigmoid of a BF16 hidden -> 1 projection) runs on
 * every token; the combine sums them.
 *
 * Conventions (unchanged): activations device-resident token-major BF16; every call enqueues on
 * `stream`, allocates nothing, never synchronizes the host; workspaces are sized by the queries
 * from the load's maxima and initialised once; results are deterministic - the routed output is
 * accumulated in exact 64-bit fixed point with 32 fractional bits, so no result depends on the
 * order in which contributions arrive; return 0, or -1 with the reason in ignis_moe_last_error().
 *
 * Where this implementation differs inside: a selected-but-absent record (NULL, or k2 outside
 * {4, 5, 6, 8}), an expert id outside the table, or a contribution that is not finite or too
 * large for the accumulator does not trap the kernel as the reference's does (ignis_moe.h:76-81,
 * :166-170): the contribution is skipped and a bit is set in the workspace's status word, which
 * ignis_moe_workspace_status reads back. Both routes (decode, prefill) run the same grouped
 * kernels: assignments are grouped by expert on the device, work items of at most 8 rows each
 * decode their expert's tiles once; `decode_route` is accepted and ignored.
 */
#ifndef IGNIS_MOE_H
#define IGNIS_MOE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The reference's geometry and the default here (ignis_moe.h:42-47). */
#define IGNIS_MOE_HIDDEN 2560
#define IGNIS_MOE_EXPERTS 512
#define IGNIS_MOE_TOP_K 10
#define IGNIS_MOE_INTERMEDIATE 640
#define IGNIS_MOE_DECODE_MAX_TOKENS 8

#define IGNIS_MOE_PROJ_GATE_UP 0 /* ignis_moe.h:51 */
#define IGNIS_MOE_PROJ_DOWN 1    /* ignis_moe.h:52 */

/* No counterpart in the reference, which compiles one geometry in (ignis_moe.h:42-47): the
 * geometry as an argument. Every b200q_moe_* entry below is the ignis_moe_* entry of the same name
 * with this struct in front - same arguments, same results - and carries no state between calls,
 * so two models (or two threads) use different geometries side by side. hidden and inter are
 * positive multiples of 128, experts 1..4096, top_k 1..min(32, experts). */
typedef struct b200q_moe_geometry {
  uint32_t hidden;
  uint32_t inter;
  uint32_t experts;
  uint32_t top_k;
} b200q_moe_geometry;

/* The geometry the reference's own entry points (ignis_moe_*, no geometry argument) work at: the
 * reference's at start. A convenience for callers bound to the verbatim ABI with another model;
 * process-wide, so set it once at load before any query. New code passes the struct instead. */
int32_t b200q_moe_set_geometry(uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t top_k);

/* Not in the reference: an expert id that means "this choice has no expert here". The expert ops
 * skip it without setting a status bit (every other id outside the table is skipped and reported),
 * so a rank of an expert-parallel group can run a token whose other choices live elsewhere. */
#define IGNIS_MOE_NO_EXPERT (-1)

/* One slot-table entry: ignis_moe.h:65-69 (16 bytes). A record is the trellis tensor, then suh
 * (fp16, `in`), then svh (fp16, `out`), each 16-byte aligned. The table of a layer is experts * 2
 * entries indexed expert * 2 + projection. */
struct ignis_moe_slot {
  const void *record;
  uint32_t k2;
  uint32_t reserved;
};

/* Bytes of one record of `projection` at `k2`, padded to 4096. reference: ignis_moe.h:73 */
int32_t ignis_moe_record_bytes(uint32_t projection, uint32_t k2, uint64_t *bytes);

/* A trellis tensor decoded to fp16 [in][out], bit for bit exllamav3's `reconstruct`; `in` and
 * `out` multiples of 16. reference: ignis_moe.h:80-81 */
int32_t ignis_moe_trellis_reconstruct(const void *trellis, uint32_t k2, uint32_t in, uint32_t out,
                                      void *w_f16, void *stream);

/* The router: logits = x . W^T over the BF16 weight [experts][hidden], fp32 accumulate, rounded
 * once to BF16; the top_k largest BF16 logits (ties to the lower id) to `ids` [tokens][top_k] in
 * descending order; their softmax in fp32 rounded to BF16, stored as fp32, to `weights`;
 * `logits` [tokens][experts] receives the fp32 logits. reference: ignis_moe.h:93-94 */
int32_t ignis_moe_router(const void *x, uint32_t tokens, const void *w_router, int32_t *ids,
                         float *weights, float *logits, void *stream);

/* The router's first launch alone. reference: ignis_moe.h:99-100 */
int32_t ignis_moe_router_logits(const void *x, uint32_t tokens, const void *w_router, float *logits,
                                void *stream);

/* Prepares the current device for every op here. reference: ignis_moe.h:108 */
int32_t ignis_moe_prepare(void);

#define IGNIS_MOE_DECODE_TICKETS 0   /* ignis_moe.h:131-133; all three run the same kernels here */
#define IGNIS_MOE_DECODE_CLUSTERS 1
#define IGNIS_MOE_DECODE_REGISTERS 2
/* reference: ignis_moe.h:134-139 (24 bytes) */
struct ignis_moe_workspace {
  void *base;
  uint32_t decode_tokens;
  uint32_t prefill_tokens;
  uint32_t decode_route;
};

/* Bytes `base` must hold. reference: ignis_moe.h:142. For more than 8 prefill tokens this includes the
 * weighted down products of the tensor-core route before they are added to `acc`: 4 bytes x tokens
 * x top_k x hidden (335 MB at 4096 tokens of the 2048 / top-10 geometry). */
uint64_t ignis_moe_workspace_bytes(uint32_t decode_tokens, uint32_t prefill_tokens);

/* Makes a fresh workspace ready and zeroes `acc` (int64 [max(decode, prefill)][hidden]); prepares
 * the device. reference: ignis_moe.h:147-148 */
int32_t ignis_moe_workspace_init(const struct ignis_moe_workspace *workspace, int64_t *acc, void *stream);

/* The plan lines of one MoE block. reference: ignis_moe.h:152-160 */
struct ignis_moe_plan {
  uint64_t workspace;
  uint64_t acc;    /* int64 [max][hidden] */
  uint64_t router; /* ids int32 [max][top_k], weights fp32 [max][top_k], logits fp32 [max][experts] */
  uint64_t shared; /* h BF16 [max][inter] and output fp32 [max][hidden] */
  uint64_t total;  /* the four lines, each rounded up to 256 bytes */
};
int32_t ignis_moe_plan_bytes(uint32_t decode_tokens, uint32_t prefill_tokens, struct ignis_moe_plan *plan);

/* The selected experts of every token, weighted and summed into `acc` (value = acc * 2^-32; the
 * ops ADD into it). Decode: 1..workspace->decode_tokens tokens; prefill: 1..prefill_tokens.
 * reference: ignis_moe.h:185-192 */
int32_t ignis_moe_experts_decode(const void *x, uint32_t tokens, const int32_t *ids, const float *weights,
                                 const struct ignis_moe_slot *slots, const struct ignis_moe_workspace *workspace,
                                 int64_t *acc, void *stream);
int32_t ignis_moe_experts_prefill(const void *x, uint32_t tokens, const int32_t *ids, const float *weights,
                                  const struct ignis_moe_slot *slots, const struct ignis_moe_workspace *workspace,
                                  int64_t *acc, void *stream);

/* CTAs per expert cluster of the IGNIS_MOE_DECODE_CLUSTERS route: 0 here, that route does not
 * exist as a separate kernel. reference: ignis_moe.h:197 */
int32_t ignis_moe_decode_cluster_size(void);

/* The shared expert's SwiGLU on FP8 row-scale weights (E4M3FN codes [rows][cols], zero padding to
 * 256 bytes, BF16 scales [rows]: kernel/include/ignis_fp8_linear.h:4-10): gate and up
 * [inter][hidden], down [hidden][inter], into `shared` fp32 [tokens][hidden]; `h` is BF16
 * [tokens][inter] scratch. reference: ignis_moe.h:203-204
 * Up to 8 tokens a warp per row; up to 64 warp-level MMAs; beyond (widths multiples of 128, x and h
 * 16-byte aligned) the codes are widened exactly to BF16 in shared memory and multiplied by
 * tcgen05, whose bounded waits report through bit 3 of ignis_moe_workspace_status. */
int32_t ignis_moe_shared_expert(const void *gate, const void *up, const void *down, const void *x,
                                uint32_t tokens, void *h, float *shared, void *stream);

/* out[t] = BF16(acc[t] * 2^-32 + sigmoid(x_t . w_gate) * shared[t]); zeroes acc behind it.
 * reference: ignis_moe.h:208-209 */
int32_t ignis_moe_combine(int64_t *acc, const float *shared, const void *x, const void *w_gate,
                          uint32_t tokens, void *out, void *stream);

/* Blocks the host until `stream` is idle. reference: ignis_moe.h:213 */
int32_t ignis_moe_stream_sync(void *stream);

/* No counterpart in the reference (its kernels trap instead): copies the workspace's status word
 * to `*status` and blocks until `stream` is idle. Bit 0: an expert id outside the table; bit 1: a
 * selected record absent or of a k2 the experts do not take; bit 2: a contribution not finite or
 * beyond the accumulator's range. Each was skipped, never read as weights. Bit 3: a bounded
 * device-side wait of the tensor-core expert kernels (calls of more than 64 tokens) ran out; that
 * call's sums are not valid. */
int32_t ignis_moe_workspace_status(const struct ignis_moe_workspace *workspace, void *stream, uint32_t *status);

/* The geometry-taking variants (see b200q_moe_geometry above). */
int32_t b200q_moe_record_bytes(const b200q_moe_geometry *geometry, uint32_t projection, uint32_t k2, uint64_t *bytes);
uint64_t b200q_moe_workspace_bytes(const b200q_moe_geometry *geometry, uint32_t decode_tokens, uint32_t prefill_tokens);
int32_t b200q_moe_workspace_init(const b200q_moe_geometry *geometry, const struct ignis_moe_workspace *workspace, int64_t *acc,
                                 void *stream);
int32_t b200q_moe_plan_bytes(const b200q_moe_geometry *geometry, uint32_t decode_tokens, uint32_t prefill_tokens,
                             struct ignis_moe_plan *plan);
int32_t b200q_moe_router_logits(const b200q_moe_geometry *geometry, const void *x, uint32_t tokens, const void *w_router,
                                float *logits, void *stream);
int32_t b200q_moe_router(const b200q_moe_geometry *geometry, const void *x, uint32_t tokens, const void *w_router, int32_t *ids,
                         float *weights, float *logits, void *stream);
int32_t b200q_moe_experts_decode(const b200q_moe_geometry *geometry, const void *x, uint32_t tokens, const int32_t *ids,
                                 const float *weights, const struct ignis_moe_slot *slots,
                                 const struct ignis_moe_workspace *workspace, int64_t *acc, void *stream);
int32_t b200q_moe_experts_prefill(const b200q_moe_geometry *geometry, const void *x, uint32_t tokens, const int32_t *ids,
                                  const float *weights, const struct ignis_moe_slot *slots,
                                  const struct ignis_moe_workspace *workspace, int64_t *acc, void *stream);
int32_t b200q_moe_shared_expert(const b200q_moe_geometry *geometry, const void *gate, const void *up, const void *down,
                                const void *x, uint32_t tokens, void *h, float *shared, void *stream);
int32_t b200q_moe_combine(const b200q_moe_geometry *geometry, int64_t *acc, const float *shared, const void *x,
                          const void *w_gate, uint32_t tokens, void *out, void *stream);

/* Thread-local message of the most recent failed call. Never NULL. reference: ignis_moe.h:216 */
const char *ignis_moe_last_error(void);

#ifdef __cplusplus
}
#endif

#endif /* IGNIS_MOE_H */
