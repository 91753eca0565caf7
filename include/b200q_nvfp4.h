/* NVFP4 linear layers for B200 (sm_100a): flat C ABI.
 *
 * The reference engine has no flat C entry for its NVFP4 linear: the op is the C++ family
 * ninfer::ops::linear (kernel/vendor/include/ninfer/ops/linear.h:20-119), called inside its kernel
 * leaf, and the weight crosses the real step ABI as an `ignis_bound_tensor`
 * (kernel/include/ignis_model.h:79-100: qdata, scales, shape, weight_scale_divisor,
 * input_scale_divisor). This header gives that op the same flat conventions the reference uses
 * for its trellis and MoE ops (kernel/include/ignis_trellis_linear.h): plain pointers and sizes,
 * caller-owned buffers, 0 / -1 return codes with a thread-local message.
 *
 * Weight format (unchanged from the reference's artifact, `blockscale-k16-m128x4-v1`,
 * kernel/vendor/src/ops/linear/nvfp4/nvfp4_format.cpp:38-71, nvfp4_codec.cuh:32-42):
 *   codes   E2M1, [n][k/2] row-major, the even k in the low nibble;
 *   scales  E4M3FN (non-negative, finite), one per 16 along k, swizzled: the scale of
 *           (row r, group g) is byte ((r/128)*(k/64) + g/4)*512 + (r%32)*16 + ((r%128)/32)*4 + g%4;
 *   w[r][c] = E2M1(code) * E4M3(scale) / weight_scale_divisor.
 * n is a positive multiple of 128, k a positive multiple of 64.
 *
 * Conventions of every entry point:
 * - Activations are device-resident, token-major BF16: x [tokens][k] contiguous, 16-byte aligned
 *   (the reference's `[K,T]` tensor with dimension zero fastest). Outputs are [tokens][ldy].
 * - A call enqueues on `stream` (a cudaStream_t, NULL for the legacy stream), allocates nothing
 *   and never synchronizes the host. Scratch lives in the caller's workspace, sized by
 *   b200q_nvfp4_workspace_bytes from the load's maxima; one workspace serves the calls of one
 *   stream in sequence.
 * - Results are deterministic: no floating-point atomics, fixed reduction order.
 * - Return 0 on success, -1 on an argument the op does not accept or a launch error; the reason
 *   is in b200q_nvfp4_last_error(). There is no CPU fallback: without a prepared CUDA device the
 *   calls fail.
 */
#ifndef B200Q_NVFP4_H
#define B200Q_NVFP4_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The fields of the reference's bound NVFP4 tensor that the linear reads
 * (kernel/include/ignis_model.h:79-100; kernel/vendor/src/core/tensor.h:49-75). */
typedef struct b200q_nvfp4_weight {
  const void *codes;  /* device, 32-byte aligned */
  const void *scales; /* device, 16-byte aligned */
  uint32_t n;
  uint32_t k;
  float weight_scale_divisor; /* finite, positive */
  float input_scale_divisor;  /* finite, positive; read by the W4A4 policy only */
} b200q_nvfp4_weight;

typedef struct b200q_nvfp4_workspace {
  void *base;     /* device, 256-byte aligned */
  uint64_t bytes; /* at least what b200q_nvfp4_workspace_bytes asked for */
} b200q_nvfp4_workspace;

/* Activation-compute policy, the reference's LinearPolicy (ninfer/ops/linear.h:20-24):
 * A16 multiplies the exactly decoded weights with the BF16 activations; ALLOW_A4 lets wide calls
 * quantize the activations to NVFP4 (nvfp4_codec.cuh:81-110) and multiply in FP4. */
#define B200Q_NVFP4_A16_ONLY 0
#define B200Q_NVFP4_ALLOW_A4 1
/* Under ALLOW_A4 the reference quantizes the activations of a call from a token count that depends
 * on the problem the weight was registered as (nvfp4_dispatch.cpp:31-39): its fused GDN input
 * always, the attention inputs from 4 tokens, gate|up from 5, the projections back to the residual
 * stream (attention out, GDN out, down) from 8. OR one of these into `policy` to say which problem a
 * call is (a grouped q | k | v call and a fused q|k|gate|v parent are both ATTN_INPUT); without one
 * the problem is told from the weights' proportions. */
#define B200Q_NVFP4_PROBLEM_MASK 0x700u
#define B200Q_NVFP4_PROBLEM_GDN_INPUT 0x100u
#define B200Q_NVFP4_PROBLEM_ATTN_INPUT 0x200u
#define B200Q_NVFP4_PROBLEM_GATE_UP 0x300u
#define B200Q_NVFP4_PROBLEM_RESIDUAL 0x400u

/* Epilogues. STORE and ADD write BF16; OR-ing B200Q_NVFP4_OUT_F32 makes `y` float32 (the FP32
 * accumulators before the final rounding, for numerical checks). Under B200Q_NVFP4_ALLOW_A4 a call
 * of more than B200Q_NVFP4_DECODE_MAX_TOKENS tokens with k a multiple of 256 takes the tensor-core
 * route (activations quantized to NVFP4 under input_scale_divisor, tcgen05 block-scaled MMA,
 * out = BF16(acc / (d_in d_w)): nvfp4_w4a4.cu:37); it serves STORE only, needs the workspace, y
 * 16-byte aligned and ldy a multiple of 8. ADD is the residual add of the
 * reference's linear_add (linear_add/nvfp4/nvfp4_linear_add_epilogue.cuh:9-17): one rounding of
 * acc + float(y). */
#define B200Q_NVFP4_STORE 0
#define B200Q_NVFP4_ADD 1
#define B200Q_NVFP4_OUT_F32 0x100

/* The most weights one b200q_nvfp4_linear_group call takes. */
#define B200Q_NVFP4_MAX_GROUP 8
/* The most tokens the decode route (weights streamed once for all tokens) serves per pass. */
#define B200Q_NVFP4_DECODE_MAX_TOKENS 32

/* Prepares the current device: kernel attributes, SM count, environment switches. Once per
 * device at load, outside any stream capture; the ops refuse to run on an unprepared device.
 * Prepares the whole library (the trellis and MoE kernels too: ignis_trellis_prepare and
 * ignis_moe_prepare do the same), so one call per device is enough whichever family's it is.
 * Stands where the reference configures its ops at ignis_model_load
 * (kernel/include/ignis_model.h:820). */
int32_t b200q_nvfp4_prepare(void);

/* Workspace bytes of a call at (n, k) with `tokens` tokens under `policy`; 0 for a shape the ops
 * refuse. Mirrors linear_workspace_capacity_bytes (ninfer/ops/linear.h:31-35). */
uint64_t b200q_nvfp4_workspace_bytes(uint32_t n, uint32_t k, uint32_t policy, uint32_t tokens);

/* Zeroes the workspace's status line, once after it is reserved (the ops leave it zero unless a
 * device-side wait ran out). Mirrors ignis_trellis_workspace_init
 * (kernel/include/ignis_trellis_linear.h:124). */
int32_t b200q_nvfp4_workspace_init(const b200q_nvfp4_workspace *workspace, void *stream);

/* Copies the workspace's status word to `*status` and blocks until `stream` has finished: 0 when
 * no kernel gave up a bounded wait (bit 0 producer, bit 1 MMA issuer, bit 2 epilogue of the
 * tensor-core route). For tests and tools, like the reference's ignis_moe_stream_sync
 * (kernel/include/ignis_moe.h:212); the reference's own kernels trap or spin instead. */
int32_t b200q_nvfp4_workspace_status(const b200q_nvfp4_workspace *workspace, void *stream, uint32_t *status);

/* y[t][r] = sum_c w[r][c] x[t][c] through `epilogue`: ninfer::ops::linear
 * (ninfer/ops/linear.h:99-119) and, with B200Q_NVFP4_ADD, ninfer::ops::linear_add. */
int32_t b200q_nvfp4_linear(const b200q_nvfp4_weight *w, const void *x, uint32_t tokens, void *y,
                           uint32_t ldy, uint32_t epilogue, uint32_t policy,
                           const b200q_nvfp4_workspace *workspace, void *stream);

/* `count` weights of the same k applied to the same x in one pass, weight i writing
 * y[i][t][..ldy[i]]: the split-output projections the reference fuses into one parent
 * (attn_input_proj's q|k|gate|v rows, kernel/vendor/src/ops/linear/nvfp4/nvfp4_w4a4_tma.cu:23-30;
 * gdn_input_proj's qkv|z), kept here as separate matrices sharing the activation read. */
int32_t b200q_nvfp4_linear_group(const b200q_nvfp4_weight *const *w, uint32_t count, const void *x,
                                 uint32_t tokens, void *const *y, const uint32_t *ldy,
                                 uint32_t epilogue, uint32_t policy,
                                 const b200q_nvfp4_workspace *workspace, void *stream);

/* One parent weight, `count` row ranges of it, each range its own output: the single-parent
 * split-output projections of the reference - ninfer::ops::attn_input_proj over the NVFP4
 * [14336, 5120] parent with row counts 6144 | 1024 | 6144 | 1024 (q | k | gate | v;
 * ninfer/ops/attn_input_proj.h:75-91) and gdn_input_proj (qkv 10240 | z 6144). Range i is rows
 * [row_begin[i], row_begin[i] + rows[i]) (multiples of 128: whole scale tiles, so every range is a
 * contiguous byte range of both planes) and writes y[i][t][..ldy[i]]; no packed parent output is
 * materialized. STORE only (BF16 or B200Q_NVFP4_OUT_F32). Narrow calls and A16: one decode launch over all ranges. Wide
 * calls under B200Q_NVFP4_ALLOW_A4: x is quantized once into the workspace
 * (b200q_nvfp4_workspace_bytes of the parent) and every range is one tensor-core product. */
int32_t b200q_nvfp4_linear_split(const b200q_nvfp4_weight *parent, uint32_t count, const uint32_t *row_begin,
                                 const uint32_t *rows, const void *x, uint32_t tokens, void *const *y,
                                 const uint32_t *ldy, uint32_t epilogue, uint32_t policy,
                                 const b200q_nvfp4_workspace *workspace, void *stream);

/* h[t][c] = BF16(silu(g) * u), g and u the products with rows [0, n/2) and [n/2, n) of the fused
 * gate_up parent: ninfer::ops::linear_swiglu at decode widths
 * (linear_swiglu/nvfp4/nvfp4_linear_swiglu_decode.cu:57-69), one rounding from FP32. */
int32_t b200q_nvfp4_linear_swiglu(const b200q_nvfp4_weight *gate_up, const void *x, uint32_t tokens,
                                  void *h, uint32_t ldh, uint32_t policy,
                                  const b200q_nvfp4_workspace *workspace, void *stream);

/* Column-sharded layers on the GPUs of one node. Not in the (single-GPU) reference.
 *
 * b200q_nvfp4_linear_group_scatter is b200q_nvfp4_linear_group on the decode route whose epilogue
 * stores every value into `peers` buffers instead of one: weight i's output [tokens][n_i] lands at
 * column col_offset[i] of y_peers[i * peers + p] (row stride ldy[i]) for every p < peers. One of
 * the pointers is this rank's own full-width buffer, the others are the same buffer of the other
 * ranks, mapped into this process (CUDA IPC or symmetric memory): the product IS the all-gather's
 * data movement, as plain stores over NVLink. STORE, BF16 or B200Q_NVFP4_OUT_F32.
 *
 * b200q_peer_barrier is the rest of the all-gather: barrier number `epoch` (1, 2, ...) between the
 * ranks, on the device, in stream order behind the product. flags_peers is a DEVICE array of
 * `peers` pointers, entry p the flag array (`peers` uint32, zero at start) of rank p, mapped like
 * the buffers. This rank publishes `epoch` in slot `rank` of every array and waits until every
 * slot of its own array has reached it; the wait is bounded (about two seconds; the number of
 * looks at a flag, 400 ns apart, is read from B200Q_PEER_BARRIER_POLLS at prepare), and a wait that
 * runs out sets bit p of status[0] for each rank p that did not arrive, after which the kernel
 * returns and later barriers on the same arrays still work. `status` is two uint32 of
 * this rank's device memory, zero at start; with epoch = 0 the kernel numbers the barrier itself
 * from status[1] (for launches captured in a CUDA graph; every rank must then pass 0 every time). */
int32_t b200q_nvfp4_linear_group_scatter(const b200q_nvfp4_weight *const *w, uint32_t count, const void *x,
                                         uint32_t tokens, void *const *y_peers, uint32_t peers,
                                         const uint32_t *ldy, const uint32_t *col_offset, uint32_t epilogue,
                                         void *stream);
int32_t b200q_peer_barrier(uint32_t *const *flags_peers, uint32_t peers, uint32_t rank, uint32_t epoch,
                           uint32_t *status, void *stream);

/* The same all-gather with no barrier launch at all: the barrier rides in the first instructions of
 * the product that READS the gathered buffer. Not in the reference.
 *
 * b200q_nvfp4_linear_group_gather is b200q_nvfp4_linear_group_scatter with one more argument. With
 * `rejoin` non-NULL the call's x is a buffer that every rank's previous call in its stream stored
 * its columns into (a scatter or gather product, or any kernel): before the call reads x, its first
 * CTA publishes the next barrier number of the point in slot `rank` of every rank's flag array
 * (system-scope release; this rank's own stores into the buffers are complete, being an earlier
 * kernel of the same stream) and every CTA waits until all slots of this rank's own array have
 * reached that number. The wait is bounded like b200q_peer_barrier's; when it runs out the call goes
 * on, state[0] says who was missing and the output is not valid.
 *
 * A b200q_peer_sync names one point of a layer where outputs are rejoined (after `o`, after
 * gate|up, after `down`): flags_peers as for b200q_peer_barrier (a DEVICE array of `peers` pointers,
 * entry p rank p's flag array of `peers` uint32, zero at start), and `state`, three uint32 of this
 * rank's device memory, zero at start: [0] bit p set when rank p was missing from a wait that ran
 * out, [1] barriers completed at this point, [2] an arrival counter. All ranks make the same
 * sequence of calls. Counting happens on the device, so a captured sequence replays. With peers = 1
 * and `rejoin` NULL this is b200q_nvfp4_linear_group.
 *
 * Reuse rule for a gathered buffer: rank A's next product into a buffer may start while rank B
 * still reads the buffer's previous contents unless something orders them. Give every point TWO
 * buffers used alternately (layer parity): before a rank stores into a buffer for the second time
 * after a use, it has passed the point's NEXT barrier, which every other rank joins only after its
 * reader of that use is done (stream order). The same rule makes b200q_nvfp4_linear_group_scatter +
 * b200q_peer_barrier safe; with a single buffer per point put a second barrier behind the reader. */
typedef struct b200q_peer_sync {
  uint32_t *const *flags_peers;
  uint32_t *state;
  uint32_t peers;
  uint32_t rank;
} b200q_peer_sync;
int32_t b200q_nvfp4_linear_group_gather(const b200q_nvfp4_weight *const *w, uint32_t count, const void *x,
                                        uint32_t tokens, void *const *y_peers, uint32_t peers, const uint32_t *ldy,
                                        const uint32_t *col_offset, uint32_t epilogue,
                                        const b200q_peer_sync *rejoin, void *stream);

/* The layers' MLP: y (+)= down(silu(g) * u), g | u = gate_up x. reference:
 * ignis::prefill_swiglu::mlp (kernel/src/prefill_swiglu.h:100-107) and, below its widths, the
 * linear_swiglu + linear_add pair it falls back to. `epilogue` is B200Q_NVFP4_STORE or
 * B200Q_NVFP4_ADD (the residual form), optionally with B200Q_NVFP4_OUT_F32.
 * Above 32 tokens under B200Q_NVFP4_ALLOW_A4 (k and n / 2 multiples of 256): x is quantized once,
 * the gate|up product's epilogue writes BF16(silu(BF16(g)) * BF16(u)) already quantized under
 * `down`'s input divisor - byte for byte what the down product's own quantizer would write from
 * the BF16 matrix (gate_up_swiglu_nvfp4, prefill_swiglu.h:84-92), which is never written - and the
 * down product reads it. Otherwise the decode route's fused SwiGLU writes h (BF16) into the
 * workspace and the decode route's down product reads it.
 * The workspace (256-byte aligned, b200q_nvfp4_mlp_workspace_bytes, its first 256 bytes cleared
 * once by b200q_nvfp4_workspace_init) holds the operands in between. */
uint64_t b200q_nvfp4_mlp_workspace_bytes(uint32_t gate_up_n, uint32_t k, uint32_t policy, uint32_t tokens);
int32_t b200q_nvfp4_mlp(const b200q_nvfp4_weight *gate_up, const b200q_nvfp4_weight *down, const void *x,
                        uint32_t tokens, void *y, uint32_t ldy, uint32_t epilogue, uint32_t policy,
                        const b200q_nvfp4_workspace *workspace, void *stream);

/* The logical weight as float32 [n][k], bit for bit the reference's host dequantizer
 * (kernel/vendor/tests/ops/quantized_weight.h:642-690). Not on the serving path: the seam the
 * decode is held to, as ignis_trellis_reconstruct is for the trellis. */
int32_t b200q_nvfp4_dequantize(const b200q_nvfp4_weight *w, float *out, void *stream);

/* The activation block quantizer of the W4A4 route as a seam: x BF16 [tokens][k] to E2M1 codes
 * [tokens][k/2] and E4M3 scales [tokens][k/16], token-major, bit for bit
 * kernel/vendor/src/ops/linear/nvfp4/nvfp4_codec.cuh:81-110 (nvfp4_w4a4_mma.cuh:388-409). */
int32_t b200q_nvfp4_quantize_activations(const void *x, uint32_t tokens, uint32_t k,
                                         float input_scale_divisor, void *codes, void *scales,
                                         void *stream);

/* The W4A4 route in its two halves, for callers that share the quantized operand: several products
 * over one x, or token-sharded quantization across the GPUs of a node (each rank quantizes its
 * tokens, the ranks all-gather the operand's bytes, every rank multiplies its row shard). Not in
 * the reference, whose fused ops quantize inside one call (nvfp4_w4a4.cu:74-110).
 *
 * The operand of a call of `tokens_total` tokens at `k` lives in a workspace of
 * b200q_nvfp4_workspace_bytes(n, k, B200Q_NVFP4_ALLOW_A4, tokens_total) bytes (any n): 256 bytes of
 * status, the codes [ceil128(tokens_total)][k / 2], then the scales as 512-byte tiles of (128 tokens
 * x 4 groups), token tile major. b200q_nvfp4_quantize_operand writes tokens [token_begin,
 * token_begin + token_count) of it from `x_rows` (the first of those tokens; BF16 [token_count][k]):
 * token_begin a multiple of 128, token_count a multiple of 128 unless the range is the call's last
 * (whose padding rows are written as zeros). The bytes of a token range are therefore two
 * contiguous pieces: codes at 256 + token_begin k / 2, scales at 256 + ceil128(tokens_total) k / 2
 * + (token_begin / 128) (k / 64) 512. b200q_nvfp4_linear_prequantized is the product over a complete
 * operand: the result of b200q_nvfp4_linear under B200Q_NVFP4_ALLOW_A4 on the tensor-core route, bit
 * for bit, for any token count. */
int32_t b200q_nvfp4_quantize_operand(const void *x_rows, uint32_t tokens_total, uint32_t token_begin,
                                     uint32_t token_count, uint32_t k, float input_scale_divisor,
                                     const b200q_nvfp4_workspace *workspace, void *stream);
int32_t b200q_nvfp4_linear_prequantized(const b200q_nvfp4_weight *w, uint32_t tokens, void *y, uint32_t ldy,
                                        uint32_t epilogue, const b200q_nvfp4_workspace *workspace, void *stream);

/* The tensor-core W4A4 linear without any caller-supplied scratch. No counterpart in the
 * reference: its ops always take a workspace the load reserved.
 *
 * Who it is for: a caller that cannot obtain device memory at the moment it calls - an engine
 * whose device arena was sealed at load with no plan line for this op, a plugin running inside a
 * host that owns all device memory, or a latency-critical loop where cudaMalloc's device-wide
 * synchronisation is not acceptable. The quantized activations and the status line live in an
 * array of B200Q_NVFP4_NOALLOC_SCRATCH_BYTES built into the library's device image; every GPU that
 * loads the library holds that array until the process exits. The call itself allocates nothing,
 * on the host or the device.
 *
 * Same result as b200q_nvfp4_linear under B200Q_NVFP4_ALLOW_A4 (any token count >= 1 takes the
 * tensor-core route here): y = BF16 (or float32 with B200Q_NVFP4_OUT_F32) of acc / (d_in d_w),
 * STORE only, k a multiple of 256, y 16-byte aligned, ldy a multiple of 8.
 * Limit: 256 + ceil128(tokens) * k * 9 / 16 bytes must fit the array (for example 2048 tokens at
 * k = 5120, 512 tokens at k = 17408); larger calls return -1 and say so.
 * The first call on a device looks the array's address up (cudaGetSymbolAddress, once per device,
 * with that device current); make that first call outside any stream capture. The array's first
 * 256 bytes are the status line of these calls: zero when the library is loaded, kernels only OR
 * bits into it when a bounded device-side wait runs out (the output of that call is then not
 * valid), and b200q_nvfp4_device_status reports it. All calls on a device share the one array and
 * it keeps the previous call's contents (each call rewrites all it reads), so two calls whose
 * kernels overlap on the GPU - different streams, no ordering between them - race; order them. */
#define B200Q_NVFP4_NOALLOC_SCRATCH_BYTES (6u << 20)
int32_t b200q_nvfp4_linear_noalloc(const b200q_nvfp4_weight *w, const void *x, uint32_t tokens, void *y,
                                   uint32_t ldy, uint32_t epilogue, void *stream);

/* The status word of the kernels that take no workspace - A16 calls of more than 16 tokens and
 * B200Q_NVFP4_ALLOW_A4 calls of up to 32 tokens run on the tensor cores with bounded device-side
 * waits - OR-ed with the status line of b200q_nvfp4_linear_noalloc's built-in scratch (bits 0..2 as
 * in b200q_nvfp4_workspace_status): copied to *status after `stream` has finished. 0 unless a wait
 * ran out, in which case that call's output is not valid. The word is per device and sticky. */
int32_t b200q_nvfp4_device_status(void *stream, uint32_t *status);

/* Measurement, not serving: the tensor cores' block-scaled FP4 rate on this device, the denominator
 * the W4A4 prefill GEMM is reported against. Stands where the reference measures its card's MMA
 * peak with a loop over resident operands (kernel/tests/bench_mma_peak.cu:1-25). One launch: every
 * SM (pair = 0: one CTA per SM, M 128 x N 256 x K 64; pair = 1: clusters of two CTAs, cta_group::2,
 * M 256 x N 256 x K 64) issues `iterations` stages of four tcgen05.mma kind::mxf4nvf4 block_scale
 * MMAs over operands that stay in shared and tensor memory; no global traffic. The caller times the
 * launch on `stream`; *flops receives the floating-point operations it performs. `sink` (device,
 * at least one float per CTA: pass the SM count) receives one accumulator word per CTA, or NULL.
 * b200q_nvfp4_mma_peak_status reads the kernel's status word (non-zero: a bounded wait ran out). */
int32_t b200q_nvfp4_mma_peak(uint32_t iterations, uint32_t pair, float *sink, uint32_t sink_count, double *flops,
                             void *stream);
int32_t b200q_nvfp4_mma_peak_status(void *stream, uint32_t *status);

/* Thread-local message from the most recent failed call. Never NULL. */
const char *b200q_nvfp4_last_error(void);

#ifdef __cplusplus
}
#endif

#endif /* B200Q_NVFP4_H */
