// Types shared by the NVFP4 kernels and their entry points.
#ifndef B200Q_NVFP4_INTERNAL_CUH
#define B200Q_NVFP4_INTERNAL_CUH

#include "common.cuh"

namespace b200q {

constexpr uint32_t kMaxGroup = 8;  // B200Q_NVFP4_MAX_GROUP

// Epilogue bits as the kernels see them (the public STORE/ADD/OUT_F32 plus the fused SwiGLU).
constexpr uint32_t kEpilogueAdd = 1u;
constexpr uint32_t kEpilogueF32 = 0x100u;
constexpr uint32_t kEpilogueSwiglu = 0x200u;
constexpr uint32_t kEpilogueQuant = 0x400u;  // with SwiGLU on the tensor-core route: h leaves as the next product's NVFP4 operand

constexpr uint32_t kMaxPeers = 8;  // ranks of one node a scattered product writes to

// One synchronization point between the ranks of a node (b200q_peer_sync): every rank owns an array
// of `peers` flags (slot s written by rank s) that all ranks have mapped, and three words of its
// own: state[0] ranks that missed a wait, state[1] the barriers completed at this point, state[2] an
// arrival counter of the waiting launch's CTAs.
struct PeerSync {
  uint32_t *const *flags_peers;  // device array of `peers` pointers; nullptr: not used
  uint32_t *state;
  uint32_t peers, rank;
  uint32_t polls;                // looks at a flag before a wait gives up
};

struct GemvWeight {
  const uint8_t *codes;
  const uint8_t *scales;
  void *y[kMaxPeers];    // [tokens][ldy], BF16 or float32: this rank's buffer, or every rank's (peer mappings)
  uint32_t peers;        // how many of them are written (1 for a plain product)
  uint32_t n;
  uint32_t ldy;
  float inv_dw;          // 1 / weight_scale_divisor
  uint32_t block_begin;  // first CTA of this weight in the launch
};

struct GemvParams {
  GemvWeight w[kMaxGroup];
  const uint16_t *x;  // BF16 [tokens][k]
  uint32_t count;
  uint32_t k;
  uint32_t ksteps;    // ceil(k / 256)
  uint32_t tokens;    // of this pass, at most 8 NT
  uint32_t epilogue;
  uint32_t rm;        // 32-row groups per CTA: 1, 2, 4 or 8
  uint32_t kc;        // cluster size: K slices across CTAs
  uint32_t xs_steps;  // steps of activation fragments shared memory holds at a time
  PeerSync wait;      // before x is read: a barrier between the ranks (every rank's shard of x has landed)
};

struct GemvPlan {
  int rm;
  int kc;
  uint32_t row_blocks;
  uint32_t xs_steps;
};

int32_t gemv_prepare(ErrorSlot &slot);
GemvPlan gemv_plan(const DeviceState &dev, uint32_t groups, uint32_t ksteps, int nt, bool swiglu);
int32_t gemv_launch(ErrorSlot &slot, const DeviceState &dev, GemvParams &p, int nt, const GemvPlan &plan, uint32_t ctas,
                    cudaStream_t stream);

int32_t dequantize_launch(ErrorSlot &slot, const uint8_t *codes, const uint8_t *scales, uint32_t n, uint32_t k, float d_w,
                          float *out, cudaStream_t stream);
int32_t quantize_activations_launch(ErrorSlot &slot, const uint16_t *x, uint32_t tokens, uint32_t k, float d_in,
                                    uint8_t *codes, uint8_t *scales, cudaStream_t stream);

// A16 products on the tensor cores (nvfp4_a16mma.cu): passes of up to 256 tokens.
int32_t a16mma_prepare(ErrorSlot &slot);
bool a16mma_takes(uint32_t k, const void *x);
int32_t a16mma_launch(ErrorSlot &slot, const DeviceState &dev, const GemvWeight *weights, uint32_t count, const uint16_t *x,
                      uint32_t k, uint32_t tokens, uint32_t epilogue, cudaStream_t stream);
int32_t a16mma_status(ErrorSlot &slot, cudaStream_t stream, uint32_t *status);

// W4A4 at decode and verify widths (nvfp4_w4a4_decode.cu): activations quantized inside the kernel,
// no workspace.
constexpr uint32_t kA4DecodeMaxTokens = 32;
struct A4Item {
  const uint8_t *codes;
  const uint8_t *scales;
  void *y;
  uint32_t n, ldy;
  float d_w, d_in;
};
int32_t w4a4_decode_prepare(ErrorSlot &slot);
bool w4a4_decode_takes(uint32_t n, uint32_t k, uint32_t tokens, uint32_t epilogue);
int32_t w4a4_decode_launch(ErrorSlot &slot, const DeviceState &dev, const A4Item *items, uint32_t count, const uint16_t *x,
                           uint32_t k, uint32_t tokens, uint32_t epilogue, cudaStream_t stream);
int32_t w4a4_decode_status(ErrorSlot &slot, cudaStream_t stream, uint32_t *status);

// The tensor-core prefill route (nvfp4_w4a4.cu).
int32_t w4a4_prepare(ErrorSlot &slot);
bool w4a4_shape_ok(uint32_t n, uint32_t k);
uint64_t w4a4_workspace_bytes(uint32_t k, uint32_t tokens);
int32_t w4a4_launch(ErrorSlot &slot, const DeviceState &dev, const uint8_t *w_codes, const uint8_t *w_scales, uint32_t n,
                    uint32_t k, float d_w, float d_in, const uint16_t *x, uint32_t tokens, void *y, uint32_t ldy,
                    uint32_t epilogue, uint8_t *workspace, cudaStream_t stream);
// The same product over activations already quantized in `workspace` by an earlier w4a4_launch of
// the same x, k and token count (split-output parents: one quantization, a product per range).
int32_t w4a4_launch_prequantized(ErrorSlot &slot, const DeviceState &dev, const uint8_t *w_codes, const uint8_t *w_scales,
                                 uint32_t n, uint32_t k, float d_w, float d_in, uint32_t tokens, void *y, uint32_t ldy,
                                 uint32_t epilogue, uint8_t *workspace, cudaStream_t stream);
int32_t w4a4_quantize_range(ErrorSlot &slot, const DeviceState &dev, const uint16_t *x_rows, uint32_t tokens_total,
                            uint32_t token_begin, uint32_t token_count, uint32_t k, float d_in, uint8_t *workspace,
                            cudaStream_t stream);
// The layers' MLP on the tensor-core route: x is quantized, the gate|up product's epilogue writes
// silu(g) u already quantized under `down`'s input divisor, the down product reads it.
uint64_t w4a4_mlp_workspace_bytes(uint32_t k, uint32_t inter, uint32_t tokens);
int32_t w4a4_mlp_launch(ErrorSlot &slot, const DeviceState &dev, const uint8_t *gu_codes, const uint8_t *gu_scales, uint32_t gu_n,
                        uint32_t k, float gu_dw, float gu_din, const uint8_t *dn_codes, const uint8_t *dn_scales, uint32_t dn_n,
                        float dn_dw, float dn_din, const uint16_t *x, uint32_t tokens, void *y, uint32_t ldy, uint32_t epilogue,
                        uint8_t *workspace, cudaStream_t stream);

// The status line of b200q_nvfp4_linear_noalloc's built-in scratch on the current device (0 before
// that entry has run there), read after `stream` has finished.
int32_t w4a4_noalloc_status(ErrorSlot &slot, cudaStream_t stream, uint32_t *status);

}  // namespace b200q

#endif
