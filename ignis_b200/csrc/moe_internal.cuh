// Types shared by the MoE expert kernels (moe.cu) and their tensor-core form (moe_tc.cu).
#ifndef B200Q_MOE_INTERNAL_CUH
#define B200Q_MOE_INTERNAL_CUH

#include "../../include/ignis_moe.h"

#include "common.cuh"

namespace b200q {

constexpr uint32_t kStatusBadExpert = 1u, kStatusAbsentRecord = 2u, kStatusRange = 4u;
constexpr uint32_t kStatusTcWait = 8u;   // a bounded wait of the tensor-core expert kernels ran out

// A work item: up to `item_rows` sorted rows of one expert (64 from the prefill entry, 8 from the
// decode entry), i.e. up to 8 row tiles of 8.
struct Item {
  uint32_t expert, first, count, tile_first;
};
// A row tile: 8 consecutive sorted rows of one expert (the MMA's N), the unit the activations are
// rotated in.
struct Tile {
  uint32_t expert, first, count, pad;
};

struct ExpertParams {
  const int32_t *ids;        // expert of every assignment: [tokens][top_k]
  const ignis_moe_slot *slots;
  const Item *items;
  const Tile *tiles;
  const uint32_t *n_items;  // [0] items, [1] tiles
  const uint32_t *sorted;   // row -> assignment index (token * top_k + rank)
  const uint16_t *x;        // BF16 [tokens][hidden]
  const float *weights;     // routing weights [tokens][top_k]
  uint2 *frag_in;           // rotated x: [tile][hidden / 128][step 8][lane 32]
  float2 *scale_in;         // (inverse scale, scale): [tile][hidden / 128][row 8]
  float *gu;                // fp32 [rows][2 inter]: gate | up products
  uint2 *frag_h;            // rotated silu(g) u: [tile][inter / 128][step 8][lane 32]
  float2 *scale_h;
  float *down_rows;         // fp32 [tokens][top_k][hidden]: the weighted down products of the tensor-core route, before they are added
  long long *acc;           // int64 [tokens][hidden]
  uint32_t *status;
  uint32_t hidden, inter, top_k, experts;
};


// The routed experts of a wide call on the tensor cores (moe_tc.cu): rows rotated once into fp16
// rows with one scale per row, items of up to 256 rows multiplied with their expert's records by
// tcgen05. `p` as for the warp-level kernels; frag_in / scale_in and frag_h / scale_h hold the
// rotated rows and their inverse scales instead of fragments.
int32_t moe_tc_prepare(ErrorSlot &slot);
constexpr uint32_t kMoeTcItemRows = 256;
int32_t moe_tc_experts(ErrorSlot &slot, const DeviceState &dev, const ExpertParams &p, uint32_t rows, uint32_t items_max,
                       const uint32_t *offsets, cudaStream_t stream, const char *what);

// The shared expert of a wide call on the tensor cores (moe_fp8_tc.cu): FP8 rows widened exactly to
// BF16 in swizzled shared memory, BF16 activations by TMA, tcgen05 kind::f16. Takes calls of more
// than 64 tokens whose widths are multiples of 128 and whose x and h are 16-byte aligned.
int32_t moe_fp8_tc_prepare(ErrorSlot &slot);
bool moe_fp8_tc_takes(const DeviceState &dev, uint32_t hidden, uint32_t inter, uint32_t tokens, const void *x, const void *h);
cudaError_t moe_fp8_tc_shared_expert(const DeviceState &dev, const uint8_t *gate, const uint8_t *up, const uint8_t *down, const uint16_t *x,
                                     uint32_t tokens, uint32_t hidden, uint32_t inter, void *h, float *shared, cudaStream_t stream);
cudaError_t moe_fp8_tc_status(uint32_t *status, cudaStream_t stream);   // non-zero: one of its bounded waits ran out

}  // namespace b200q

#endif
