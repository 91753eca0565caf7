// Dense trellis linear: the entry points of include/ignis_trellis_linear.h and their kernels.
//
// Format (the reference's definition: kernel/src/trellis_decode.cuh:6-24,
// kernel/tests/fixtures/flash_next/record.py:84-160): a 16 x 16 tile is a bitstream of 256 steps,
// step p adding k_p bits (K, or 2/3 alternating for K = 2.5), big-endian inside little-endian u32
// words; the state of step p is the 16 stream bits ending at end_p (wrapping around the tile), its
// value fp16((1024 + bytesum(state * 0x83DCD12D)) * h(0x1EEE) + h(0xC931)) with one rounding, and
// steps 8 t .. 8 t + 7 are the elements lane t of a warp holds in an m16n8k16 fragment.
//
// Decode on this GPU: a lane funnels the (at most three) words that hold its window into two
// registers with its first bit on top, cuts each state with one or two shifts whose distances are
// compile-time constants of K, and maps it with IMAD, DP4A (the byte sum lands on the fp16 bits of
// 1024 + sum) and half an HFMA2. The eight values of a lane are, without any shuffle, the A
// fragment of the transposed tile (M = output column, K = input row), so tokens are the MMA's N.
//
// The linear (1..8 tokens per pass): one kernel. A CTA serves one block of 128 output columns and
// a slice of the 128-input blocks; it first rotates its slice of the activations (x o suh, then
// the 128-wide Hadamard in fp32 on a warp, a power-of-two scale per token and block, fp16) into
// B fragments in shared memory, then each warp walks its blocks: 8 tiles per 16 inputs, decoded
// and multiplied with fp32 accumulation, folded by the block's inverse scale every 128 inputs.
// Warps meet in shared memory, the CTAs of a cluster (the split of the inputs) in distributed
// shared memory, in a fixed order; the first CTA applies the output Hadamard, svh and the
// epilogue. Weight words are prefetched one 16-input step ahead, the first before the grid waits
// for its predecessor in the stream.
#include "../../include/ignis_trellis_linear.h"

#include "trellis_device.cuh"

namespace b200q {
namespace {

using namespace trellis_dev;

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr uint32_t kMaxSliceBlocks = 40;  // 128-input blocks of rotated activations a CTA holds (80 KB)

// ---- reconstruct: one warp per tile ---------------------------------------------------------
__global__ void __launch_bounds__(kThreads) trellis_reconstruct_kernel(const uint32_t *__restrict__ trellis, uint32_t k2,
                                                                       uint32_t tiles_k, uint32_t tiles_n,
                                                                       uint32_t tile_stride, uint16_t *__restrict__ out) {
  const int lane = threadIdx.x & 31;
  const LaneWindow win = lane_window(k2, lane);
  const uint64_t tiles = static_cast<uint64_t>(tiles_k) * tiles_n;
  const uint32_t ld = tiles_n * 16u;
  const int r0 = (lane & 3) * 2, c0 = lane >> 2;
  for (uint64_t tile = static_cast<uint64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5); tile < tiles;
       tile += static_cast<uint64_t>(gridDim.x) * kWarps) {
    const uint32_t tk = static_cast<uint32_t>(tile / tiles_n), tn = static_cast<uint32_t>(tile % tiles_n);
    const uint32_t *words = trellis + (static_cast<uint64_t>(tk) * tile_stride + tn) * (4u * k2);
    uint32_t frag[4];
    decode8_any(k2, words[win.w0], words[win.w1], words[win.w2], win.off, frag);
    uint16_t *dst = out + static_cast<uint64_t>(tk * 16u + r0) * ld + tn * 16u + c0;
    dst[0] = static_cast<uint16_t>(frag[0] & 0xFFFFu);
    dst[ld] = static_cast<uint16_t>(frag[0] >> 16);
    dst[8 * static_cast<uint64_t>(ld)] = static_cast<uint16_t>(frag[1] & 0xFFFFu);
    dst[9 * static_cast<uint64_t>(ld)] = static_cast<uint16_t>(frag[1] >> 16);
    dst[8] = static_cast<uint16_t>(frag[2] & 0xFFFFu);
    dst[ld + 8] = static_cast<uint16_t>(frag[2] >> 16);
    dst[8 * static_cast<uint64_t>(ld) + 8] = static_cast<uint16_t>(frag[3] & 0xFFFFu);
    dst[9 * static_cast<uint64_t>(ld) + 8] = static_cast<uint16_t>(frag[3] >> 16);
  }
}

// ---- the linear -------------------------------------------------------------------------------

struct TrellisSide {
  const uint32_t *trellis;
  const uint16_t *suh;
  const uint16_t *svh;
  uint32_t k2;
  uint32_t tile_stride;
};

struct TrellisParams {
  TrellisSide side[2];  // [1] is the up weight of a SwiGLU call
  const uint16_t *x;    // BF16 [tokens][in]
  uint16_t *y;          // BF16 [tokens][ldy]
  uint32_t in, out, tokens, ldy;
  uint32_t epilogue;    // 0 store, 1 add, 2 SwiGLU
  uint32_t kc;          // cluster size: slices of the input blocks
  uint32_t slice_cap;   // 128-input blocks the shared-memory fragment buffer holds
};

constexpr uint32_t kEpiAdd = 1, kEpiSwiglu = 2;  // 0 stores

__global__ void __launch_bounds__(kThreads, 2) trellis_linear_kernel(const __grid_constant__ TrellisParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank(), kc = p.kc;
  const uint32_t col_block = blockIdx.x / kc;
  const bool swiglu = p.epilogue == kEpiSwiglu;
  const int sides = swiglu ? 2 : 1;
  const int side = swiglu ? warp >> 2 : 0;           // which weight this warp multiplies
  const int lanes_per_side = swiglu ? 4 : 8;          // warps sharing a side
  const int wslot = swiglu ? (warp & 3) : warp;       // this warp's index inside its side
  const TrellisSide &S = p.side[side];

  // input blocks of this CTA
  const uint32_t nblk = p.in / 128u;
  const uint32_t b0 = static_cast<uint32_t>(static_cast<uint64_t>(nblk) * rank / kc);
  const uint32_t b1 = static_cast<uint32_t>(static_cast<uint64_t>(nblk) * (rank + 1) / kc);
  const uint32_t slice = b1 - b0;

  // shared memory: [fragments | reduction scratch (aliased)] [part] [inverse scales] [scales]
  const size_t frag_bytes = static_cast<size_t>(sides) * p.slice_cap * 2048u;
  const size_t red_bytes = static_cast<size_t>(kWarps - sides) * 8 * 32 * 16;
  const size_t region = frag_bytes > red_bytes ? frag_bytes : red_bytes;
  uint2 *xs = reinterpret_cast<uint2 *>(smem_raw);                  // [side][block][kt 8][lane 32] (b0, b1)
  float4 *red = reinterpret_cast<float4 *>(smem_raw);               // after the main loop
  float4 *part = reinterpret_cast<float4 *>(smem_raw + region);     // [side][tile 8][lane 32]
  float *inv_s = reinterpret_cast<float *>(smem_raw + region + 2 * 8 * 32 * 16);  // [side][block][token 8]
  float *scale_s = inv_s + static_cast<size_t>(sides) * p.slice_cap * 8;

  const LaneWindow win = lane_window(S.k2, lane);
  const uint32_t tile_words = 4u * S.k2;
  const uint32_t *col_base = S.trellis + static_cast<uint64_t>(col_block) * 8u * tile_words;
  const uint64_t tk_stride = static_cast<uint64_t>(S.tile_stride) * tile_words;
  const uint32_t blk_first = b0 + static_cast<uint32_t>(wslot);  // this warp's first block

  griddep_launch_dependents();
  griddep_wait();

  // ---- rotate the slice of the activations into B fragments (each weight has its own suh) ----
  {
    const uint32_t items = slice * 8u * static_cast<uint32_t>(sides);  // (side, block, token slot), dealt to the warps
    for (uint32_t item = static_cast<uint32_t>(warp); item < items; item += kWarps) {
      const uint32_t tok = item & 7u, bl = (item >> 3) % slice, sd = (item >> 3) / slice;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (tok < p.tokens) {
        const size_t k0 = static_cast<size_t>(b0 + bl) * 128u + 4u * lane;
        const uint2 xb = ldg64_coherent(p.x + static_cast<size_t>(tok) * p.in + k0);
        const uint2 sb = *reinterpret_cast<const uint2 *>(p.side[sd].suh + k0);
        const __half2 s01 = *reinterpret_cast<const __half2 *>(&sb.x), s23 = *reinterpret_cast<const __half2 *>(&sb.y);
        v[0] = bf16_bits_to_f32(xb.x & 0xFFFFu) * __low2float(s01);
        v[1] = __uint_as_float(xb.x & 0xFFFF0000u) * __high2float(s01);
        v[2] = bf16_bits_to_f32(xb.y & 0xFFFFu) * __low2float(s23);
        v[3] = __uint_as_float(xb.y & 0xFFFF0000u) * __high2float(s23);
      }
      hadamard128(v, lane);
      float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
      int shift = 0;
      if (m > 0.0f && m <= 3.0e38f) {
        int e;
        (void)frexpf(m, &e);
        shift = max(-126, min(126, 14 - e));
      }
      const float scale = ldexpf(1.0f, shift);
      const __half2 h01 = __floats2half2_rn(v[0] * scale, v[1] * scale);
      const __half2 h23 = __floats2half2_rn(v[2] * scale, v[3] * scale);
      // element e = 4 lane + i of the block: step kt = e / 16, inside it k16 = e % 16; the reader
      // lane (g = token, t) keeps k16 in {2t, 2t+1} in .x and {2t+8, 2t+9} in .y
      const int kt = lane >> 2, k16 = (lane & 3) * 4;  // k16 in {0, 4, 8, 12}
      const int t_first = (k16 & 7) >> 1;              // reader t of elements k16, k16 + 1
      const int reg = k16 >> 3;                        // .x or .y
      const size_t blk_slot = static_cast<size_t>(sd) * p.slice_cap + bl;
      uint32_t *dst = reinterpret_cast<uint32_t *>(xs + (blk_slot * 8 + kt) * 32 + tok * 4);
      dst[(t_first) * 2 + reg] = *reinterpret_cast<const uint32_t *>(&h01);
      dst[(t_first + 1) * 2 + reg] = *reinterpret_cast<const uint32_t *>(&h23);
      if (lane == 0) {
        inv_s[blk_slot * 8 + tok] = tok < p.tokens ? ldexpf(1.0f, -shift) : 0.0f;
        scale_s[blk_slot * 8 + tok] = scale;
      }
    }
  }
  __syncthreads();

  // ---- main loop: this warp's blocks, 8 steps of 16 inputs each ----
  float tot[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) tot[j][e] = 0.0f;
  {
    const size_t side_slot = static_cast<size_t>(side) * p.slice_cap;
    const uint2 *xs_side = xs + side_slot * 8 * 32;
    const float *inv_side = inv_s + side_slot * 8, *scale_side = scale_s + side_slot * 8;
    switch (S.k2) {
      case 4: walk_blocks<4>(col_base, tk_stride, win, blk_first, b0, b1, lanes_per_side, xs_side, inv_side, scale_side, lane, tot); break;
      case 5: walk_blocks<5>(col_base, tk_stride, win, blk_first, b0, b1, lanes_per_side, xs_side, inv_side, scale_side, lane, tot); break;
      case 6: walk_blocks<6>(col_base, tk_stride, win, blk_first, b0, b1, lanes_per_side, xs_side, inv_side, scale_side, lane, tot); break;
      case 8: walk_blocks<8>(col_base, tk_stride, win, blk_first, b0, b1, lanes_per_side, xs_side, inv_side, scale_side, lane, tot); break;
      case 10: walk_blocks<10>(col_base, tk_stride, win, blk_first, b0, b1, lanes_per_side, xs_side, inv_side, scale_side, lane, tot); break;
      default: walk_blocks<12>(col_base, tk_stride, win, blk_first, b0, b1, lanes_per_side, xs_side, inv_side, scale_side, lane, tot); break;
    }
  }

  // ---- reduce the warps of each side (fixed order), then the cluster ----
  __syncthreads();  // the fragments are dead: the reduction scratch aliases them
  if (wslot > 0) {
    const int slot = side * (lanes_per_side - 1) + (wslot - 1);
#pragma unroll
    for (int j = 0; j < 8; ++j) red[(slot * 8 + j) * 32 + lane] = make_float4(tot[j][0], tot[j][1], tot[j][2], tot[j][3]);
  }
  __syncthreads();
  if (wslot == 0) {
    for (int o = 1; o < lanes_per_side; ++o) {
      const int slot = side * (lanes_per_side - 1) + (o - 1);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 v = red[(slot * 8 + j) * 32 + lane];
        tot[j][0] += v.x;
        tot[j][1] += v.y;
        tot[j][2] += v.z;
        tot[j][3] += v.w;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) part[(side * 8 + j) * 32 + lane] = make_float4(tot[j][0], tot[j][1], tot[j][2], tot[j][3]);
  }
  cluster_barrier();

  // ---- the first CTA of the cluster finishes: warp = token, lane = 4 output columns ----
  if (rank == 0 && static_cast<uint32_t>(warp) < p.tokens) {
    const int tok = warp;
    const int tq = tok >> 1, te = tok & 1;
    float v[2][4];
#pragma unroll
    for (int sd = 0; sd < 2; ++sd) {
#pragma unroll
      for (int i = 0; i < 4; ++i) v[sd][i] = 0.0f;
    }
    for (int sd = 0; sd < sides; ++sd) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 4 * lane + i;  // column inside the block
        const int j = c >> 4, cc = c & 15;
        const float *src = reinterpret_cast<const float *>(&part[(sd * 8 + j) * 32 + (cc & 7) * 4 + tq]) + te + 2 * (cc >> 3);
        float sum = 0.0f;
        for (uint32_t r = 0; r < kc; ++r) sum += ld_cluster_f32(src, r);
        v[sd][i] = sum;
      }
      hadamard128(v[sd], lane);
      const uint2 sv = *reinterpret_cast<const uint2 *>(p.side[sd].svh + static_cast<size_t>(col_block) * 128u + 4u * lane);
      const __half2 s01 = *reinterpret_cast<const __half2 *>(&sv.x), s23 = *reinterpret_cast<const __half2 *>(&sv.y);
      v[sd][0] *= __low2float(s01);
      v[sd][1] *= __high2float(s01);
      v[sd][2] *= __low2float(s23);
      v[sd][3] *= __high2float(s23);
    }
    uint16_t *dst = p.y + static_cast<size_t>(tok) * p.ldy + static_cast<size_t>(col_block) * 128u + 4u * lane;
    float r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = swiglu ? v[0][i] / (1.0f + __expf(-v[0][i])) * v[1][i] : v[0][i];
    if (p.epilogue == kEpiAdd) {
      const uint2 old = *reinterpret_cast<const uint2 *>(dst);
      r[0] += bf16_bits_to_f32(old.x & 0xFFFFu);
      r[1] += __uint_as_float(old.x & 0xFFFF0000u);
      r[2] += bf16_bits_to_f32(old.y & 0xFFFFu);
      r[3] += __uint_as_float(old.y & 0xFFFF0000u);
    }
    const __nv_bfloat162 o01 = __floats2bfloat162_rn(r[0], r[1]), o23 = __floats2bfloat162_rn(r[2], r[3]);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t *>(&o01);
    packed.y = *reinterpret_cast<const uint32_t *>(&o23);
    *reinterpret_cast<uint2 *>(dst) = packed;
  }
  cluster_barrier();  // peers keep their partial sums alive until the first CTA has read them
}

size_t linear_smem_bytes(uint32_t slice_cap, int sides) {
  const size_t frag_bytes = static_cast<size_t>(sides) * slice_cap * 2048u;
  const size_t red_bytes = static_cast<size_t>(kWarps - sides) * 8 * 32 * 16;
  return (frag_bytes > red_bytes ? frag_bytes : red_bytes) + 2 * 8 * 32 * 16 +
         static_cast<size_t>(sides) * slice_cap * 8 * 4 * 2;
}

bool aligned(const void *p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

bool valid_k2(uint32_t k2) { return k2 == 4 || k2 == 5 || k2 == 6 || k2 == 8 || k2 == 10 || k2 == 12; }

int32_t check_weight(ErrorSlot &slot, const ignis_trellis_weight *w, const char *what) {
  if (w == nullptr) return fail(slot, "%s: weight is NULL", what);
  if (w->trellis == nullptr || w->suh == nullptr || w->svh == nullptr) return fail(slot, "%s: weight pointers are NULL", what);
  if (!valid_k2(w->k2)) return fail(slot, "%s: k2 = %u is not one of 4, 5, 6, 8, 10, 12", what, w->k2);
  if (w->in == 0 || (w->in % 128u) != 0) return fail(slot, "%s: in = %u is not a positive multiple of 128", what, w->in);
  if (w->out == 0 || (w->out % 128u) != 0 || w->out > IGNIS_TRELLIS_MAX_OUT) {
    return fail(slot, "%s: out = %u is not a positive multiple of 128 up to %d", what, w->out, IGNIS_TRELLIS_MAX_OUT);
  }
  if (w->tile_stride != 0 && w->tile_stride < w->out / 16u) return fail(slot, "%s: tile_stride is narrower than the view", what);
  if (!aligned(w->trellis, 16)) return fail(slot, "%s: trellis is not 16-byte aligned", what);
  if (!aligned(w->suh, 8) || !aligned(w->svh, 8)) return fail(slot, "%s: suh / svh are not 8-byte aligned", what);
  return 0;
}

const DeviceState *prepared(ErrorSlot &slot, const char *what) {
  const DeviceState *dev = device_state(slot);
  if (dev == nullptr) return nullptr;
  if (!dev->prepared) {
    fail(slot, "%s: the device was not prepared (call ignis_trellis_prepare at load)", what);
    return nullptr;
  }
  return dev;
}

TrellisSide make_side(const ignis_trellis_weight *w) {
  TrellisSide s;
  s.trellis = static_cast<const uint32_t *>(w->trellis);
  s.suh = static_cast<const uint16_t *>(w->suh);
  s.svh = static_cast<const uint16_t *>(w->svh);
  s.k2 = w->k2;
  s.tile_stride = w->tile_stride ? w->tile_stride : w->out / 16u;
  return s;
}

// Cluster size for (in, out): enough slices that every slice fits shared memory, then the size
// that fills the device's CTA slots best with the fewest idle warps.
uint32_t plan_kc(const DeviceState &dev, uint32_t in, uint32_t out, int sides) {
  const uint32_t nblk = in / 128u, col_blocks = out / 128u;
  const uint32_t sms = dev.sm_cap > 0 ? static_cast<uint32_t>(dev.sm_cap) : static_cast<uint32_t>(dev.sm_count);
  const double slots = 2.0 * sms;
  const uint32_t warps_per_side = sides == 2 ? 4u : 8u;
  uint32_t best = 0;
  double best_cost = 1e30;
  for (uint32_t kc = 1; kc <= 8; ++kc) {
    if (kc > nblk) break;
    const uint32_t slice = (nblk + kc - 1) / kc;
    if (slice * static_cast<uint32_t>(sides) > kMaxSliceBlocks) continue;
    const double ctas = static_cast<double>(col_blocks) * kc;
    const double waves = ceil(ctas / slots);
    const double per_warp = ceil(static_cast<double>(slice) / warps_per_side);
    // a block of 128 inputs costs 1 per warp; rotating the slice costs about 0.19 per block; 1.5
    // stands for the reductions and the launch ramp
    const double cost = waves * (per_warp + 0.19 * slice / 8.0 * 8.0 / warps_per_side + 1.5) + 0.01 * kc;
    if (cost < best_cost) {
      best_cost = cost;
      best = kc;
    }
  }
  return best;
}

int32_t run_linear(ErrorSlot &slot, const ignis_trellis_weight *a, const ignis_trellis_weight *b, const void *x,
                   uint32_t tokens, void *y, uint32_t ldy, uint32_t epilogue, void *stream, const char *what) {
  if (check_weight(slot, a, what) != 0) return -1;
  const bool swiglu = epilogue == kEpiSwiglu;
  if (swiglu) {
    if (check_weight(slot, b, what) != 0) return -1;
    if (a->in != b->in || a->out != b->out) return fail(slot, "%s: gate and up must share (in, out)", what);
  }
  if (tokens == 0) return fail(slot, "%s: tokens must be positive", what);
  if (x == nullptr || !aligned(x, 16)) return fail(slot, "%s: x is NULL or not 16-byte aligned", what);
  if (y == nullptr || !aligned(y, 8)) return fail(slot, "%s: y is NULL or not 8-byte aligned", what);
  if ((ldy % 4u) != 0 || ldy < a->out) return fail(slot, "%s: ldy = %u must be a multiple of 4 and at least out", what, ldy);
  if (epilogue > kEpiSwiglu) return fail(slot, "%s: unknown epilogue %u", what, epilogue);
  const DeviceState *dev = prepared(slot, what);
  if (dev == nullptr) return -1;
  const int sides = swiglu ? 2 : 1;
  const uint32_t kc = plan_kc(*dev, a->in, a->out, sides);
  if (kc == 0) return fail(slot, "%s: in = %u is too long for one call (at most %u)", what, a->in, 8u * kMaxSliceBlocks * 128u / static_cast<uint32_t>(sides));
  TrellisParams p = {};
  p.side[0] = make_side(a);
  p.side[1] = swiglu ? make_side(b) : p.side[0];
  p.in = a->in;
  p.out = a->out;
  p.ldy = ldy;
  p.epilogue = epilogue;
  p.kc = kc;
  p.slice_cap = (a->in / 128u + kc - 1) / kc;
  const size_t smem = linear_smem_bytes(p.slice_cap, sides);
  for (uint32_t t0 = 0; t0 < tokens; t0 += 8) {
    p.tokens = tokens - t0 < 8u ? tokens - t0 : 8u;
    p.x = static_cast<const uint16_t *>(x) + static_cast<size_t>(t0) * a->in;
    p.y = static_cast<uint16_t *>(y) + static_cast<size_t>(t0) * ldy;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((a->out / 128u) * kc, 1, 1);
    config.blockDim = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kc;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = dev->pdl ? 2 : 1;
    const cudaError_t err = cudaLaunchKernelEx(&config, trellis_linear_kernel, p);
    if (err != cudaSuccess) return fail(slot, "%s: launch failed: %s", what, cudaGetErrorString(err));
  }
  return 0;
}

}  // namespace

// The tile decoder as a launch over any [in][out] tensor with 16-aligned extents: shared by
// ignis_trellis_reconstruct and ignis_moe_trellis_reconstruct.
int32_t trellis_reconstruct_raw(ErrorSlot &slot, const char *what, const void *trellis, uint32_t k2, uint32_t in,
                                uint32_t out, uint32_t tile_stride, void *w_f16, void *stream) {
  if (trellis == nullptr || w_f16 == nullptr) return fail(slot, "%s: NULL argument", what);
  if (!valid_k2(k2)) return fail(slot, "%s: k2 = %u is not one of 4, 5, 6, 8, 10, 12", what, k2);
  if (in == 0 || (in % 16u) != 0 || out == 0 || (out % 16u) != 0) return fail(slot, "%s: in and out must be positive multiples of 16", what);
  if (!aligned(trellis, 4)) return fail(slot, "%s: trellis is not 4-byte aligned", what);
  if (prepared(slot, what) == nullptr) return -1;
  const uint32_t tiles_k = in / 16u, tiles_n = out / 16u;
  const uint32_t stride = tile_stride ? tile_stride : tiles_n;
  const uint64_t tiles = static_cast<uint64_t>(tiles_k) * tiles_n;
  const uint32_t grid = static_cast<uint32_t>(tiles / kWarps + 1 < 148u * 8u ? tiles / kWarps + 1 : 148u * 8u);
  trellis_reconstruct_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t *>(trellis), k2, tiles_k, tiles_n, stride, static_cast<uint16_t *>(w_f16));
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(slot, "%s: launch failed: %s", what, cudaGetErrorString(err));
  return 0;
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int32_t ignis_trellis_prepare(void) {
  ErrorSlot &slot = trellis_error();
  if (prepare_device(slot) != 0) return -1;
  const cudaError_t err = cudaFuncSetAttribute(trellis_linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(linear_smem_bytes(kMaxSliceBlocks, 1)));
  if (err != cudaSuccess) return fail(slot, "ignis_trellis_prepare: %s", cudaGetErrorString(err));
  return 0;
}

uint32_t ignis_trellis_sm_cap(void) {
  const DeviceState *dev = device_state(trellis_error());
  return dev != nullptr && dev->prepared ? static_cast<uint32_t>(dev->sm_cap) : 0u;
}

uint64_t ignis_trellis_workspace_bytes(uint32_t in, uint32_t out, uint32_t weights, uint32_t tokens) {
  const DeviceState *dev = device_state(trellis_error());
  if (dev == nullptr || !dev->prepared) return 0;
  if (in == 0 || (in % 128u) != 0 || out == 0 || (out % 128u) != 0 || out > IGNIS_TRELLIS_MAX_OUT) return 0;
  if (weights < 1 || weights > 2 || tokens == 0) return 0;
  if (plan_kc(*dev, in, out, static_cast<int>(weights)) == 0) return 0;
  return 256;  // partial sums meet in distributed shared memory: one aligned line, never read
}

int32_t ignis_trellis_workspace_init(const ignis_trellis_workspace *workspace, void *stream) {
  ErrorSlot &slot = trellis_error();
  if (workspace == nullptr || workspace->base == nullptr) return fail(slot, "ignis_trellis_workspace_init: workspace is NULL");
  if (!aligned(workspace->base, 256)) return fail(slot, "ignis_trellis_workspace_init: base is not 256-byte aligned");
  if (prepared(slot, "ignis_trellis_workspace_init") == nullptr) return -1;
  const cudaError_t err = cudaMemsetAsync(workspace->base, 0, workspace->bytes, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(slot, "ignis_trellis_workspace_init: %s", cudaGetErrorString(err));
  return 0;
}

int32_t ignis_trellis_linear(const ignis_trellis_weight *w, const void *x, uint32_t tokens, void *y, uint32_t ldy,
                             uint32_t epilogue, const ignis_trellis_workspace *workspace, void *stream) {
  (void)workspace;
  if (epilogue != IGNIS_TRELLIS_STORE && epilogue != IGNIS_TRELLIS_ADD) {
    return fail(trellis_error(), "ignis_trellis_linear: unknown epilogue %u", epilogue);
  }
  return run_linear(trellis_error(), w, nullptr, x, tokens, y, ldy, epilogue, stream, "ignis_trellis_linear");
}

int32_t ignis_trellis_linear_swiglu(const ignis_trellis_weight *gate, const ignis_trellis_weight *up, const void *x,
                                    uint32_t tokens, void *h, uint32_t ldh, const ignis_trellis_workspace *workspace,
                                    void *stream) {
  (void)workspace;
  return run_linear(trellis_error(), gate, up, x, tokens, h, ldh, kEpiSwiglu, stream, "ignis_trellis_linear_swiglu");
}

int32_t ignis_trellis_reconstruct(const ignis_trellis_weight *w, void *w_f16, void *stream) {
  ErrorSlot &slot = trellis_error();
  if (w == nullptr) return fail(slot, "ignis_trellis_reconstruct: weight is NULL");
  return trellis_reconstruct_raw(slot, "ignis_trellis_reconstruct", w->trellis, w->k2, w->in, w->out, w->tile_stride, w_f16,
                                 stream);
}

const char *ignis_trellis_last_error(void) { return trellis_error().text; }

}  // extern "C"
