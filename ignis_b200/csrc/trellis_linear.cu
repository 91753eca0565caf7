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
// The linear (1..64 tokens per pass): one kernel. A CTA serves one block of 128 output columns and
// a slice of the 128-input blocks; it rotates its slice of the activations (x o suh, then the
// 128-wide Hadamard in fp32 on a warp, a power-of-two scale per token and block, fp16) into B
// fragments in shared memory, a chunk at a time, then warp j walks tile column j down the slice:
// one tile per 16 inputs, decoded once and multiplied with every token tile of 8, fp32
// accumulation, folded by the block's inverse scale every 128 inputs. The CTAs of a cluster (the
// split of the inputs) meet in distributed shared memory in a fixed order; each applies the
// output Hadamard, svh and the epilogue to its share of the tokens. Weight words are requested
// one 128-input block ahead, the first block before the grid waits for its predecessor in the
// stream.
#include "../../include/ignis_trellis_linear.h"

#include "trellis_device.cuh"
#include "trellis_internal.cuh"

namespace b200q {
namespace {

using namespace trellis_dev;

constexpr int kThreads = 256;
constexpr int kWarps = 8;

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

constexpr uint32_t kMaxGroup = 4;  // weights one grouped call takes

// One weight of a call with its output and the first CTA that serves it.
struct TrellisTarget {
  TrellisSide side;
  uint16_t *y;  // BF16 [tokens][ldy]
  uint32_t ldy;
  uint32_t cta_begin;
};

struct TrellisParams {
  TrellisTarget target[kMaxGroup];  // the weights of a grouped call share x (and `in`); a plain call has one
  TrellisSide up;                   // the up weight of a SwiGLU call (target[0] is the gate)
  const uint16_t *x;                // BF16 [tokens][in]
  uint32_t count;
  uint32_t in, tokens;
  uint32_t epilogue;    // 0 store, 1 add, 2 SwiGLU
  uint32_t kc;          // cluster size: slices of the input blocks
  uint32_t chunk;       // 128-input blocks of rotated activations shared memory holds at a time
};

constexpr uint32_t kEpiAdd = 1, kEpiSwiglu = 2;  // 0 stores

// The lane's words of the 8 steps of one 128-input block of one tile column.
struct BlockWords {
  uint32_t w[8][3];
};

// K2 = 0 decodes with the side's runtime k2 (a SwiGLU pair whose weights differ in width).
template <int K2>
__device__ __forceinline__ void decode_tile(uint32_t k2, uint32_t a, uint32_t b, uint32_t c, uint32_t off, uint32_t (&frag)[4]) {
  if (K2 == 0) {
    decode8_any(k2, a, b, c, off, frag);
  } else {
    decode8<(K2 == 0 ? 4 : K2)>(a, b, c, off, frag);
  }
}

// Work split. A CTA serves one block of 128 output columns and a slice of the 128-input blocks
// (the cluster splits the inputs); warp j owns tile column j of the block, all the way down the
// slice, so the warps of a CTA never add into each other and the loop body is one tile: a few
// hundred bytes of code that stay in the instruction cache. The words of the next 128-input block
// are requested as the current block's are consumed (24 registers per weight in flight per lane).
// NT token tiles of 8 share every decoded tile (up to 64 tokens a pass).
template <int K2, int NT, int SIDES, bool GROUP>
__global__ void __launch_bounds__(kThreads, (SIDES == 1 && NT <= 2) ? 3 : ((NT * SIDES <= 8) ? 2 : 1))
    trellis_linear_kernel(const __grid_constant__ TrellisParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank(), kc = p.kc;
  // The target this CTA serves. A plain call (GROUP false) reads target[0] straight from the launch
  // constants, which keeps the walk's address arithmetic on the uniform datapath; a grouped call
  // selects a copy, and pays about 5 % more instructions per tile for it.
  TrellisTarget picked = {};
  if (GROUP) {
    picked = p.target[0];
    if (p.count > 3u && blockIdx.x >= p.target[3].cta_begin) picked = p.target[3];
    else if (p.count > 2u && blockIdx.x >= p.target[2].cta_begin) picked = p.target[2];
    else if (blockIdx.x >= p.target[1].cta_begin) picked = p.target[1];
  }
  const TrellisSide &side0 = GROUP ? picked.side : p.target[0].side;
  uint16_t *const y_out = GROUP ? picked.y : p.target[0].y;
  const uint32_t ldy = GROUP ? picked.ldy : p.target[0].ldy;
  const uint32_t col_block = (blockIdx.x - (GROUP ? picked.cta_begin : 0u)) / kc;

  const uint32_t nblk = p.in / 128u;
  const uint32_t b0 = static_cast<uint32_t>(static_cast<uint64_t>(nblk) * rank / kc);
  const uint32_t b1 = static_cast<uint32_t>(static_cast<uint64_t>(nblk) * (rank + 1) / kc);

  // shared memory: [fragments (side, block, step, token tile, lane)] [part] [inverse scales] [scales]
  const size_t frag_bytes = static_cast<size_t>(SIDES) * p.chunk * NT * 2048u;
  uint2 *xs = reinterpret_cast<uint2 *>(smem_raw);
  float4 *part = reinterpret_cast<float4 *>(smem_raw + frag_bytes);                       // [side][tile column 8][NT][lane 32]
  float *inv_s = reinterpret_cast<float *>(smem_raw + frag_bytes + static_cast<size_t>(SIDES) * 8 * NT * 32 * 16);
  float *scale_s = inv_s + static_cast<size_t>(SIDES) * p.chunk * NT * 8;                  // [side][block][token]

  // the lane's word pointers of this warp's tile column, at the slice's first step
  LaneWindow win[SIDES];
  const uint32_t *q[SIDES][3];
  int64_t step_words[SIDES];
#pragma unroll
  for (int sd = 0; sd < SIDES; ++sd) {
    const TrellisSide &S = sd == 0 ? side0 : p.up;
    win[sd] = lane_window(K2 != 0 ? static_cast<uint32_t>(K2) : S.k2, lane);
    const uint32_t tile_words = 4u * S.k2;
    step_words[sd] = static_cast<int64_t>(S.tile_stride) * tile_words;
    const uint32_t *base = S.trellis + (static_cast<uint64_t>(col_block) * 8u + static_cast<uint32_t>(warp)) * tile_words +
                           static_cast<uint64_t>(b0) * 8u * static_cast<uint64_t>(step_words[sd]);
    q[sd][0] = base + win[sd].w0;
    q[sd][1] = base + win[sd].w1;
    q[sd][2] = base + win[sd].w2;
  }
  BlockWords bw[SIDES];
  if (b0 < b1) {  // the weights never depend on the previous kernel: request the first block now
#pragma unroll
    for (int sd = 0; sd < SIDES; ++sd)
#pragma unroll
      for (int kt = 0; kt < 8; ++kt)
#pragma unroll
        for (int c = 0; c < 3; ++c) bw[sd].w[kt][c] = __ldg(q[sd][c] + kt * step_words[sd]);
  }

  griddep_launch_dependents();
  griddep_wait();

  float tot[SIDES][NT][4];
#pragma unroll
  for (int sd = 0; sd < SIDES; ++sd)
#pragma unroll
    for (int tt = 0; tt < NT; ++tt)
#pragma unroll
      for (int e = 0; e < 4; ++e) tot[sd][tt][e] = 0.0f;
  float carry[SIDES][NT][2];  // the previous block's inverse scales of this lane's two tokens per tile
#pragma unroll
  for (int sd = 0; sd < SIDES; ++sd)
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) carry[sd][tt][0] = carry[sd][tt][1] = 0.0f;
  const int t2 = (lane & 3) * 2;

  for (uint32_t cb = b0; cb < b1; cb += p.chunk) {
    const uint32_t ce = min(cb + p.chunk, b1), nb = ce - cb;
    if (cb != b0) __syncthreads();  // the previous chunk's fragments are no longer read
    // ---- rotate the chunk of the activations into B fragments (each weight has its own suh) ----
    {
      const uint32_t items = nb * 8u * NT * SIDES;  // (side, block, token), dealt to the warps
      for (uint32_t item = static_cast<uint32_t>(warp); item < items; item += kWarps) {
        const uint32_t tok = item % (8u * NT), rest = item / (8u * NT), bl = rest % nb, sd = rest / nb;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (tok < p.tokens) {
          const size_t k0 = static_cast<size_t>(cb + bl) * 128u + 4u * lane;
          const uint2 xb = ldg64_coherent(p.x + static_cast<size_t>(tok) * p.in + k0);
          const uint2 sb = *reinterpret_cast<const uint2 *>((sd == 0 ? side0.suh : p.up.suh) + k0);
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
        // lane (g = token slot, t) keeps k16 in {2t, 2t+1} in .x and {2t+8, 2t+9} in .y
        const int kt = lane >> 2, k16 = (lane & 3) * 4;
        const int t_first = (k16 & 7) >> 1, reg = k16 >> 3;
        const uint32_t tt = tok >> 3, slot = tok & 7u;
        const size_t blk_slot = static_cast<size_t>(sd) * p.chunk + bl;
        uint32_t *dst = reinterpret_cast<uint32_t *>(xs + ((blk_slot * 8 + kt) * NT + tt) * 32 + slot * 4);
        dst[t_first * 2 + reg] = *reinterpret_cast<const uint32_t *>(&h01);
        dst[(t_first + 1) * 2 + reg] = *reinterpret_cast<const uint32_t *>(&h23);
        if (lane == 0) {
          inv_s[blk_slot * 8 * NT + tok] = tok < p.tokens ? ldexpf(1.0f, -shift) : 0.0f;
          scale_s[blk_slot * 8 * NT + tok] = scale;
        }
      }
    }
    __syncthreads();

    // ---- this warp's tile column down the chunk ----
    for (uint32_t bl = 0; bl < nb; ++bl) {
      const bool more = cb + bl + 1 < b1;  // uniform: another block follows in this CTA's slice
#pragma unroll
      for (int sd = 0; sd < SIDES; ++sd) {
        const size_t blk_slot = static_cast<size_t>(sd) * p.chunk + bl;
        // into this block's units: accumulators were in the previous block's
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) {
          const float2 sc = *reinterpret_cast<const float2 *>(scale_s + blk_slot * 8 * NT + tt * 8 + t2);
          const float f0 = carry[sd][tt][0] * sc.x, f1 = carry[sd][tt][1] * sc.y;
          tot[sd][tt][0] *= f0;
          tot[sd][tt][1] *= f1;
          tot[sd][tt][2] *= f0;
          tot[sd][tt][3] *= f1;
          const float2 iv = *reinterpret_cast<const float2 *>(inv_s + blk_slot * 8 * NT + tt * 8 + t2);
          carry[sd][tt][0] = iv.x;
          carry[sd][tt][1] = iv.y;
        }
        if (more) q[sd][0] += 8 * step_words[sd], q[sd][1] += 8 * step_words[sd], q[sd][2] += 8 * step_words[sd];
      }
#pragma unroll
      for (int kt = 0; kt < 8; ++kt) {
#pragma unroll
        for (int sd = 0; sd < SIDES; ++sd) {
          uint32_t frag[4];
          decode_tile<K2>(sd == 0 ? side0.k2 : p.up.k2, bw[sd].w[kt][0], bw[sd].w[kt][1], bw[sd].w[kt][2], win[sd].off, frag);
          if (more) {  // the same step of the next block, into the registers just consumed
#pragma unroll
            for (int c = 0; c < 3; ++c) bw[sd].w[kt][c] = __ldg(q[sd][c] + kt * step_words[sd]);
          }
          const uint2 *xb = xs + ((static_cast<size_t>(sd) * p.chunk + bl) * 8 + kt) * NT * 32 + lane;
#pragma unroll
          for (int tt = 0; tt < NT; ++tt) {
            const uint2 b = xb[tt * 32];
            mma_f16_f32(tot[sd][tt], frag[0], frag[2], frag[1], frag[3], b.x, b.y);
          }
        }
      }
    }
  }
  // back to the activations' own units, and out to the cluster
#pragma unroll
  for (int sd = 0; sd < SIDES; ++sd)
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) {
      tot[sd][tt][0] *= carry[sd][tt][0];
      tot[sd][tt][1] *= carry[sd][tt][1];
      tot[sd][tt][2] *= carry[sd][tt][0];
      tot[sd][tt][3] *= carry[sd][tt][1];
      part[((sd * 8 + warp) * NT + tt) * 32 + lane] = make_float4(tot[sd][tt][0], tot[sd][tt][1], tot[sd][tt][2], tot[sd][tt][3]);
    }
  cluster_barrier();

  // ---- finish: tokens dealt over the cluster's CTAs and their warps; lane = 4 output columns ----
  for (uint32_t tok = rank + kc * static_cast<uint32_t>(warp); tok < p.tokens; tok += kc * kWarps) {
    const uint32_t tt = tok >> 3, slot = tok & 7u;
    const int tq = static_cast<int>(slot >> 1), te = static_cast<int>(slot & 1u);
    float v[SIDES][4];
#pragma unroll
    for (int sd = 0; sd < SIDES; ++sd) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 4 * lane + i;  // column inside the block
        const int j = c >> 4, cc = c & 15;
        const float *src = reinterpret_cast<const float *>(&part[((sd * 8 + j) * NT + tt) * 32 + (cc & 7) * 4 + tq]) + te + 2 * (cc >> 3);
        float sum = 0.0f;
        for (uint32_t r = 0; r < kc; ++r) sum += ld_cluster_f32(src, r);
        v[sd][i] = sum;
      }
      hadamard128(v[sd], lane);
      const uint2 sv = *reinterpret_cast<const uint2 *>((sd == 0 ? side0.svh : p.up.svh) + static_cast<size_t>(col_block) * 128u + 4u * lane);
      const __half2 s01 = *reinterpret_cast<const __half2 *>(&sv.x), s23 = *reinterpret_cast<const __half2 *>(&sv.y);
      v[sd][0] *= __low2float(s01);
      v[sd][1] *= __high2float(s01);
      v[sd][2] *= __low2float(s23);
      v[sd][3] *= __high2float(s23);
    }
    uint16_t *dst = y_out + static_cast<size_t>(tok) * ldy + static_cast<size_t>(col_block) * 128u + 4u * lane;
    float r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = SIDES == 2 ? v[0][i] / (1.0f + __expf(-v[0][i])) * v[SIDES - 1][i] : v[0][i];
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
  cluster_barrier();  // peers keep their partial sums alive until every CTA has read them
}

constexpr size_t kLinearMaxSmem = 200 * 1024;

size_t linear_smem_bytes(uint32_t chunk, int nt, int sides) {
  return static_cast<size_t>(sides) * chunk * nt * 2048u + static_cast<size_t>(sides) * 8 * nt * 32 * 16 +
         static_cast<size_t>(sides) * chunk * nt * 8 * 4 * 2;
}

// Blocks of rotated activations that fit the kernel's shared memory.
uint32_t chunk_cap(int nt, int sides) {
  const size_t fixed = static_cast<size_t>(sides) * 8 * nt * 32 * 16;
  const size_t per_block = static_cast<size_t>(sides) * nt * (2048u + 64u);
  return static_cast<uint32_t>((kLinearMaxSmem - fixed) / per_block);
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

// CTAs of the linear kernel an SM holds at once, by (token tiles x weights).
int ctas_per_sm(int nt, int sides) { return (sides == 1 && nt <= 2) ? 3 : (nt * sides <= 8 ? 2 : 1); }

// Cluster size for (in, out): the one that costs least in waves of CTAs, each costing its warps'
// walk down the slice (one tile per 16 inputs), the rotation of the slice and a fixed part.
uint32_t plan_kc(const DeviceState &dev, uint32_t in, uint32_t out, int nt, int sides) {
  const uint32_t nblk = in / 128u, col_blocks = out / 128u;
  const uint32_t sms = dev.sm_cap > 0 ? static_cast<uint32_t>(dev.sm_cap) : static_cast<uint32_t>(dev.sm_count);
  const double slots = static_cast<double>(ctas_per_sm(nt, sides)) * sms;
  uint32_t best = 1;
  double best_cost = 1e30;
  for (uint32_t kc = 1; kc <= 8; ++kc) {
    if (kc > nblk || static_cast<int>(kc) > dev.trellis_kc_max) break;
    const uint32_t slice = (nblk + kc - 1) / kc;
    const double ctas = static_cast<double>(col_blocks) * kc;
    const double waves = ceil(ctas / slots);
    // in units of one decoded tile: 8 tiles per block and side, the rotation about 1.2 tiles per
    // (block, token, side) shared by 8 warps, 25 for the reductions, the epilogue and the ramp
    const double walk = 8.0 * slice * sides * (1.0 + 0.12 * (nt - 1));
    const double rotate = 1.2 * slice * 8.0 * nt * sides / 8.0;
    const double cost = waves * (walk + rotate + 25.0) + 0.05 * kc;
    if (cost < best_cost) {
      best_cost = cost;
      best = kc;
    }
  }
  return best;
}

template <int K2, int NT, int SIDES>
cudaError_t launch_linear(const cudaLaunchConfig_t &config, const TrellisParams &p) {
  if (SIDES == 1 && p.count > 1u) return cudaLaunchKernelEx(&config, trellis_linear_kernel<K2, NT, 1, true>, p);
  return cudaLaunchKernelEx(&config, trellis_linear_kernel<K2, NT, SIDES, false>, p);
}

template <int K2, int NT>
cudaError_t launch_sides(int sides, const cudaLaunchConfig_t &config, const TrellisParams &p) {
  return sides == 2 ? launch_linear<K2, NT, 2>(config, p) : launch_linear<K2, NT, 1>(config, p);
}

template <int K2>
cudaError_t launch_nt(int nt, int sides, const cudaLaunchConfig_t &config, const TrellisParams &p) {
  switch (nt) {
    case 1: return launch_sides<K2, 1>(sides, config, p);
    case 2: return launch_sides<K2, 2>(sides, config, p);
    case 4: return launch_sides<K2, 4>(sides, config, p);
    default: return launch_sides<K2, 8>(sides, config, p);
  }
}

cudaError_t launch_k2(uint32_t k2, int nt, int sides, const cudaLaunchConfig_t &config, const TrellisParams &p) {
  switch (k2) {
    case 0: return launch_nt<0>(nt, sides, config, p);
    case 4: return launch_nt<4>(nt, sides, config, p);
    case 5: return launch_nt<5>(nt, sides, config, p);
    case 6: return launch_nt<6>(nt, sides, config, p);
    case 8: return launch_nt<8>(nt, sides, config, p);
    case 10: return launch_nt<10>(nt, sides, config, p);
    default: return launch_nt<12>(nt, sides, config, p);
  }
}

template <int K2, int NT, int SIDES>
cudaError_t set_linear_attr() {
  cudaError_t err = cudaFuncSetAttribute(trellis_linear_kernel<K2, NT, SIDES, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kLinearMaxSmem));
  if (err == cudaSuccess && SIDES == 1) {
    err = cudaFuncSetAttribute(trellis_linear_kernel<K2, NT, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kLinearMaxSmem));
  }
  return err;
}

template <int K2>
cudaError_t set_linear_attrs() {
  cudaError_t err = set_linear_attr<K2, 1, 1>();
  if (err == cudaSuccess) err = set_linear_attr<K2, 1, 2>();
  if (err == cudaSuccess) err = set_linear_attr<K2, 2, 1>();
  if (err == cudaSuccess) err = set_linear_attr<K2, 2, 2>();
  if (err == cudaSuccess) err = set_linear_attr<K2, 4, 1>();
  if (err == cudaSuccess) err = set_linear_attr<K2, 4, 2>();
  if (err == cudaSuccess) err = set_linear_attr<K2, 8, 1>();
  if (err == cudaSuccess) err = set_linear_attr<K2, 8, 2>();
  return err;
}

cudaError_t set_all_linear_attrs() {
  cudaError_t err = set_linear_attrs<0>();
  if (err == cudaSuccess) err = set_linear_attrs<4>();
  if (err == cudaSuccess) err = set_linear_attrs<5>();
  if (err == cudaSuccess) err = set_linear_attrs<6>();
  if (err == cudaSuccess) err = set_linear_attrs<8>();
  if (err == cudaSuccess) err = set_linear_attrs<10>();
  if (err == cudaSuccess) err = set_linear_attrs<12>();
  return err;
}

// `count` weights over one x (count > 1: a grouped call, no SwiGLU), or the gate/up pair of a
// SwiGLU call (`up` non-NULL, count 1).
int32_t run_linear(ErrorSlot &slot, const ignis_trellis_weight *const *w, uint32_t count, const ignis_trellis_weight *up,
                   const void *x, uint32_t tokens, void *const *y, const uint32_t *ldy, uint32_t epilogue, void *stream,
                   const char *what, const ignis_trellis_workspace *workspace = nullptr) {
  if (w == nullptr || y == nullptr || ldy == nullptr) return fail(slot, "%s: NULL argument array", what);
  if (count == 0 || count > kMaxGroup) return fail(slot, "%s: count = %u is outside 1..%u", what, count, kMaxGroup);
  const bool swiglu = epilogue == kEpiSwiglu;
  if (epilogue > kEpiSwiglu) return fail(slot, "%s: unknown epilogue %u", what, epilogue);
  for (uint32_t i = 0; i < count; ++i) {
    if (check_weight(slot, w[i], what) != 0) return -1;
    if (w[i]->in != w[0]->in) return fail(slot, "%s: the weights of a group must share `in`", what);
    if (y[i] == nullptr || !aligned(y[i], 8)) return fail(slot, "%s: y is NULL or not 8-byte aligned", what);
    if ((ldy[i] % 4u) != 0 || ldy[i] < w[i]->out) return fail(slot, "%s: ldy = %u must be a multiple of 4 and at least out", what, ldy[i]);
  }
  if (swiglu) {
    if (check_weight(slot, up, what) != 0) return -1;
    if (w[0]->in != up->in || w[0]->out != up->out) return fail(slot, "%s: gate and up must share (in, out)", what);
  }
  if (tokens == 0) return fail(slot, "%s: tokens must be positive", what);
  if (x == nullptr || !aligned(x, 16)) return fail(slot, "%s: x is NULL or not 16-byte aligned", what);
  const DeviceState *dev = prepared(slot, what);
  if (dev == nullptr) return -1;
  const int sides = swiglu ? 2 : 1;
  const uint32_t in = w[0]->in;
  // beyond one pass of 64 tokens, with a workspace for the rotated rows: the tensor-core route
  if (count == 1 && trellis_tc_takes(*dev, in, tokens, static_cast<uint32_t>(sides), workspace)) {
    return trellis_tc_linear(slot, *dev, w[0], swiglu ? up : nullptr, x, tokens, y[0], ldy[0], epilogue, workspace,
                             static_cast<cudaStream_t>(stream), what);
  }
  uint32_t out_total = 0, k2 = w[0]->k2;
  for (uint32_t i = 0; i < count; ++i) {
    out_total += w[i]->out;
    if (w[i]->k2 != k2) k2 = 0u;  // 0: every weight decodes with its own width
  }
  if (swiglu && up->k2 != k2) k2 = 0u;
  TrellisParams p = {};
  p.count = count;
  p.in = in;
  p.epilogue = epilogue;
  if (swiglu) p.up = make_side(up);
  // passes of up to 64 tokens (IGNIS_TRELLIS_DECODE_MAX_TOKENS): every decoded tile serves the
  // pass's token tiles of 8
  for (uint32_t t0 = 0; t0 < tokens; t0 += IGNIS_TRELLIS_DECODE_MAX_TOKENS) {
    p.tokens = tokens - t0 < IGNIS_TRELLIS_DECODE_MAX_TOKENS ? tokens - t0 : IGNIS_TRELLIS_DECODE_MAX_TOKENS;
    const int nt = p.tokens <= 8 ? 1 : (p.tokens <= 16 ? 2 : (p.tokens <= 32 ? 4 : 8));
    const uint32_t kc = plan_kc(*dev, in, out_total, nt, sides);
    const uint32_t slice = (in / 128u + kc - 1) / kc;
    const uint32_t cap = chunk_cap(nt, sides);
    p.kc = kc;
    p.chunk = slice < cap ? slice : cap;
    p.x = static_cast<const uint16_t *>(x) + static_cast<size_t>(t0) * in;
    uint32_t ctas = 0;
    for (uint32_t i = 0; i < count; ++i) {
      p.target[i].side = make_side(w[i]);
      p.target[i].y = static_cast<uint16_t *>(y[i]) + static_cast<size_t>(t0) * ldy[i];
      p.target[i].ldy = ldy[i];
      p.target[i].cta_begin = ctas;
      ctas += (w[i]->out / 128u) * kc;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(ctas, 1, 1);
    config.blockDim = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = linear_smem_bytes(p.chunk, nt, sides);
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
    const cudaError_t err = launch_k2(k2, nt, sides, config, p);
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

namespace b200q {
int32_t prepare_trellis_kernels(ErrorSlot &slot) {
  const cudaError_t err = set_all_linear_attrs();
  if (err != cudaSuccess) return fail(slot, "ignis_trellis_prepare: %s", cudaGetErrorString(err));
  return trellis_tc_prepare(slot);
}
}  // namespace b200q

using namespace b200q;

extern "C" {

int32_t ignis_trellis_prepare(void) { return prepare_all(trellis_error()); }

uint32_t ignis_trellis_sm_cap(void) {
  const DeviceState *dev = device_state(trellis_error());
  return dev != nullptr && dev->prepared ? static_cast<uint32_t>(dev->sm_cap) : 0u;
}

uint64_t ignis_trellis_workspace_bytes(uint32_t in, uint32_t out, uint32_t weights, uint32_t tokens) {
  const DeviceState *dev = device_state(trellis_error());
  if (dev == nullptr || !dev->prepared) return 0;
  if (in == 0 || (in % 128u) != 0 || out == 0 || (out % 128u) != 0 || out > IGNIS_TRELLIS_MAX_OUT) return 0;
  if (weights < 1 || weights > 2 || tokens == 0) return 0;
  // Up to 64 tokens partial sums meet in distributed shared memory: one aligned line, never read.
  // Beyond, the tensor-core route keeps the rotated activations (fp16 rows and a scale per token) here.
  if (tokens > IGNIS_TRELLIS_DECODE_MAX_TOKENS) return trellis_tc_workspace_bytes(in, weights, tokens);
  return 256;
}

int32_t ignis_trellis_workspace_init(const ignis_trellis_workspace *workspace, void *stream) {
  ErrorSlot &slot = trellis_error();
  if (workspace == nullptr || workspace->base == nullptr) return fail(slot, "ignis_trellis_workspace_init: workspace is NULL");
  if (!aligned(workspace->base, 256)) return fail(slot, "ignis_trellis_workspace_init: base is not 256-byte aligned");
  if (prepared(slot, "ignis_trellis_workspace_init") == nullptr) return -1;
  // only the first line carries state; the rest is rewritten by every call that reads it
  const cudaError_t err = cudaMemsetAsync(workspace->base, 0, workspace->bytes < 256u ? workspace->bytes : 256u, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(slot, "ignis_trellis_workspace_init: %s", cudaGetErrorString(err));
  return 0;
}

int32_t ignis_trellis_linear(const ignis_trellis_weight *w, const void *x, uint32_t tokens, void *y, uint32_t ldy,
                             uint32_t epilogue, const ignis_trellis_workspace *workspace, void *stream) {
  if (epilogue != IGNIS_TRELLIS_STORE && epilogue != IGNIS_TRELLIS_ADD) {
    return fail(trellis_error(), "ignis_trellis_linear: unknown epilogue %u", epilogue);
  }
  const ignis_trellis_weight *ws[1] = {w};
  void *ys[1] = {y};
  const uint32_t lds[1] = {ldy};
  return run_linear(trellis_error(), ws, 1, nullptr, x, tokens, ys, lds, epilogue, stream, "ignis_trellis_linear", workspace);
}

int32_t b200q_trellis_linear_group(const ignis_trellis_weight *const *w, uint32_t count, const void *x, uint32_t tokens,
                                   void *const *y, const uint32_t *ldy, uint32_t epilogue, void *stream) {
  if (epilogue != IGNIS_TRELLIS_STORE && epilogue != IGNIS_TRELLIS_ADD) {
    return fail(trellis_error(), "b200q_trellis_linear_group: unknown epilogue %u", epilogue);
  }
  return run_linear(trellis_error(), w, count, nullptr, x, tokens, y, ldy, epilogue, stream, "b200q_trellis_linear_group");
}

int32_t ignis_trellis_linear_swiglu(const ignis_trellis_weight *gate, const ignis_trellis_weight *up, const void *x,
                                    uint32_t tokens, void *h, uint32_t ldh, const ignis_trellis_workspace *workspace,
                                    void *stream) {
  const ignis_trellis_weight *ws[1] = {gate};
  void *ys[1] = {h};
  const uint32_t lds[1] = {ldh};
  return run_linear(trellis_error(), ws, 1, up, x, tokens, ys, lds, kEpiSwiglu, stream, "ignis_trellis_linear_swiglu", workspace);
}

int32_t ignis_trellis_reconstruct(const ignis_trellis_weight *w, void *w_f16, void *stream) {
  ErrorSlot &slot = trellis_error();
  if (w == nullptr) return fail(slot, "ignis_trellis_reconstruct: weight is NULL");
  return trellis_reconstruct_raw(slot, "ignis_trellis_reconstruct", w->trellis, w->k2, w->in, w->out, w->tile_stride, w_f16,
                                 stream);
}

int32_t b200q_trellis_device_status(void *stream, uint32_t *status) {
  ErrorSlot &slot = trellis_error();
  if (status == nullptr) return fail(slot, "b200q_trellis_device_status: status is NULL");
  return trellis_tc_status(slot, static_cast<cudaStream_t>(stream), status);
}

const char *ignis_trellis_last_error(void) { return trellis_error().text; }

}  // extern "C"
