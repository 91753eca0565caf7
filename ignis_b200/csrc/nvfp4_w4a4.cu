// NVFP4 prefill route (W4A4): out[t][r] = bf16(alpha * sum_k E2M1(a) E4M3(sa) E2M1(w) E4M3(sw)),
// alpha = 1 / (d_in d_w), on the 5th-generation tensor cores.
//
// Stands where the reference quantizes activations and runs its FP4 GEMMs
// (kernel/vendor/src/ops/linear/nvfp4/nvfp4_w4a4_mma.cuh:203-436, nvfp4_w4a4_tma.cuh:264-508,
// launch_problem nvfp4_w4a4.cu:74-110) - warp-level mma.sync on its RTX target. Here:
//
//  1. `quantize_swizzled_kernel` turns the BF16 activations into E2M1 codes [T_pad][K/2] and E4M3
//     scales, bit for bit the reference's rule (nvfp4_codec.cuh:81-110), the scales written in the
//     same 512-byte (128 rows x 4 groups) tiles the weight plane uses - which is the scale-factor
//     atom the block-scaled MMA reads, so neither operand's scales are ever reshuffled.
//  2. The product, in two forms that share the stage layout and the epilogue:
//     `w4a4_gemm_persistent_kernel` - one CTA per SM walking 128-token x 256-row tiles: a producer
//     thread streams K in stages of 256 (TMA 2-D tiles of codes with the 128-byte swizzle, bulk
//     copies of the scale tiles) into an mbarrier ring that keeps running across tile boundaries;
//     two threads copy each stage's scale atoms to tensor memory (tcgen05.cp); one thread issues
//     tcgen05.mma kind::mxf4nvf4 block_scale scale_vec::4X (M 128, N 256, K 64) with the fp32
//     accumulator in tensor memory; four warps pull the accumulator (tcgen05.ld), hand tensor
//     memory back and store under the next tile's MMAs. Kept behind B200Q_W4A4_PAIR = 0.
//     `w4a4_gemm_pair_kernel` (the default) - the same on clusters of two CTAs sharing 256 x 256
//     tiles (cta_group::2): fewer operand bytes per FLOP.
//
// Every wait on an mbarrier is bounded: after the limit the thread records a status bit in the
// workspace, stops issuing and the CTA tears down (tensor memory freed) instead of hanging.
#include "../../include/b200q_nvfp4.h"

#include "nvfp4_internal.cuh"
#include "nvfp4_tc.cuh"

#include <cmath>
#include <mutex>

namespace b200q {
namespace {

constexpr int kBM = 128;          // tokens per tile (MMA M)
constexpr int kBKBytes = 128;     // bytes of codes per row per stage: 256 values along K
constexpr uint32_t kABytes = kBM * kBKBytes;        // 16 KB
constexpr uint32_t kSfaBytes = 4 * 512;             // 4 K-atoms of one 128-row tile

// Two tile shapes. 128 x 256 (one CTA per SM, 4 stages, all 512 tensor-memory columns) is the
// fused-SwiGLU form: 128 gate rows and their 128 up rows side by side. 128 x 128 (3 stages, 256
// columns) lets two CTAs share an SM, so one's pipeline fill and accumulator drain hide under the
// other's MMAs: the plain product.
template <int BN>
struct Tile {
  static constexpr int kStages = BN == 256 ? 4 : 3;
  static constexpr uint32_t kBBytes = BN * kBKBytes;
  static constexpr uint32_t kSfbBytes = (BN / 128) * 4 * 512;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + 256 + 1024;  // + barriers + alignment slack
  static constexpr uint32_t kTmemCols = BN == 256 ? 512 : 256;
  static constexpr uint32_t kSfColsPerStage = 16 + (BN / 128) * 16;  // activations, then weights
};

constexpr uint32_t kStatusProducerTimeout = 1u, kStatusMmaTimeout = 2u, kStatusEpilogueTimeout = 4u;

// ---- activation quantizer, scales in tile order -------------------------------------------------
// One thread per (token row of the padded range, 32 values): two blocks of 16, i.e. 64 bytes in,
// 16 bytes of codes and two of the four scale bytes that lie side by side in a scale tile out. The
// kernel is bound by instruction issue as much as by memory (about 13 instructions per value), so a
// thread is kept small: 48 registers, five CTAs an SM, their load and arithmetic phases interleaved
// (four blocks a thread at 65 registers and three CTAs: 2.6 % slower on the configs[2] step).
// Rows at and beyond `tokens` get zero codes and zero scales.
__global__ void __launch_bounds__(256, 5) quantize_swizzled_kernel(const uint16_t *x, uint32_t tokens, uint32_t tokens_pad,
                                                                   uint32_t k, float d_in, uint8_t *codes, uint8_t *scales) {
  griddep_launch_dependents();
  griddep_wait();
  const uint32_t halves = k / 32u, quads = k / 64u;
  const uint64_t total = static_cast<uint64_t>(tokens_pad) * halves;
  for (uint64_t hi = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; hi < total;
       hi += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
    const uint32_t t = static_cast<uint32_t>(hi / halves), h = static_cast<uint32_t>(hi % halves);
    uint2 c[2];
    uint32_t sw = 0;
    if (t < tokens) {
      const uint16_t *src = x + static_cast<uint64_t>(t) * k + h * 32u;
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = ldg128_coherent(src + 8 * j);
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        uint8_t s;
        quantize_block16(v[2 * b], v[2 * b + 1], d_in, c[b], s);
        sw |= static_cast<uint32_t>(s) << (8 * b);
      }
    } else {
#pragma unroll
      for (int b = 0; b < 2; ++b) c[b] = make_uint2(0u, 0u);
    }
    *reinterpret_cast<uint4 *>(codes + hi * 16u) = make_uint4(c[0].x, c[0].y, c[1].x, c[1].y);
    const uint32_t q = h >> 1;
    const uint64_t so = (static_cast<uint64_t>(t >> 7) * quads + q) * 512u + (t & 31u) * 16u + ((t & 127u) >> 5) * 4u + (h & 1u) * 2u;
    *reinterpret_cast<uint16_t *>(scales + so) = static_cast<uint16_t>(sw);
  }
}

struct W4A4Params {
  const uint8_t *sfa;   // activation scales, tile order
  const uint8_t *sfb;   // weight scales, tile order
  void *y;
  uint32_t *status;
  uint32_t tokens, n, k, ldy;
  float alpha;
  uint32_t epilogue;  // STORE / ADD / OUT_F32, or the fused SwiGLU (the tile's columns 0..127 are gate rows, 128..255 the up rows)
  uint8_t *q_codes;   // kEpilogueQuant: h as the next product's operand, codes [pad tokens][n / 4] ...
  uint8_t *q_scales;  // ... and scales in 512-byte tiles
  float q_din;        // the next weight's input divisor
};

// ---- the persistent form ------------------------------------------------------------------------
// One CTA per SM walks 128 x 256 tiles (tile = blockIdx.x, + gridDim.x, ...; the token tile index
// runs fastest, so the CTAs at work share weight rows in the L2). The producer keeps the 4-stage ring
// full across tile boundaries, so a tile's first MMAs find their operands waiting; the epilogue
// warps pull the whole accumulator into registers (as packed BF16: 128 registers a thread - the
// CTA has the SM's register file to itself), hand tensor memory back to the MMA thread and only
// then store, under the next tile's MMAs. What a tile costs beyond its MMAs is the pull alone.
// ---- the persistent kernels' epilogue for one 128-token x 256-row tile ---------------------------
// The calling warp q owns accumulator lanes (tokens) 32 q .. 32 q + 31 at `lane_base`. `release()`
// hands tensor memory back to the MMA thread; it is called as soon as the accumulator has been
// read, so that whatever follows runs under the next tile's MMAs.
template <class Release>
__device__ __forceinline__ void w4a4_epilogue_tile(const W4A4Params &p, uint32_t lane_base, int warp, int lane, uint32_t m_tile,
                                                   uint32_t n_tile, bool swiglu, Release release) {
  constexpr int kBN = 256;
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t token = m_tile * kBM + warp * 32 + lane;
  if (p.epilogue & (kEpilogueF32 | kEpilogueAdd)) {
    // float32 rows do not fit the register file, and a residual has to be read before the one
    // rounding: these forms store chunk by chunk, then release
#pragma unroll 1
    for (uint32_t c = 0; c < kBN; c += 32) {
      uint32_t r[32];
      tmem_ld32(lane_base + c, r);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const uint32_t row0 = n_tile * kBN + c;
      if (token < p.tokens && row0 < p.n) {
        const bool add = (p.epilogue & kEpilogueAdd) != 0u;
        if (p.epilogue & kEpilogueF32) {
          float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(p.y) + static_cast<size_t>(token) * p.ldy + row0);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 o = make_float4(__uint_as_float(r[4 * j]) * p.alpha, __uint_as_float(r[4 * j + 1]) * p.alpha,
                                   __uint_as_float(r[4 * j + 2]) * p.alpha, __uint_as_float(r[4 * j + 3]) * p.alpha);
            if (add) {
              const float4 old = dst[j];
              o.x += old.x, o.y += old.y, o.z += old.z, o.w += old.w;
            }
            dst[j] = o;
          }
        } else {
          uint4 *dst = reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(p.y) + static_cast<size_t>(token) * p.ldy + row0);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 old = dst[j];
            const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(
                  __uint_as_float(r[8 * j + 2 * e]) * p.alpha + bf16_bits_to_f32(ow[e] & 0xFFFFu),
                  __uint_as_float(r[8 * j + 2 * e + 1]) * p.alpha + __uint_as_float(ow[e] & 0xFFFF0000u));
              o[e] = *reinterpret_cast<const uint32_t *>(&h);
            }
            dst[j] = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    release();
    return;
  }
  // The thread's row as packed BF16: 256 columns of the product, or (SwiGLU) BF16(g alpha) in
  // [0, 64) and BF16(u alpha) in [64, 128) - the two roundings the reference's formula makes first.
  uint32_t out[128];
#pragma unroll
  for (uint32_t c = 0; c < kBN; c += 32) {
    uint32_t r[32];
    tmem_ld32(lane_base + c, r);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * j]) * p.alpha, __uint_as_float(r[2 * j + 1]) * p.alpha);
      out[c / 2 + j] = *reinterpret_cast<const uint32_t *>(&h);
    }
  }
  // tensor memory is free for the next tile's MMAs; the rest runs under them
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncwarp();
  release();
  if (swiglu) {
    // h = BF16(silu(BF16(g)) * BF16(u)), in place over the gate half
#pragma unroll
    for (int j = 0; j < 64; ++j) {
      const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&out[j]));
      const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&out[64 + j]));
      const __nv_bfloat162 h = __floats2bfloat162_rn(g.x / (1.0f + __expf(-g.x)) * u.x, g.y / (1.0f + __expf(-g.y)) * u.y);
      out[j] = *reinterpret_cast<const uint32_t *>(&h);
    }
  }
  if (swiglu && (p.epilogue & kEpilogueQuant)) {
    // h leaves as the down product's operand: 8 blocks of 16 along its K, quantized as the
    // standalone quantizer would from the BF16 values (padding rows are zeros and stay zeros)
    const uint32_t inter = p.n / 2u, g0 = n_tile * 8u;
    uint32_t sc[2] = {0u, 0u};
    uint4 *code_dst = reinterpret_cast<uint4 *>(p.q_codes + static_cast<uint64_t>(token) * (inter / 2u) + n_tile * 64u);
#pragma unroll
    for (int b = 0; b < 8; b += 2) {
      uint2 c0, c1;
      uint8_t s0, s1;
      quantize_block16(make_uint4(out[8 * b], out[8 * b + 1], out[8 * b + 2], out[8 * b + 3]),
                       make_uint4(out[8 * b + 4], out[8 * b + 5], out[8 * b + 6], out[8 * b + 7]), p.q_din, c0, s0);
      quantize_block16(make_uint4(out[8 * b + 8], out[8 * b + 9], out[8 * b + 10], out[8 * b + 11]),
                       make_uint4(out[8 * b + 12], out[8 * b + 13], out[8 * b + 14], out[8 * b + 15]), p.q_din, c1, s1);
      code_dst[b / 2] = make_uint4(c0.x, c0.y, c1.x, c1.y);
      sc[b >> 2] |= (static_cast<uint32_t>(s0) << (8 * (b & 3))) | (static_cast<uint32_t>(s1) << (8 * ((b + 1) & 3)));
    }
    const uint64_t atom = (static_cast<uint64_t>(token >> 7) * (inter / 64u) + (g0 >> 2)) * 512u + (token & 31u) * 16u +
                          ((token & 127u) >> 5) * 4u;
    *reinterpret_cast<uint32_t *>(p.q_scales + atom) = sc[0];
    *reinterpret_cast<uint32_t *>(p.q_scales + atom + 512u) = sc[1];
    return;
  }
  if (token < p.tokens) {
    const uint32_t width = swiglu ? 128u : kBN;
    const uint32_t col0 = n_tile * width;
    const uint32_t limit = swiglu ? p.n / 2u : p.n;
    __nv_bfloat16 *row = static_cast<__nv_bfloat16 *>(p.y) + static_cast<size_t>(token) * p.ldy + col0;
#pragma unroll
    for (uint32_t c = 0; c < kBN; c += 8) {
      if (c < width && col0 + c < limit) {  // n is a multiple of 128: an 8-column piece is whole
        *reinterpret_cast<uint4 *>(row + c) = make_uint4(out[c / 2], out[c / 2 + 1], out[c / 2 + 2], out[c / 2 + 3]);
      }
    }
  }
}

__global__ void __launch_bounds__(256, 1) w4a4_gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                     const __grid_constant__ CUtensorMap map_b,
                                                                     const __grid_constant__ W4A4Params p) {
  constexpr int kBN = 256;
  constexpr int kStages = Tile<256>::kStages;
  constexpr uint32_t kBBytes = Tile<256>::kBBytes, kStageBytes = Tile<256>::kStageBytes;
  constexpr uint32_t kTmemCols = Tile<256>::kTmemCols, kSfColsPerStage = Tile<256>::kSfColsPerStage;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw);
  // barriers: full[4], empty[4], accumulator full, accumulator empty; then the tensor-memory slot
  const uint32_t bars = base + kStages * kStageBytes;
  const uint32_t bar_acc_full = bars + 8 * 2 * kStages, bar_acc_empty = bar_acc_full + 8;
  const uint32_t bar_sf_ready = bar_acc_empty + 8;   // [4]: a stage's scales are in tensor memory
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + kStages * kStageBytes + 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t k_iters = p.k / 256u, k_atoms = p.k / 64u;
  const bool swiglu = (p.epilogue & kEpilogueSwiglu) != 0u;
  const uint32_t m_tiles = (p.tokens + kBM - 1) / kBM;
  const uint32_t n_tiles = swiglu ? p.n / 256u : (p.n + 255u) / 256u;
  const uint32_t tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bars + 8 * s, 1);
      mbar_init(bars + 8 * (kStages + s), 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, 4);  // one arrival per epilogue warp
    for (int s = 0; s < kStages; ++s) mbar_init(bar_sf_ready + 8 * s, 2);  // the two scale copiers' commits
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  griddep_launch_dependents();
  griddep_wait();  // the quantized activations come from the previous kernel in the stream

  if (warp == 4 && lane == 0) {
    // ---- producer ----
    uint32_t git = 0;  // stage uses since the kernel began
    bool ok = true;
    for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      const uint32_t m_tile = tile % m_tiles, n_tile = tile / m_tiles;
      const uint32_t row_a = swiglu ? n_tile * 128u : n_tile * kBN;
      const uint32_t row_b = swiglu ? p.n / 2u + n_tile * 128u : n_tile * kBN + 128u;
      const bool second_half = row_b < p.n;
      for (uint32_t it = 0; it < k_iters; ++it, ++git) {
        const uint32_t s = git % kStages;
        if (!mbar_wait(bars + 8 * (kStages + s), ((git / kStages) & 1u) ^ 1u)) {
          atomicOr(p.status, kStatusProducerTimeout);
          ok = false;
          break;
        }
        const uint32_t full = bars + 8 * s;
        const uint32_t stage = base + s * kStageBytes;
        mbar_expect_tx(full, kABytes + kSfaBytes + (second_half ? 2u : 1u) * (128u * kBKBytes + 2048u));
        tma_load_2d(stage, &map_a, full, static_cast<int32_t>(it * kBKBytes), static_cast<int32_t>(m_tile * kBM));
        tma_load_2d(stage + kABytes, &map_b, full, static_cast<int32_t>(it * kBKBytes), static_cast<int32_t>(row_a));
        if (second_half) {
          tma_load_2d(stage + kABytes + 128u * kBKBytes, &map_b, full, static_cast<int32_t>(it * kBKBytes), static_cast<int32_t>(row_b));
        }
        bulk_load(stage + kABytes + kBBytes, p.sfa + (static_cast<uint64_t>(m_tile) * k_atoms + it * 4u) * 512u, kSfaBytes, full);
        bulk_load(stage + kABytes + kBBytes + kSfaBytes, p.sfb + (static_cast<uint64_t>(row_a / 128u) * k_atoms + it * 4u) * 512u, 2048u, full);
        if (second_half) {
          bulk_load(stage + kABytes + kBBytes + kSfaBytes + 2048u, p.sfb + (static_cast<uint64_t>(row_b / 128u) * k_atoms + it * 4u) * 512u,
                    2048u, full);
        }
      }
    }
  } else if (warp == 5 && lane == 0) {
    // ---- MMA issuer ----
    // The scale copies of a stage (twelve of 512 bytes) cost this thread more issue time than its four
    // MMAs when it issues both (880 cycles a stage, measured with clock64), so they come from the
    // two copier warps below and this thread only waits for their commits.
    const uint32_t idesc = (1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((kBM >> 4) << 24);
    uint32_t git = 0, tile_i = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++tile_i) {
      // the epilogue warps have pulled the previous tile out of tensor memory
      if (!mbar_wait(bar_acc_empty, (tile_i & 1u) ^ 1u)) {
        atomicOr(p.status, kStatusMmaTimeout);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (uint32_t it = 0; it < k_iters; ++it, ++git) {
        const uint32_t s = git % kStages;
        if (!mbar_wait(bar_sf_ready + 8 * s, (git / kStages) & 1u)) {   // operands landed and scales copied
          atomicOr(p.status, kStatusMmaTimeout);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t stage = base + s * kStageBytes;
        const uint32_t sf_cols = tmem + kBN + s * kSfColsPerStage;
        const uint64_t a_desc = smem_desc(stage, 1024u, 2u);
        const uint64_t b_desc = smem_desc(stage + kABytes, 1024u, 2u);
#pragma unroll
        for (uint32_t kb = 0; kb < 4; ++kb) {
          mma_mxf4nvf4(tmem, a_desc + 2u * kb, b_desc + 2u * kb, idesc, sf_cols + kb * 4u, sf_cols + 16u + kb * 8u,
                       (it | kb) != 0u ? 1u : 0u);
        }
        mma_commit(bars + 8 * (kStages + s));
      }
      if (ok) mma_commit(bar_acc_full);
    }
  } else if (warp >= 6 && lane == 0) {
    // ---- scale copiers: a stage's scale tiles go to tensor memory from threads of their own,
    //      warp 6 the first two K-atoms, warp 7 the other two ----
    const uint32_t kb0 = static_cast<uint32_t>(warp - 6) * 2u;
    const uint32_t my_tiles = tiles > blockIdx.x ? (tiles - blockIdx.x + gridDim.x - 1u) / gridDim.x : 0u;
    const uint32_t total = my_tiles * k_iters;
    for (uint32_t g = 0; g < total; ++g) {
      const uint32_t s = g % kStages;
      if (!mbar_wait(bars + 8 * s, (g / kStages) & 1u)) {
        atomicOr(p.status, kStatusMmaTimeout);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t stage = base + s * kStageBytes;
      const uint32_t sf_cols = tmem + kBN + s * kSfColsPerStage;
      const uint32_t sfa_smem = stage + kABytes + kBBytes, sfb_smem = sfa_smem + kSfaBytes;
#pragma unroll
      for (uint32_t kb = kb0; kb < kb0 + 2u; ++kb) {
        tmem_cp_sf(sf_cols + kb * 4u, smem_desc(sfa_smem + kb * 512u, 128u, 0u));
        tmem_cp_sf(sf_cols + 16u + kb * 8u, smem_desc(sfb_smem + kb * 512u, 128u, 0u));
        tmem_cp_sf(sf_cols + 16u + kb * 8u + 4u, smem_desc(sfb_smem + 2048u + kb * 512u, 128u, 0u));
      }
      mma_commit(bar_sf_ready + 8 * s);
    }
  } else if (warp < 4) {
    // ---- epilogue: warp q owns accumulator lanes (tokens) 32 q .. 32 q + 31 ----
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    uint32_t tile_i = 0;
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++tile_i) {
      const uint32_t m_tile = tile % m_tiles, n_tile = tile / m_tiles;
      if (!mbar_wait(bar_acc_full, tile_i & 1u)) {
        if (lane == 0) atomicOr(p.status, kStatusEpilogueTimeout);
        break;
      }
      w4a4_epilogue_tile(p, lane_base, warp, lane, m_tile, n_tile, swiglu, [&] {
        if (lane == 0) mbar_arrive(bar_acc_empty);
      });
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- the persistent form on CTA pairs ------------------------------------------------------------
// Two CTAs of a cluster share a 256-token x 256-row tile (tcgen05 cta_group::2): each CTA holds its
// 128 tokens' codes and accumulator rows, and only half of the weight rows - the tensor cores read
// the other half from the peer's shared memory - so a CTA brings 38 KB per K stage where the
// single-CTA form brings 54 KB for the same FLOPs, and five stages fit where four did. Every load
// of both CTAs reports to the barrier of the pair's first CTA, whose MMA thread issues for both;
// its commits arrive at both CTAs' barriers (two plain commits, one per CTA). The scale tiles
// travel as TMA tiles too (a bulk copy cannot report to the peer's barrier): the scale planes as
// [tile][128] words.
constexpr int kPairStages = 5;
constexpr uint32_t kPairBBytes = 128 * kBKBytes;                                   // this CTA's half of the weight rows
constexpr uint32_t kPairStageBytes = kABytes + kPairBBytes + kSfaBytes + 2 * 2048;  // + token scales + both halves' weight scales
constexpr uint32_t kPairSmemBytes = kPairStages * kPairStageBytes + 256 + 1024;
constexpr uint32_t kPairSfCols = 48;  // per stage: 16 columns of token scales, 32 of weight scales
// The shared::cluster address of this CTA's `addr` in the cluster's CTA `rank`.
__device__ __forceinline__ uint32_t in_cta(uint32_t addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  return remote;
}

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void mma_mxf4nvf4_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                                  uint32_t accumulate) {
  asm volatile("{ .reg .pred p; setp.ne.u32 p, %6, 0;\n"
               "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p; }"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
               : "memory");
}
// Arrives at `bar` (a shared::cluster address: this CTA's or the peer's) once the pair's MMAs so far have retired.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__global__ void __launch_bounds__(256, 1) w4a4_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_b,
                                                               const __grid_constant__ CUtensorMap map_sfa,
                                                               const __grid_constant__ CUtensorMap map_sfb,
                                                               const __grid_constant__ W4A4Params p) {
  constexpr int kBN = 256;
  constexpr int kStages = kPairStages;
  constexpr uint32_t kTmemCols = 512;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;   // the same offset in both CTAs: they run the same kernel
  uint8_t *base_ptr = smem_raw + (base - raw);
  // barriers: full[5], empty[5], accumulator full, accumulator empty; then the tensor-memory slot
  const uint32_t bars = base + kStages * kPairStageBytes;
  const uint32_t bar_acc_full = bars + 8 * 2 * kStages, bar_acc_empty = bar_acc_full + 8;
  const uint32_t bar_sf_ready = bar_acc_empty + 8;   // [5], the first CTA's: a stage's scales are in both CTAs' tensor memory
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + kStages * kPairStageBytes + 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0: the pair's first CTA, which issues the MMAs
  const uint32_t k_iters = p.k / 256u, k_atoms = p.k / 64u;
  const bool swiglu = (p.epilogue & kEpilogueSwiglu) != 0u;
  const uint32_t m_tiles = (p.tokens + kBM - 1) / kBM, m_pairs = (m_tiles + 1u) / 2u;
  const uint32_t n_tiles = swiglu ? p.n / 256u : (p.n + 255u) / 256u;
  const uint32_t tiles = m_pairs * n_tiles;
  const uint32_t first = blockIdx.x / 2u, step = gridDim.x / 2u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bars + 8 * s, 1);               // the first CTA's: its producer's expect_tx arrival (the bytes of both CTAs)
      mbar_init(bars + 8 * (kStages + s), 1);   // one commit
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, 8);                // the first CTA's: one arrival per epilogue warp of the pair
    for (int s = 0; s < kStages; ++s) mbar_init(bar_sf_ready + 8 * s, 2);   // the two scale copiers' commits
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything is sent to them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  griddep_launch_dependents();
  griddep_wait();  // the quantized activations come from the previous kernel in the stream

  if (warp == 4 && lane == 0) {
    // ---- producer (both CTAs): own tokens, own half of the weight rows, the scales of both halves ----
    uint32_t git = 0;
    bool ok = true;
    for (uint32_t tile = first; tile < tiles && ok; tile += step) {
      const uint32_t m_tile = 2u * (tile % m_pairs) + rank, n_tile = tile / m_pairs;
      const uint32_t row_a = swiglu ? n_tile * 128u : n_tile * kBN;
      const uint32_t row_b = swiglu ? p.n / 2u + n_tile * 128u : n_tile * kBN + 128u;
      for (uint32_t it = 0; it < k_iters; ++it, ++git) {
        const uint32_t s = git % kStages;
        if (!mbar_wait(bars + 8 * (kStages + s), ((git / kStages) & 1u) ^ 1u)) {
          atomicOr(p.status, kStatusProducerTimeout);
          ok = false;
          break;
        }
        const uint32_t full = in_cta(bars + 8 * s, 0u);   // the first CTA's barrier collects both CTAs' bytes
        const uint32_t stage = base + s * kPairStageBytes;
        if (rank == 0u) mbar_expect_tx(bars + 8 * s, 2u * kPairStageBytes);
        tma_load_2d_pair(stage, &map_a, full, static_cast<int32_t>(it * kBKBytes), static_cast<int32_t>(m_tile * kBM));
        tma_load_2d_pair(stage + kABytes, &map_b, full, static_cast<int32_t>(it * kBKBytes), static_cast<int32_t>(rank == 0u ? row_a : row_b));
        tma_load_2d_pair(stage + kABytes + kPairBBytes, &map_sfa, full, 0, static_cast<int32_t>(m_tile * k_atoms + it * 4u));
        tma_load_2d_pair(stage + kABytes + kPairBBytes + kSfaBytes, &map_sfb, full, 0,
                         static_cast<int32_t>((row_a / 128u) * k_atoms + it * 4u));
        tma_load_2d_pair(stage + kABytes + kPairBBytes + kSfaBytes + 2048u, &map_sfb, full, 0,
                         static_cast<int32_t>((row_b / 128u) * k_atoms + it * 4u));
      }
    }
  } else if (warp == 5 && lane == 0 && rank == 0u) {
    // ---- MMA issuer of the pair: M 256 (128 per CTA), N 256, K 64 ----
    const uint32_t idesc = (1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((256u >> 4) << 24);
    uint32_t git = 0, tile_i = 0;
    bool ok = true;
    for (uint32_t tile = first; tile < tiles && ok; tile += step, ++tile_i) {
      if (!mbar_wait(bar_acc_empty, (tile_i & 1u) ^ 1u)) {   // both CTAs have pulled the previous tile out of tensor memory
        atomicOr(p.status, kStatusMmaTimeout);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (uint32_t it = 0; it < k_iters; ++it, ++git) {
        const uint32_t s = git % kStages;
        if (!mbar_wait(bar_sf_ready + 8 * s, (git / kStages) & 1u)) {   // operands landed in both CTAs and scales copied
          atomicOr(p.status, kStatusMmaTimeout);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t stage = base + s * kPairStageBytes;
        const uint32_t sf_cols = tmem + kBN + s * kPairSfCols;
        const uint64_t a_desc = smem_desc(stage, 1024u, 2u);
        const uint64_t b_desc = smem_desc(stage + kABytes, 1024u, 2u);
#pragma unroll
        for (uint32_t kb = 0; kb < 4; ++kb) {
          mma_mxf4nvf4_pair(tmem, a_desc + 2u * kb, b_desc + 2u * kb, idesc, sf_cols + kb * 4u, sf_cols + 16u + kb * 8u,
                            (it | kb) != 0u ? 1u : 0u);
        }
        mma_commit_pair(in_cta(bars + 8 * (kStages + s), 0u));   // this CTA's stage ...
        mma_commit_pair(in_cta(bars + 8 * (kStages + s), 1u));   // ... and the peer's
      }
      if (ok) {
        mma_commit_pair(in_cta(bar_acc_full, 0u));
        mma_commit_pair(in_cta(bar_acc_full, 1u));
      }
    }
  } else if (warp >= 6 && lane == 0 && rank == 0u) {
    // ---- scale copiers of the pair (one copy instruction serves both CTAs): warp 6 the first two
    //      K-atoms of a stage, warp 7 the other two ----
    const uint32_t kb0 = static_cast<uint32_t>(warp - 6) * 2u;
    const uint32_t my_tiles = tiles > first ? (tiles - first + step - 1u) / step : 0u;
    const uint32_t total = my_tiles * k_iters;
    for (uint32_t g = 0; g < total; ++g) {
      const uint32_t s = g % kStages;
      if (!mbar_wait(bars + 8 * s, (g / kStages) & 1u)) {
        atomicOr(p.status, kStatusMmaTimeout);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t stage = base + s * kPairStageBytes;
      const uint32_t sf_cols = tmem + kBN + s * kPairSfCols;
      const uint32_t sfa_smem = stage + kABytes + kPairBBytes, sfb_smem = sfa_smem + kSfaBytes;
#pragma unroll
      for (uint32_t kb = kb0; kb < kb0 + 2u; ++kb) {
        tmem_cp_sf_pair(sf_cols + kb * 4u, smem_desc(sfa_smem + kb * 512u, 128u, 0u));
        tmem_cp_sf_pair(sf_cols + 16u + kb * 8u, smem_desc(sfb_smem + kb * 512u, 128u, 0u));
        tmem_cp_sf_pair(sf_cols + 16u + kb * 8u + 4u, smem_desc(sfb_smem + 2048u + kb * 512u, 128u, 0u));
      }
      mma_commit_pair(in_cta(bar_sf_ready + 8 * s, 0u));
    }
  } else if (warp < 4) {
    // ---- epilogue (both CTAs): warp q owns this CTA's accumulator lanes (tokens) 32 q .. 32 q + 31 ----
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    const uint32_t acc_empty_first = in_cta(bar_acc_empty, 0u);
    uint32_t tile_i = 0;
    for (uint32_t tile = first; tile < tiles; tile += step, ++tile_i) {
      const uint32_t m_tile = 2u * (tile % m_pairs) + rank, n_tile = tile / m_pairs;
      if (!mbar_wait(bar_acc_full, tile_i & 1u)) {
        if (lane == 0) atomicOr(p.status, kStatusEpilogueTimeout);
        break;
      }
      if (m_tile >= m_tiles) {   // the odd pair's second CTA: nothing of this tile is its to store
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_first);
        continue;
      }
      w4a4_epilogue_tile(p, lane_base, warp, lane, m_tile, n_tile, swiglu, [&] {
        if (lane == 0) mbar_arrive_cluster(acc_empty_first);
      });
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves while the other may still reach its shared memory or barriers
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- host side --------------------------------------------------------------------------------
// A [rows][k/2]-byte plane as a 2-D byte tensor with (128 bytes x box_rows) boxes, 128-byte swizzle.
bool make_code_map(CUtensorMap *map, const void *codes, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBKBytes), box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(codes), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A scale plane of 512-byte tiles as a 2-D tensor [tiles][128 words] with boxes of four tiles (one K stage).
bool make_scale_map(CUtensorMap *map, const void *scales, uint64_t tiles) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {128, tiles};
  const cuuint64_t strides[1] = {512};
  const cuuint32_t box[2] = {128, 4};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(scales), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

uint32_t w4a4_tokens_pad(uint32_t tokens) { return (tokens + kBM - 1) / kBM * kBM; }

// Workspace of a W4A4 call: one status line, then the codes, then the scale tiles.
uint64_t w4a4_workspace_bytes(uint32_t k, uint32_t tokens) {
  const uint64_t pad = w4a4_tokens_pad(tokens);
  return 256u + pad * (k / 2u) + pad * (k / 16u);
}

bool w4a4_shape_ok(uint32_t n, uint32_t k) { return (k % 256u) == 0 && (n % 128u) == 0; }

int32_t w4a4_prepare(ErrorSlot &slot) {
  cudaError_t err = cudaFuncSetAttribute(w4a4_gemm_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(Tile<256>::kSmemBytes));
  if (err == cudaSuccess) {
    err = cudaFuncSetAttribute(w4a4_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kPairSmemBytes));
  }
  if (err != cudaSuccess) return fail(slot, "nvfp4 prefill kernel attributes: %s", cudaGetErrorString(err));
  if (encode_tiled_fn() == nullptr) return fail(slot, "cuTensorMapEncodeTiled is not available from this driver");
  return 0;
}

namespace {
struct QuantTarget {
  uint8_t *codes = nullptr;
  uint8_t *scales = nullptr;
  float d_in = 1.0f;
};

// One product over activations at `a_codes` / `a_scales`; `x` non-NULL quantizes them there first.
int32_t w4a4_product(ErrorSlot &slot, const DeviceState &dev, const uint8_t *w_codes, const uint8_t *w_scales, uint32_t n,
                     uint32_t k, float d_w, float d_in, const uint16_t *x, uint32_t tokens, void *y, uint32_t ldy,
                     uint32_t epilogue, uint32_t *status, uint8_t *a_codes, uint8_t *a_scales, const QuantTarget &q,
                     cudaStream_t stream) {
  const uint32_t pad = w4a4_tokens_pad(tokens);
  if (x != nullptr) {
    const uint64_t total = static_cast<uint64_t>(pad) * (k / 32u);
    const uint32_t grid = static_cast<uint32_t>(total / 256u < 148u * 24u ? (total + 255u) / 256u : 148u * 24u);
    const cudaError_t err = launch(quantize_swizzled_kernel, dim3(grid), dim3(256), 0, stream, dev.pdl != 0, x, tokens, pad,
                                   k, d_in, a_codes, a_scales);
    if (err != cudaSuccess) return fail(slot, "nvfp4 activation quantizer launch: %s", cudaGetErrorString(err));
  }
  CUtensorMap map_a, map_b;
  if (!make_code_map(&map_a, a_codes, pad, k / 2u, kBM) || !make_code_map(&map_b, w_codes, n, k / 2u, 128u)) {
    return fail(slot, "nvfp4 prefill: tensor map encoding failed");
  }
  W4A4Params p = {};
  p.sfa = a_scales;
  p.sfb = w_scales;
  p.y = y;
  p.status = status;
  p.tokens = tokens;
  p.n = n;
  p.k = k;
  p.ldy = ldy;
  p.alpha = 1.0f / (d_in * d_w);
  p.epilogue = epilogue;
  p.q_codes = q.codes;
  p.q_scales = q.scales;
  p.q_din = q.d_in;
  const bool swiglu = (epilogue & kEpilogueSwiglu) != 0u;
  // the fused SwiGLU needs the wide tile (gate and up boxes side by side); the plain product takes
  // the narrow one, two CTAs per SM
  if (dev.w4a4_pair != 0) {
    // CTA pairs on 256-token x 256-row tiles
    CUtensorMap map_sfa, map_sfb;
    if (!make_scale_map(&map_sfa, a_scales, static_cast<uint64_t>(pad / kBM) * (k / 64u)) ||
        !make_scale_map(&map_sfb, w_scales, static_cast<uint64_t>(n / 128u) * (k / 64u))) {
      return fail(slot, "nvfp4 prefill: tensor map encoding failed");
    }
    const uint32_t m_pairs = (pad / kBM + 1u) / 2u;
    const uint32_t tiles = m_pairs * (swiglu ? n / 256u : (n + 255u) / 256u);
    const uint32_t pairs_max = static_cast<uint32_t>(dev.sm_count) / 2u;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2u * (tiles < pairs_max ? tiles : pairs_max), 1, 1);
    config.blockDim = dim3(256, 1, 1);
    config.dynamicSmemBytes = kPairSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = dev.pdl ? 2 : 1;
    const cudaError_t perr = cudaLaunchKernelEx(&config, w4a4_gemm_pair_kernel, map_a, map_b, map_sfa, map_sfb, p);
    if (perr != cudaSuccess) return fail(slot, "nvfp4 prefill launch: %s", cudaGetErrorString(perr));
    return 0;
  }
  // B200Q_W4A4_PAIR = 0: the persistent form on single CTAs, 128-token x 256-row tiles
  const uint32_t tiles = (pad / kBM) * (swiglu ? n / 256u : (n + 255u) / 256u);
  const uint32_t ctas = tiles < static_cast<uint32_t>(dev.sm_count) ? tiles : static_cast<uint32_t>(dev.sm_count);
  const cudaError_t perr = launch(w4a4_gemm_persistent_kernel, dim3(ctas), dim3(256), Tile<256>::kSmemBytes, stream, dev.pdl != 0, map_a, map_b, p);
  if (perr != cudaSuccess) return fail(slot, "nvfp4 prefill launch: %s", cudaGetErrorString(perr));
  return 0;
}
}  // namespace

int32_t w4a4_launch(ErrorSlot &slot, const DeviceState &dev, const uint8_t *w_codes, const uint8_t *w_scales, uint32_t n,
                    uint32_t k, float d_w, float d_in, const uint16_t *x, uint32_t tokens, void *y, uint32_t ldy,
                    uint32_t epilogue, uint8_t *workspace, cudaStream_t stream) {
  const uint32_t pad = w4a4_tokens_pad(tokens);
  uint8_t *a_codes = workspace + 256;
  uint8_t *a_scales = a_codes + static_cast<uint64_t>(pad) * (k / 2u);
  return w4a4_product(slot, dev, w_codes, w_scales, n, k, d_w, d_in, x, tokens, y, ldy, epilogue,
                      reinterpret_cast<uint32_t *>(workspace), a_codes, a_scales, QuantTarget(), stream);
}

int32_t w4a4_launch_prequantized(ErrorSlot &slot, const DeviceState &dev, const uint8_t *w_codes, const uint8_t *w_scales,
                                 uint32_t n, uint32_t k, float d_w, float d_in, uint32_t tokens, void *y, uint32_t ldy,
                                 uint32_t epilogue, uint8_t *workspace, cudaStream_t stream) {
  const uint32_t pad = w4a4_tokens_pad(tokens);
  uint8_t *a_codes = workspace + 256;
  uint8_t *a_scales = a_codes + static_cast<uint64_t>(pad) * (k / 2u);
  return w4a4_product(slot, dev, w_codes, w_scales, n, k, d_w, d_in, nullptr, tokens, y, ldy, epilogue,
                      reinterpret_cast<uint32_t *>(workspace), a_codes, a_scales, QuantTarget(), stream);
}

// Quantizes tokens [token_begin, token_begin + token_count) of a call of `tokens_total` tokens into
// their place of the operand in `workspace` (token_begin a multiple of 128: whole scale tiles);
// `x_rows` points at the first of those tokens. Rows between the range's end and the next multiple
// of 128 are written as zeros.
int32_t w4a4_quantize_range(ErrorSlot &slot, const DeviceState &dev, const uint16_t *x_rows, uint32_t tokens_total,
                            uint32_t token_begin, uint32_t token_count, uint32_t k, float d_in, uint8_t *workspace,
                            cudaStream_t stream) {
  const uint64_t pad_total = w4a4_tokens_pad(tokens_total);
  const uint32_t pad = w4a4_tokens_pad(token_count);
  uint8_t *codes = workspace + 256 + static_cast<uint64_t>(token_begin) * (k / 2u);
  uint8_t *scales = workspace + 256 + pad_total * (k / 2u) + static_cast<uint64_t>(token_begin / 128u) * (k / 64u) * 512u;
  const uint64_t total = static_cast<uint64_t>(pad) * (k / 32u);
  const uint32_t grid = static_cast<uint32_t>(total / 256u < 148u * 24u ? (total + 255u) / 256u : 148u * 24u);
  const cudaError_t err = launch(quantize_swizzled_kernel, dim3(grid), dim3(256), 0, stream, dev.pdl != 0, x_rows, token_count, pad, k,
                                 d_in, codes, scales);
  if (err != cudaSuccess) return fail(slot, "nvfp4 activation quantizer launch: %s", cudaGetErrorString(err));
  return 0;
}

// Workspace of the MLP: the status line, x quantized (K = k), h quantized (K = inter).
uint64_t w4a4_mlp_workspace_bytes(uint32_t k, uint32_t inter, uint32_t tokens) {
  const uint64_t pad = w4a4_tokens_pad(tokens);
  return 256u + pad * (k / 2u) + pad * (k / 16u) + pad * (inter / 2u) + pad * (inter / 16u);
}

int32_t w4a4_mlp_launch(ErrorSlot &slot, const DeviceState &dev, const uint8_t *gu_codes, const uint8_t *gu_scales, uint32_t gu_n,
                        uint32_t k, float gu_dw, float gu_din, const uint8_t *dn_codes, const uint8_t *dn_scales, uint32_t dn_n,
                        float dn_dw, float dn_din, const uint16_t *x, uint32_t tokens, void *y, uint32_t ldy, uint32_t epilogue,
                        uint8_t *workspace, cudaStream_t stream) {
  const uint64_t pad = w4a4_tokens_pad(tokens);
  const uint32_t inter = gu_n / 2u;
  uint32_t *status = reinterpret_cast<uint32_t *>(workspace);
  uint8_t *x_codes = workspace + 256;
  uint8_t *x_scales = x_codes + pad * (k / 2u);
  QuantTarget h;
  h.codes = x_scales + pad * (k / 16u);
  h.scales = h.codes + pad * (inter / 2u);
  h.d_in = dn_din;
  if (w4a4_product(slot, dev, gu_codes, gu_scales, gu_n, k, gu_dw, gu_din, x, tokens, nullptr, 0, kEpilogueSwiglu | kEpilogueQuant,
                   status, x_codes, x_scales, h, stream) != 0) {
    return -1;
  }
  return w4a4_product(slot, dev, dn_codes, dn_scales, dn_n, inter, dn_dw, dn_din, nullptr, tokens, y, ldy, epilogue, status,
                      h.codes, h.scales, QuantTarget(), stream);
}

}  // namespace b200q

// ---- the entry that allocates nothing ------------------------------------------------------------
//
// The W4A4 route keeps the quantized activations and a status line in scratch memory. Here that
// scratch is a fixed array inside the library's own device image instead of a caller-supplied
// workspace, for callers that have no way to hand over device memory when they call.
namespace b200q {
namespace {

static __device__ __align__(256) uint8_t g_static_scratch[B200Q_NVFP4_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxScratchDevices = 64;
// The array's address on each device. In host code the symbol `g_static_scratch` itself is only a
// handle for the runtime, never a device pointer: the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device while that device is current.
uint8_t *g_scratch_address[kMaxScratchDevices] = {};
std::mutex g_scratch_mutex;

int32_t static_scratch(ErrorSlot &slot, uint8_t **out) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return fail(slot, "b200q_nvfp4_linear_noalloc: no CUDA device: %s", cudaGetErrorString(err));
  if (device < 0 || device >= kMaxScratchDevices) return fail(slot, "b200q_nvfp4_linear_noalloc: device ordinal %d is out of range", device);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_address[device] == nullptr) {
    void *address = nullptr;
    err = cudaGetSymbolAddress(&address, g_static_scratch);
    if (err != cudaSuccess || address == nullptr) {
      return fail(slot, "b200q_nvfp4_linear_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
    }
    // The status line needs no clearing: a file-scope __device__ array is zero when the module is
    // loaded, the kernels only ever OR bits into it, and everything behind it is rewritten by
    // every call before it is read.
    g_scratch_address[device] = static_cast<uint8_t *>(address);
  }
  *out = g_scratch_address[device];
  return 0;
}

bool is_aligned(const void *p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace

// The status line of the built-in scratch array on the current device, after `stream` has
// finished: 0 when b200q_nvfp4_linear_noalloc has not run on this device yet.
int32_t w4a4_noalloc_status(ErrorSlot &slot, cudaStream_t stream, uint32_t *status) {
  *status = 0;
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return fail(slot, "b200q_nvfp4_device_status: no CUDA device: %s", cudaGetErrorString(err));
  const uint8_t *address = nullptr;
  if (device >= 0 && device < kMaxScratchDevices) {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    address = g_scratch_address[device];
  }
  if (address == nullptr) return 0;
  err = cudaMemcpyAsync(status, address, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
  if (err != cudaSuccess) return fail(slot, "b200q_nvfp4_device_status: %s", cudaGetErrorString(err));
  return 0;
}

}  // namespace b200q

extern "C" int32_t b200q_nvfp4_linear_noalloc(const b200q_nvfp4_weight *w, const void *x, uint32_t tokens, void *y,
                                              uint32_t ldy, uint32_t epilogue, void *stream) {
  using namespace b200q;
  ErrorSlot &slot = nvfp4_error();
  const char *what = "b200q_nvfp4_linear_noalloc";
  if (w == nullptr || w->codes == nullptr || w->scales == nullptr) return fail(slot, "%s: weight is NULL", what);
  if (w->n == 0 || (w->n % 128u) != 0) return fail(slot, "%s: n = %u is not a positive multiple of 128", what, w->n);
  if (w->k == 0 || (w->k % 256u) != 0) return fail(slot, "%s: k = %u is not a positive multiple of 256", what, w->k);
  if (!is_aligned(w->codes, 32) || !is_aligned(w->scales, 16)) return fail(slot, "%s: weight planes are misaligned", what);
  if (!std::isfinite(w->weight_scale_divisor) || !(w->weight_scale_divisor > 0.0f) ||
      !std::isfinite(w->input_scale_divisor) || !(w->input_scale_divisor > 0.0f)) {
    return fail(slot, "%s: both scale divisors must be finite and positive", what);
  }
  if (tokens == 0) return fail(slot, "%s: tokens must be positive", what);
  if ((epilogue & ~static_cast<uint32_t>(B200Q_NVFP4_OUT_F32)) != 0u) return fail(slot, "%s: only STORE (optionally OUT_F32) is served", what);
  if (x == nullptr || !is_aligned(x, 16)) return fail(slot, "%s: x is NULL or not 16-byte aligned", what);
  if (y == nullptr || !is_aligned(y, 16) || (ldy % 8u) != 0 || ldy < w->n) {
    return fail(slot, "%s: y must be 16-byte aligned, ldy a multiple of 8 and at least n", what);
  }
  const uint64_t need = w4a4_workspace_bytes(w->k, tokens);
  if (need > B200Q_NVFP4_NOALLOC_SCRATCH_BYTES) {
    return fail(slot, "%s: %u tokens at k = %u need %llu bytes of scratch, the built-in array holds %llu", what, tokens, w->k,
                static_cast<unsigned long long>(need), static_cast<unsigned long long>(B200Q_NVFP4_NOALLOC_SCRATCH_BYTES));
  }
  const DeviceState *dev = device_state(slot);
  if (dev == nullptr) return -1;
  if (!dev->prepared) return fail(slot, "%s: the device was not prepared (call b200q_nvfp4_prepare at load)", what);
  uint8_t *scratch = nullptr;
  if (static_scratch(slot, &scratch) != 0) return -1;
  return w4a4_launch(slot, *dev, static_cast<const uint8_t *>(w->codes), static_cast<const uint8_t *>(w->scales), w->n, w->k,
                     w->weight_scale_divisor, w->input_scale_divisor, static_cast<const uint16_t *>(x), tokens, y, ldy,
                     epilogue, scratch, static_cast<cudaStream_t>(stream));
}

