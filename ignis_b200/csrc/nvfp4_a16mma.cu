// NVFP4 A16 products on the tensor cores: y[t][r] = sum_k w[r][k] x[t][k] with BF16 activations
// kept as they are and the weights decoded exactly, for token counts where the decode kernel's
// warp-level MMAs become the limit (more than 8 tokens) up to prefill widths. Stands where the
// reference runs nvfp4_small_t_kernel above a few tokens and nvfp4_a16_mma_kernel from 64 tokens
// (kernel/vendor/src/ops/linear/nvfp4/nvfp4_small_t.cuh:211-377, kernel/src/linear.cu:119-124);
// the design is not theirs.
//
//  * A CTA owns 128 weight rows (the MMA's M) and a token tile of BN = 32..256 (the MMA's N), and
//    walks K in stages of 64. Thread r of warps 0-3 owns row r: per stage it loads the row's 32
//    bytes of codes and its 4 scale bytes (one word of the swizzled plane: a stage is exactly one
//    scale tile column), widens them to BF16(code * scale) - exact, at most 6 significant bits -
//    and stores the 128 bytes into the stage's A tile in the K-major 128-byte-swizzle layout the
//    tensor core reads. Three further stages of codes are in flight in registers.
//  * Warp 4 streams the activations: one TMA load per stage of BN tokens x 64 BF16 values, the
//    same swizzle, straight from the caller's [tokens][k] matrix (tokens past the end read as
//    zero). Nothing is converted or scaled: BF16 x BF16 products are exact in the FP32 accumulator.
//  * Warp 5 owns tensor memory and issues tcgen05.mma kind::f16 (A and B BF16, M 128, N BN, K 16,
//    four per stage) into BN columns of FP32, then commits the stage back to its writers.
//  * K can be split over the CTAs of a cluster (narrow weights cannot fill the device otherwise):
//    every CTA pulls its accumulator to shared memory, the cluster meets in distributed shared
//    memory, and the tokens are dealt to the CTAs, which add the partial sums in rank order:
//    bit-reproducible, no global scratch.
//  * Every mbarrier wait is bounded; a wait that runs out sets a bit in the library's status word
//    (b200q_nvfp4_device_status) and the CTA falls through to the common exit, frees its tensor
//    memory and returns.
#include "nvfp4_internal.cuh"
#include "nvfp4_tc.cuh"

#include <mutex>

namespace b200q {
namespace {

constexpr int kBM = 128;             // weight rows per CTA
constexpr uint32_t kABytes = kBM * 128;  // one stage of BF16 weights: 128 rows x 64 values
constexpr uint32_t kProducerTimeout = 0x10u, kMmaTimeout = 0x20u, kEpilogueTimeout = 0x40u, kDecodeTimeout = 0x80u;
constexpr int kRing = 4;             // stages of codes a thread keeps in registers

__device__ uint32_t g_a16_status = 0;

struct A16Weight {
  const uint8_t *codes;
  const uint8_t *scales;
  void *y;
  uint32_t n, ldy;
  float inv_dw;
  uint32_t block_begin;  // first CTA of this weight
};

struct A16Params {
  A16Weight w[kMaxGroup];
  uint32_t count;
  uint32_t k, tokens;   // all tokens of the call; token tile blockIdx.y covers [bn y, bn y + bn)
  uint32_t bn;          // token tile: 32, 64, 128, 256, or 512 as two MMA tiles of 256 with an accumulator each
  uint32_t stages;      // ring depth in shared memory
  uint32_t kc;          // cluster size: K slices
  uint32_t epilogue;    // STORE / ADD / OUT_F32
};

struct CodeStage {
  uint32_t c[8];   // 64 codes
  uint32_t sc;     // their 4 scales
};

__global__ void __launch_bounds__(192) nvfp4_a16_mma_kernel(const __grid_constant__ CUtensorMap map_x,
                                                            const __grid_constant__ A16Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw);
  const uint32_t b_bytes = p.bn * 128u;                       // one stage of activations
  const uint32_t stage_bytes = kABytes + b_bytes;
  const uint32_t bars = base + p.stages * stage_bytes;        // full[stages], empty[stages], accumulator full; then the TMEM slot
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + p.stages * stage_bytes + 8u * (2u * p.stages + 1u) + 8u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank(), kc = p.kc;

  // Which weight, row tile and token tile this CTA serves. Without a K split the grid is walked
  // token tile first, so the CTAs running at one time share weight rows (read from HBM once, then
  // from the L2) rather than activations.
  uint32_t bx = blockIdx.x, by = blockIdx.y;
  if (kc == 1u) {
    const uint32_t id = blockIdx.y * gridDim.x + blockIdx.x;
    by = id % gridDim.y;
    bx = id / gridDim.y;
  }
  uint32_t wi = 0;
#pragma unroll
  for (uint32_t i = 1; i < kMaxGroup; ++i) {
    if (i < p.count && bx >= p.w[i].block_begin) wi = i;
  }
  const A16Weight &W = p.w[wi];
  const uint32_t m_tile = (bx - W.block_begin) / kc;
  const uint32_t k_stages = p.k / 64u;
  const uint32_t s0 = static_cast<uint32_t>(static_cast<uint64_t>(k_stages) * rank / kc);
  const uint32_t s1 = static_cast<uint32_t>(static_cast<uint64_t>(k_stages) * (rank + 1) / kc);
  const uint32_t tmem_cols = p.bn < 32u ? 32u : p.bn;
  const uint32_t mma_n = p.bn > 256u ? 256u : p.bn;   // tokens per MMA
  const uint32_t tok0 = by * p.bn;   // first token of this CTA's tile

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_init(bars + 8 * s, 128 + 1);               // 128 row threads and the producer's expect_tx arrival
      mbar_init(bars + 8 * (p.stages + s), 1);        // the MMA thread's commit
    }
    mbar_init(bars + 8 * 2 * p.stages, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp < 4) {
    // ---- row threads: decode this row's codes into the A tiles ----
    const uint32_t r = threadIdx.x;  // row of the tile, and later the accumulator lane
    const uint8_t *codes = W.codes + (static_cast<size_t>(m_tile) * 128u + r) * (p.k / 2u);
    const uint8_t *scales = W.scales + static_cast<size_t>(m_tile) * k_stages * 512u + (r & 31u) * 16u + (r >> 5) * 4u;
    const uint64_t policy = l2_evict_first_policy();
    CodeStage ring[kRing];
#pragma unroll
    for (int d = 0; d < kRing; ++d) {   // the weights never depend on the previous kernel
      const uint32_t s = s0 + d;
      if (s < s1) {
        ldg256_stream(codes + static_cast<size_t>(s) * 32u, ring[d].c, policy);
        ring[d].sc = *reinterpret_cast<const uint32_t *>(scales + static_cast<size_t>(s) * 512u);
      }
    }
    griddep_launch_dependents();
    griddep_wait();
    const uint32_t row_off = (r >> 3) * 1024u + (r & 7u) * 128u, sw = r & 7u;
    bool ok = true;
    for (uint32_t s = s0, it = 0; s < s1 && ok; s += kRing) {
#pragma unroll
      for (int d = 0; d < kRing; ++d) {
        if (s + d >= s1 || !ok) break;
        const uint32_t slot = it % p.stages;
        if (!mbar_wait(bars + 8 * (p.stages + slot), ((it / p.stages) & 1u) ^ 1u)) {
          if (lane == 0) atomicOr(&g_a16_status, kDecodeTimeout);
          ok = false;
          break;
        }
        // Both operands of the MMA are BF16, so the weights leave as BF16(code * scale): exact, at most
        // 6 significant bits. A code's fp16 bits moved down three places are a BF16 with the same
        // significand and an exponent 112 too small (zero stays zero); one BF16 multiply by
        // scale * 2^112 restores it and applies the group's scale at once.
        const uint32_t sc = ring[d].sc;
        const uint32_t s01 = e4m3x2_to_half2(sc & 0xFFFFu), s23 = e4m3x2_to_half2(sc >> 16);
        const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&s01));
        const float2 f23 = __half22float2(*reinterpret_cast<const __half2 *>(&s23));
        const float up = 5.192296858534828e33f;  // 2^112
        const float fs[4] = {f01.x * up, f01.y * up, f23.x * up, f23.y * up};
        __nv_bfloat162 sg[4];
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) sg[g4] = __floats2bfloat162_rn(fs[g4], fs[g4]);
        const uint32_t tile = base + slot * stage_bytes + row_off;
#pragma unroll
        for (int c = 0; c < 8; ++c) {   // word c: values 8 c .. 8 c + 7 of the stage, group c / 2
          uint32_t h[4];
          e2m1x8_to_half2x4(ring[d].c[c], h);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t tiny = ((h[j] & 0x7FFF7FFFu) >> 3) | (h[j] & 0x80008000u);
            const __nv_bfloat162 prod = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&tiny), sg[c >> 1]);
            h[j] = *reinterpret_cast<const uint32_t *>(&prod);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile + ((static_cast<uint32_t>(c) ^ sw) << 4)), "r"(h[0]),
                       "r"(h[1]), "r"(h[2]), "r"(h[3])
                       : "memory");
        }
        // the tile is read by the tensor core (async proxy): order these writes before it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(bars + 8 * slot);
        const uint32_t next = s + d + kRing;
        if (next < s1) {
          ldg256_stream(codes + static_cast<size_t>(next) * 32u, ring[d].c, policy);
          ring[d].sc = *reinterpret_cast<const uint32_t *>(scales + static_cast<size_t>(next) * 512u);
        }
        ++it;
      }
    }
  } else if (warp == 4) {
    // ---- producer of the activation tiles ----
    griddep_launch_dependents();
    griddep_wait();   // the activations may come from the previous kernel
    if (lane == 0) {
      for (uint32_t s = s0, it = 0; s < s1; ++s, ++it) {
        const uint32_t slot = it % p.stages;
        if (!mbar_wait(bars + 8 * (p.stages + slot), ((it / p.stages) & 1u) ^ 1u)) {
          atomicOr(&g_a16_status, kProducerTimeout);
          break;
        }
        const uint32_t full = bars + 8 * slot;
        mbar_expect_tx(full, b_bytes);
        tma_load_2d(base + slot * stage_bytes + kABytes, &map_x, full, static_cast<int32_t>(s * 64u), static_cast<int32_t>(tok0));
        if (p.bn > 256u) {   // the second MMA tile's tokens
          tma_load_2d(base + slot * stage_bytes + kABytes + 256u * 128u, &map_x, full, static_cast<int32_t>(s * 64u),
                      static_cast<int32_t>(tok0 + 256u));
        }
      }
    }
  } else {
    // ---- MMA issuer ----
    griddep_launch_dependents();
    griddep_wait();
    if (lane == 0) {
      // instruction descriptor: FP32 accumulator (bit 4), A and B BF16 (format 1 at bits 7 and
      // 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((mma_n >> 3) << 17) | ((static_cast<uint32_t>(kBM) >> 4) << 24);
      bool ok = true;
      for (uint32_t s = s0, it = 0; s < s1; ++s, ++it) {
        const uint32_t slot = it % p.stages;
        if (!mbar_wait(bars + 8 * slot, (it / p.stages) & 1u)) {
          atomicOr(&g_a16_status, kMmaTimeout);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t stage = base + slot * stage_bytes;
        const uint64_t a_desc = smem_desc_sw128(stage), b_desc = smem_desc_sw128(stage + kABytes);
#pragma unroll
        for (uint32_t kb = 0; kb < 4; ++kb) {   // 16 values along K are 32 bytes: two 16-byte units further
          mma_f16(tmem, a_desc + 2u * kb, b_desc + 2u * kb, idesc, (it | kb) != 0u ? 1u : 0u);
          if (p.bn > 256u) {   // the same decoded weights against the second 256 tokens, into their own accumulator
            mma_f16(tmem + 256u, a_desc + 2u * kb, b_desc + (256u * 128u >> 4) + 2u * kb, idesc, (it | kb) != 0u ? 1u : 0u);
          }
        }
        mma_commit(bars + 8 * (p.stages + slot));
      }
      if (ok) mma_commit(bars + 8 * 2 * p.stages);
    }
  }

  // ---- epilogue: thread r of warps 0-3 owns accumulator lane r = weight row r of the tile ----
  const uint32_t out_elem_f32 = p.epilogue & kEpilogueF32;
  const uint32_t row = m_tile * 128u + threadIdx.x;
  float *part = reinterpret_cast<float *>(base_ptr);   // [token][128] partial sums, over the (now idle) stage ring
  bool have = false;
  if (warp < 4) {
    have = mbar_wait(bars + 8 * 2 * p.stages, 0u);
    if (!have && lane == 0) atomicOr(&g_a16_status, kEpilogueTimeout);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  if (kc == 1u) {
    if (warp < 4 && have) {
      const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
      for (uint32_t c = 0; c < p.bn; c += 32) {
        uint32_t v[32];
        tmem_ld32(lane_base + c, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const uint32_t tok = tok0 + c + j;
          if (tok >= p.tokens) break;
          const size_t at = static_cast<size_t>(tok) * W.ldy + row;
          const float val = __fmul_rn(__uint_as_float(v[j]), W.inv_dw);  // not contracted into the residual add: one value for every epilogue
          if (out_elem_f32) {
            float *y = static_cast<float *>(W.y);
            y[at] = (p.epilogue & kEpilogueAdd) ? y[at] + val : val;
          } else {
            __nv_bfloat16 *y = static_cast<__nv_bfloat16 *>(W.y);
            y[at] = __float2bfloat16_rn((p.epilogue & kEpilogueAdd) ? val + __bfloat162float(y[at]) : val);
          }
        }
      }
    }
  } else {
    __syncthreads();   // every role is done with the stage ring: the partial sums take its place
    if (warp < 4) {
      const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
      for (uint32_t c = 0; c < p.bn; c += 32) {
        uint32_t v[32];
        if (have) {
          tmem_ld32(lane_base + c, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) part[static_cast<size_t>(c + j) * 128u + threadIdx.x] = have ? __uint_as_float(v[j]) : 0.0f;
      }
    }
    __syncwarp();
    cluster_sync_all();
    if (warp < 4) {
      // tokens dealt over the cluster's CTAs; partial sums added in rank order
      for (uint32_t tl = rank; tl < p.bn && tok0 + tl < p.tokens; tl += kc) {
        float sum = 0.0f;
        for (uint32_t q = 0; q < kc; ++q) sum += ld_cluster_f32(part + static_cast<size_t>(tl) * 128u + threadIdx.x, q);
        const size_t at = static_cast<size_t>(tok0 + tl) * W.ldy + row;
        const float val = __fmul_rn(sum, W.inv_dw);
        if (out_elem_f32) {
          float *y = static_cast<float *>(W.y);
          y[at] = (p.epilogue & kEpilogueAdd) ? y[at] + val : val;
        } else {
          __nv_bfloat16 *y = static_cast<__nv_bfloat16 *>(W.y);
          y[at] = __float2bfloat16_rn((p.epilogue & kEpilogueAdd) ? val + __bfloat162float(y[at]) : val);
        }
      }
    }
    __syncwarp();
    cluster_sync_all();   // no CTA leaves while a peer may still read its partial sums
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
  }
}

// ---- host side --------------------------------------------------------------------------------
constexpr size_t kA16MaxSmem = 220 * 1024;

size_t a16_smem_bytes(uint32_t bn, uint32_t stages) { return static_cast<size_t>(stages) * (kABytes + bn * 128u) + 8u * (2u * stages + 1u) + 16u + 1024u; }

}  // namespace

int32_t a16mma_prepare(ErrorSlot &slot) {
  const cudaError_t err = cudaFuncSetAttribute(nvfp4_a16_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(kA16MaxSmem));
  if (err != cudaSuccess) return fail(slot, "nvfp4 A16 tensor-core kernel attributes: %s", cudaGetErrorString(err));
  if (encode_tiled_fn() == nullptr) return fail(slot, "cuTensorMapEncodeTiled is not available from this driver");
  return 0;
}

bool a16mma_takes(uint32_t k, const void *x) { return (k % 64u) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0; }

// `count` weights sharing x, any number of tokens: token tiles of up to 256 side by side in the grid.
int32_t a16mma_launch(ErrorSlot &slot, const DeviceState &dev, const GemvWeight *weights, uint32_t count, const uint16_t *x,
                      uint32_t k, uint32_t tokens, uint32_t epilogue, cudaStream_t stream) {
  A16Params p = {};
  p.count = count;
  p.k = k;
  p.tokens = tokens;
  p.bn = tokens <= 32u ? 32u : (tokens <= 64u ? 64u : (tokens <= 128u ? 128u : (tokens <= 256u || dev.a16_mma_wide == 0 ? 256u : 512u)));
  p.epilogue = epilogue;
  // ring depth: as many stages as fit beside the other CTAs this token tile leaves room for
  const uint32_t stage_bytes = kABytes + p.bn * 128u;
  const uint32_t ctas_per_sm = p.bn <= 32u ? 3u : (p.bn <= 64u ? 2u : 1u);
  const uint32_t budget = static_cast<uint32_t>(kA16MaxSmem / ctas_per_sm) - 2048u;
  uint32_t stages = budget / stage_bytes;
  if (stages > 8u) stages = 8u;
  if (stages < 2u) return fail(slot, "nvfp4 A16 tensor-core route: no room for two stages");
  p.stages = stages;
  // cluster size: narrow weights split K so the launch fills the device
  uint32_t row_tiles = 0;
  for (uint32_t i = 0; i < count; ++i) row_tiles += weights[i].n / 128u;
  const uint32_t slots = static_cast<uint32_t>(dev.sm_count) * ctas_per_sm;
  const uint32_t k_stages = k / 64u;
  const uint32_t token_tiles = (tokens + p.bn - 1u) / p.bn;
  uint32_t kc = 1;
  if (p.bn * 512u <= stages * stage_bytes) {  // the cluster reduction keeps bn x 128 floats in shared memory, over the idle ring
    while (kc < 8u && row_tiles * token_tiles * (kc + 1u) <= slots && k_stages / (kc + 1u) >= 2u * stages) ++kc;
  }
  p.kc = kc;
  uint32_t ctas = 0;
  for (uint32_t i = 0; i < count; ++i) {
    A16Weight &g = p.w[i];
    g.codes = weights[i].codes;
    g.scales = weights[i].scales;
    g.y = weights[i].y[0];
    g.n = weights[i].n;
    g.ldy = weights[i].ldy;
    g.inv_dw = weights[i].inv_dw;
    g.block_begin = ctas;
    ctas += weights[i].n / 128u * kc;
  }
  EncodeTiledFn encode = encode_tiled_fn();
  CUtensorMap map_x;
  {
    const cuuint64_t dims[2] = {k, tokens};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2u};
    const cuuint32_t box[2] = {64u, p.bn > 256u ? 256u : p.bn};
    const cuuint32_t elem[2] = {1, 1};
    if (encode == nullptr ||
        encode(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(x), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return fail(slot, "nvfp4 A16 tensor-core route: tensor map encoding failed");
    }
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(ctas, (tokens + p.bn - 1u) / p.bn, 1);
  config.blockDim = dim3(192, 1, 1);
  config.dynamicSmemBytes = a16_smem_bytes(p.bn, stages);
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kc;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = dev.pdl ? 2 : 1;
  const cudaError_t err = cudaLaunchKernelEx(&config, nvfp4_a16_mma_kernel, map_x, p);
  if (err != cudaSuccess) return fail(slot, "nvfp4 A16 tensor-core launch: %s", cudaGetErrorString(err));
  return 0;
}

int32_t a16mma_status(ErrorSlot &slot, cudaStream_t stream, uint32_t *status) {
  cudaError_t err = cudaMemcpyFromSymbolAsync(status, g_a16_status, sizeof(uint32_t), 0, cudaMemcpyDeviceToHost, stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
  if (err != cudaSuccess) return fail(slot, "b200q_nvfp4_device_status: %s", cudaGetErrorString(err));
  return 0;
}

}  // namespace b200q
