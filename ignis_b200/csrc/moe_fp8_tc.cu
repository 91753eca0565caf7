// The MoE block's shared expert (FP8 E4M3 rows with a BF16 scale per row,
// kernel/include/ignis_fp8_linear.h:4-10) for wide calls, on the tensor cores:
// h = BF16(silu(gate x) * (up x)), shared = down h in FP32. Stands where the reference runs its FP8
// row-scale linear over the prefill's tokens (kernel/src/moe_prefill.cu:454-492 calls it between the
// routed experts and the combine); the design is the A16 NVFP4 tensor-core kernel's.
//
//  * A CTA owns 128 weight rows (the MMA's M) and a tile of 256 tokens (the MMA's N) and walks K in
//    stages of 64. Thread r of warps 0-3 owns row r: per stage it loads the row's 64 codes, widens
//    them to BF16 - exact: the fp16 bits of an E4M3 value moved down three places are a BF16 with
//    an exponent 112 too small, one BF16 multiply by 2^112 restores it - and stores the 128 bytes
//    into the stage's A tile in the K-major 128-byte-swizzle layout. MODE 0 does this for the gate
//    row and the up row of the same index: two A tiles, two accumulators, one token tile.
//  * Warp 4 streams the BF16 activations by TMA as the caller holds them (tokens past the end read
//    as zero); warp 5 owns tensor memory and issues tcgen05.mma kind::f16 (BF16 x BF16, FP32).
//  * Epilogue: thread r owns accumulator lane r = weight row r; the row scale multiplies the sum
//    once. MODE 0 writes BF16(silu(g) * u), MODE 1 FP32.
//  * Every mbarrier wait is bounded; a wait that runs out sets a bit in a status word that
//    ignis_moe_workspace_status reports (bit 3), and the CTA frees its tensor memory and returns.
#include "moe_internal.cuh"
#include "nvfp4_tc.cuh"

namespace b200q {
namespace {

constexpr uint32_t kBM = 128, kBN = 256;
constexpr uint32_t kABytes = kBM * 128u;   // one stage of one weight: 128 rows x 64 BF16
constexpr uint32_t kBBytes = kBN * 128u;   // one stage of activations: 256 tokens x 64 BF16
constexpr int kRing = 2;                   // stages of codes a row thread keeps in registers
constexpr uint32_t kProducerTimeout = 1u, kMmaTimeout = 2u, kEpilogueTimeout = 4u, kDecodeTimeout = 8u;

__device__ uint32_t g_fp8_tc_status = 0;

struct Fp8TcParams {
  const uint8_t *w0, *w1;   // MODE 0: gate, up; MODE 1: down (w1 unused)
  uint32_t rows, cols, tokens, stages;
  void *y;                  // MODE 0: BF16 [tokens][rows]; MODE 1: FP32 [tokens][rows]
};

// Eight E4M3 codes (two words) as eight BF16 values in four registers, exactly.
__device__ __forceinline__ void e4m3x8_to_bf16x8(uint32_t lo, uint32_t hi, uint32_t (&out)[4]) {
  const uint32_t h[4] = {e4m3x2_to_half2(lo & 0xFFFFu), e4m3x2_to_half2(lo >> 16), e4m3x2_to_half2(hi & 0xFFFFu),
                         e4m3x2_to_half2(hi >> 16)};
  const __nv_bfloat162 up = __floats2bfloat162_rn(5.192296858534828e33f, 5.192296858534828e33f);   // 2^112
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t tiny = ((h[j] & 0x7FFF7FFFu) >> 3) | (h[j] & 0x80008000u);
    const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&tiny), up);
    out[j] = *reinterpret_cast<const uint32_t *>(&v);
  }
}

template <int MODE>
__global__ void __launch_bounds__(192) moe_fp8_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ Fp8TcParams p) {
  constexpr int S = MODE == 0 ? 2 : 1;
  constexpr uint32_t kStageBytes = S * kABytes + kBBytes;
  constexpr uint32_t kTmemCols = S * kBN;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw);
  const uint32_t bars = base + p.stages * kStageBytes;   // full[stages], empty[stages], accumulator full; then the TMEM slot
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + p.stages * kStageBytes + 8u * (2u * p.stages + 1u) + 8u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t m_tile = blockIdx.x, tok0 = blockIdx.y * kBN;
  const uint32_t k_stages = p.cols / 64u;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_init(bars + 8 * s, 128 + 1);              // 128 row threads and the producer's expect_tx arrival
      mbar_init(bars + 8 * (p.stages + s), 1);       // the MMA thread's commit
    }
    mbar_init(bars + 8 * 2 * p.stages, 1);
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

  if (warp < 4) {
    // ---- row threads: widen this row's codes into the A tiles ----
    const uint32_t r = threadIdx.x;
    const uint8_t *rows_of[2] = {p.w0 + (static_cast<size_t>(m_tile) * kBM + r) * p.cols, p.w1 + (static_cast<size_t>(m_tile) * kBM + r) * p.cols};
    uint4 ring[kRing][S][4];
#pragma unroll
    for (int d = 0; d < kRing; ++d) {   // the weights never depend on the previous kernel
      if (static_cast<uint32_t>(d) < k_stages) {
#pragma unroll
        for (int s = 0; s < S; ++s)
#pragma unroll
          for (int q = 0; q < 4; ++q) ring[d][s][q] = __ldg(reinterpret_cast<const uint4 *>(rows_of[s] + static_cast<size_t>(d) * 64u) + q);
      }
    }
    griddep_launch_dependents();
    griddep_wait();
    const uint32_t row_off = (r >> 3) * 1024u + (r & 7u) * 128u, sw = r & 7u;
    bool ok = true;
    for (uint32_t st = 0, it = 0; st < k_stages && ok; st += kRing) {
#pragma unroll
      for (int d = 0; d < kRing; ++d) {
        if (st + d >= k_stages || !ok) break;
        const uint32_t slot = it % p.stages;
        if (!mbar_wait(bars + 8 * (p.stages + slot), ((it / p.stages) & 1u) ^ 1u)) {
          if (lane == 0) atomicOr(&g_fp8_tc_status, kDecodeTimeout);
          ok = false;
          break;
        }
#pragma unroll
        for (int s = 0; s < S; ++s) {
          const uint32_t tile = base + slot * kStageBytes + static_cast<uint32_t>(s) * kABytes + row_off;
#pragma unroll
          for (int q = 0; q < 4; ++q) {   // 16 codes: two 16-byte chunks of BF16
            const uint4 c = ring[d][s][q];
            uint32_t lo[4], hi[4];
            e4m3x8_to_bf16x8(c.x, c.y, lo);
            e4m3x8_to_bf16x8(c.z, c.w, hi);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile + ((static_cast<uint32_t>(2 * q) ^ sw) << 4)), "r"(lo[0]),
                         "r"(lo[1]), "r"(lo[2]), "r"(lo[3])
                         : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile + ((static_cast<uint32_t>(2 * q + 1) ^ sw) << 4)), "r"(hi[0]),
                         "r"(hi[1]), "r"(hi[2]), "r"(hi[3])
                         : "memory");
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads the tile through the async proxy
        mbar_arrive(bars + 8 * slot);
        const uint32_t next = st + d + kRing;
        if (next < k_stages) {
#pragma unroll
          for (int s = 0; s < S; ++s)
#pragma unroll
            for (int q = 0; q < 4; ++q) ring[d][s][q] = __ldg(reinterpret_cast<const uint4 *>(rows_of[s] + static_cast<size_t>(next) * 64u) + q);
        }
        ++it;
      }
    }
  } else if (warp == 4) {
    // ---- producer of the activation tiles ----
    griddep_launch_dependents();
    griddep_wait();   // MODE 1 reads what MODE 0 wrote
    if (lane == 0) {
      for (uint32_t st = 0; st < k_stages; ++st) {
        const uint32_t slot = st % p.stages;
        if (!mbar_wait(bars + 8 * (p.stages + slot), ((st / p.stages) & 1u) ^ 1u)) {
          atomicOr(&g_fp8_tc_status, kProducerTimeout);
          break;
        }
        const uint32_t full = bars + 8 * slot;
        mbar_expect_tx(full, kBBytes);
        tma_load_2d(base + slot * kStageBytes + S * kABytes, &map_x, full, static_cast<int32_t>(st * 64u), static_cast<int32_t>(tok0));
      }
    }
  } else {
    // ---- MMA issuer ----
    griddep_launch_dependents();
    griddep_wait();
    if (lane == 0) {
      // FP32 accumulator (bit 4), A and B BF16 (format 1 at bits 7 and 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((kBM >> 4) << 24);
      bool ok = true;
      for (uint32_t st = 0; st < k_stages; ++st) {
        const uint32_t slot = st % p.stages;
        if (!mbar_wait(bars + 8 * slot, (st / p.stages) & 1u)) {
          atomicOr(&g_fp8_tc_status, kMmaTimeout);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t stage = base + slot * kStageBytes;
        const uint64_t b_desc = smem_desc_sw128(stage + S * kABytes);
#pragma unroll
        for (int s = 0; s < S; ++s) {
          const uint64_t a_desc = smem_desc_sw128(stage + static_cast<uint32_t>(s) * kABytes);
#pragma unroll
          for (uint32_t kb = 0; kb < 4; ++kb) {
            mma_f16(tmem + static_cast<uint32_t>(s) * kBN, a_desc + 2u * kb, b_desc + 2u * kb, idesc, (st | kb) != 0u ? 1u : 0u);
          }
        }
        mma_commit(bars + 8 * (p.stages + slot));
      }
      if (ok) mma_commit(bars + 8 * 2 * p.stages);
    }
  }

  // ---- epilogue: thread r of warps 0-3 owns accumulator lane r = weight row r of the tile ----
  if (warp < 4) {
    const bool have = mbar_wait(bars + 8 * 2 * p.stages, 0u);
    if (!have && lane == 0) atomicOr(&g_fp8_tc_status, kEpilogueTimeout);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t row = m_tile * kBM + threadIdx.x;
    if (have && row < p.rows) {
      const uint64_t scale_off = (static_cast<uint64_t>(p.rows) * p.cols + 255u) & ~static_cast<uint64_t>(255u);
      const float s0 = bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(p.w0 + scale_off)[row]);
      const float s1 = MODE == 0 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(p.w1 + scale_off)[row]) : 0.0f;
      const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
      for (uint32_t c = 0; c < kBN && tok0 + c < p.tokens; c += 32) {
        uint32_t g[32], u[32];
        tmem_ld32(lane_base + c, g);
        if (MODE == 0) tmem_ld32(lane_base + kBN + c, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const uint32_t tok = tok0 + c + j;
          if (tok >= p.tokens) break;
          const size_t at = static_cast<size_t>(tok) * p.rows + row;
          if (MODE == 0) {
            const float gv = __uint_as_float(g[j]) * s0, uv = __uint_as_float(u[j]) * s1;
            static_cast<__nv_bfloat16 *>(p.y)[at] = __float2bfloat16_rn(gv / (1.0f + __expf(-gv)) * uv);
          } else {
            static_cast<float *>(p.y)[at] = __uint_as_float(g[j]) * s0;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

constexpr size_t kFp8TcMaxSmem = 220 * 1024;

template <int MODE>
size_t fp8_tc_smem(uint32_t stages) {
  constexpr uint32_t kStageBytes = (MODE == 0 ? 2u : 1u) * kABytes + kBBytes;
  return static_cast<size_t>(stages) * kStageBytes + 8u * (2u * stages + 1u) + 16u + 1024u;
}

template <int MODE>
cudaError_t fp8_tc_launch(const uint8_t *w0, const uint8_t *w1, uint32_t rows, uint32_t cols, const uint16_t *x, uint32_t tokens, void *y,
                          bool pdl, cudaStream_t stream) {
  Fp8TcParams p = {};
  p.w0 = w0;
  p.w1 = w1;
  p.rows = rows;
  p.cols = cols;
  p.tokens = tokens;
  p.y = y;
  p.stages = MODE == 0 ? 3u : 4u;
  EncodeTiledFn encode = encode_tiled_fn();
  CUtensorMap map_x;
  const cuuint64_t dims[2] = {cols, tokens};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2u};
  const cuuint32_t box[2] = {64u, kBN};
  const cuuint32_t elem[2] = {1, 1};
  if (encode == nullptr ||
      encode(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(x), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    return cudaErrorInvalidValue;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(rows / kBM, (tokens + kBN - 1u) / kBN, 1);
  config.blockDim = dim3(192, 1, 1);
  config.dynamicSmemBytes = fp8_tc_smem<MODE>(p.stages);
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&config, moe_fp8_tc_kernel<MODE>, map_x, p);
}

}  // namespace

int32_t moe_fp8_tc_prepare(ErrorSlot &slot) {
  cudaError_t err = cudaFuncSetAttribute(moe_fp8_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kFp8TcMaxSmem));
  if (err == cudaSuccess) {
    err = cudaFuncSetAttribute(moe_fp8_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kFp8TcMaxSmem));
  }
  if (err != cudaSuccess) return fail(slot, "MoE shared-expert tensor-core kernel attributes: %s", cudaGetErrorString(err));
  if (encode_tiled_fn() == nullptr) return fail(slot, "cuTensorMapEncodeTiled is not available from this driver");
  return 0;
}

bool moe_fp8_tc_takes(const DeviceState &dev, uint32_t hidden, uint32_t inter, uint32_t tokens, const void *x, const void *h) {
  return dev.moe_tc != 0 && tokens > 64u && hidden % 128u == 0 && inter % 128u == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(h) & 15u) == 0;
}

cudaError_t moe_fp8_tc_shared_expert(const DeviceState &dev, const uint8_t *gate, const uint8_t *up, const uint8_t *down, const uint16_t *x,
                                     uint32_t tokens, uint32_t hidden, uint32_t inter, void *h, float *shared, cudaStream_t stream) {
  cudaError_t err = fp8_tc_launch<0>(gate, up, inter, hidden, x, tokens, h, dev.pdl != 0, stream);
  if (err == cudaSuccess) {
    err = fp8_tc_launch<1>(down, down, hidden, inter, static_cast<const uint16_t *>(h), tokens, shared, dev.pdl != 0, stream);
  }
  return err;
}

cudaError_t moe_fp8_tc_status(uint32_t *status, cudaStream_t stream) {
  return cudaMemcpyFromSymbolAsync(status, g_fp8_tc_status, sizeof(uint32_t), 0, cudaMemcpyDeviceToHost, stream);
}

}  // namespace b200q
