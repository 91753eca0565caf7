// The tensor cores' block-scaled FP4 rate, measured: tcgen05.mma kind::mxf4nvf4 block_scale
// scale_vec::4X in a loop over operands that never leave the SM (codes in shared memory, scales in
// tensor memory, the accumulator in tensor memory), so nothing but the tensor pipe and its
// shared-memory reads is timed. It is the denominator the prefill GEMM (nvfp4_w4a4.cu) is reported
// against, the way the reference measures its card with a register-resident mma.sync loop
// (kernel/tests/bench_mma_peak.cu:1-25: independent chains, no memory traffic, the clock printed
// beside every rate).
//
// Two forms, the two the product kernels use: one CTA per SM issuing M 128 x N 256 x K 64, and a
// cluster of two CTAs issuing M 256 x N 256 x K 64 through cta_group::2 (each CTA holds its own 128
// rows of A and half of B). A CTA keeps one stage of operands (K = 256: four MMAs) and issues it
// `iterations` times into the same accumulator; commits go out in batches of eight stages on two
// alternating mbarriers, so the issuing thread waits for batch i - 1 while batch i runs and the
// pipe never drains. Every wait is bounded; a wait that runs out sets the status word and the CTA
// tears down.
#include "../../include/b200q_nvfp4.h"

#include "nvfp4_internal.cuh"
#include "nvfp4_tc.cuh"

namespace b200q {
namespace {

constexpr uint32_t kPeakABytes = 128 * 128;      // 128 rows x 256 E2M1 values
constexpr uint32_t kPeakBBytes = 256 * 128;      // 256 rows (one CTA's form); the pair form uses the first half
constexpr uint32_t kPeakSfBytes = 3 * 2048;      // scale tiles: A's 128 rows, B's two row tiles, four K atoms each
constexpr uint32_t kPeakSmem = kPeakABytes + kPeakBBytes + kPeakSfBytes + 64 + 1024;
constexpr uint32_t kBatch = 8;                   // stages per commit

__device__ uint32_t g_peak_status = 0;

__device__ __forceinline__ uint32_t peak_in_cta(uint32_t addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  return remote;
}

template <bool PAIR>
__device__ __forceinline__ void peak_cp(uint32_t taddr, uint64_t desc) {
  if (PAIR) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
  } else {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
  }
}
template <bool PAIR>
__device__ __forceinline__ void peak_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
  if (PAIR) {
    asm volatile("{ .reg .pred p; setp.ne.u32 p, %6, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p; }"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
                 : "memory");
  } else {
    asm volatile("{ .reg .pred p; setp.ne.u32 p, %6, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p; }"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
                 : "memory");
  }
}
template <bool PAIR>
__device__ __forceinline__ void peak_commit(uint32_t bar) {
  if (PAIR) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  }
}

template <bool PAIR>
__global__ void __launch_bounds__(128, 1) fp4_mma_peak_kernel(uint32_t iterations, float *sink) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;   // the 128-byte swizzle wants 1024-byte aligned tiles
  uint8_t *base_ptr = smem_raw + (base - raw);
  const uint32_t a_smem = base, b_smem = base + kPeakABytes, sf_smem = b_smem + kPeakBBytes;
  const uint32_t bars = sf_smem + kPeakSfBytes;   // two batch barriers, one for the scale copies
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + kPeakABytes + kPeakBBytes + kPeakSfBytes + 32);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank = 0;
  if (PAIR) rank = cluster_ctarank();

  // operands: codes from a counter hash (every nibble pattern occurs), every scale 1.0 (0x38)
  {
    uint32_t *codes = reinterpret_cast<uint32_t *>(base_ptr);
    for (uint32_t i = threadIdx.x; i < (kPeakABytes + kPeakBBytes) / 4u; i += blockDim.x) {
      uint32_t h = (i + 1u + blockIdx.x * 7919u) * 0x9E3779B9u;
      h ^= h >> 16;
      h *= 0x7FEB352Du;
      h ^= h >> 15;
      codes[i] = h;
    }
    uint32_t *sf = reinterpret_cast<uint32_t *>(base_ptr + kPeakABytes + kPeakBBytes);
    for (uint32_t i = threadIdx.x; i < kPeakSfBytes / 4u; i += blockDim.x) sf[i] = 0x38383838u;
  }
  if (threadIdx.x == 0) {
    mbar_init(bars, 1);
    mbar_init(bars + 8, 1);
    mbar_init(bars + 16, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads what the threads wrote
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's operands and barriers exist before the first MMA reads them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  bool ok = true;
  if (warp == 0 && lane == 0 && rank == 0u) {
    // scale columns behind the 256 accumulator columns: 16 for A's rows, 32 for B's
    const uint32_t sf_cols = tmem + 256u;
#pragma unroll
    for (uint32_t kb = 0; kb < 4; ++kb) {
      peak_cp<PAIR>(sf_cols + kb * 4u, smem_desc(sf_smem + kb * 512u, 128u, 0u));
      peak_cp<PAIR>(sf_cols + 16u + kb * 8u, smem_desc(sf_smem + 2048u + kb * 512u, 128u, 0u));
      peak_cp<PAIR>(sf_cols + 16u + kb * 8u + 4u, smem_desc(sf_smem + 4096u + kb * 512u, 128u, 0u));
    }
    peak_commit<PAIR>(PAIR ? peak_in_cta(bars + 16, 0u) : bars + 16);
    ok = mbar_wait(bars + 16, 0u);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // E2M1 x E2M1 (format 1 at bits 7 and 10), both K-major, N >> 3 at bit 17, UE4M3 scales, M >> 4 at bit 24
    const uint32_t idesc = (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | (((PAIR ? 256u : 128u) >> 4) << 24);
    const uint64_t a_desc = smem_desc(a_smem, 1024u, 2u), b_desc = smem_desc(b_smem, 1024u, 2u);
    uint32_t batches = 0;
    for (uint32_t it = 0; it < iterations && ok; ++it) {
#pragma unroll
      for (uint32_t kb = 0; kb < 4; ++kb) {
        peak_mma<PAIR>(tmem, a_desc + 2u * kb, b_desc + 2u * kb, idesc, sf_cols + kb * 4u, sf_cols + 16u + kb * 8u, (it | kb) != 0u ? 1u : 0u);
      }
      if ((it + 1u) % kBatch == 0u || it + 1u == iterations) {
        const uint32_t bar = bars + 8u * (batches & 1u);
        peak_commit<PAIR>(PAIR ? peak_in_cta(bar, 0u) : bar);
        if (batches > 0u) {   // the batch before this one: batches - 1 is use number (batches - 1) / 2 of its barrier
          ok = mbar_wait(bars + 8u * ((batches - 1u) & 1u), ((batches - 1u) >> 1) & 1u);
        }
        ++batches;
      }
    }
    if (ok && batches > 0u) ok = mbar_wait(bars + 8u * ((batches - 1u) & 1u), ((batches - 1u) >> 1) & 1u);
    if (!ok) atomicOr(&g_peak_status, 1u);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer stays until the pair's MMAs have retired
  if (warp == 0) {   // one accumulator word leaves the SM, so the loop has an observable result
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t v[32];
    tmem_ld32(tmem, v);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if (lane == 0 && sink != nullptr) sink[blockIdx.x] = __uint_as_float(v[0]);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    } else {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
  }
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int32_t b200q_nvfp4_mma_peak(uint32_t iterations, uint32_t pair, float *sink, uint32_t sink_count, double *flops,
                                        void *stream) {
  ErrorSlot &slot = nvfp4_error();
  const char *what = "b200q_nvfp4_mma_peak";
  if (iterations == 0 || iterations > (1u << 24)) return fail(slot, "%s: iterations must lie in 1..2^24", what);
  if (pair > 1u) return fail(slot, "%s: pair must be 0 or 1", what);
  const DeviceState *dev = device_state(slot);
  if (dev == nullptr) return -1;
  if (!dev->prepared) return fail(slot, "%s: the device was not prepared (call b200q_nvfp4_prepare at load)", what);
  const uint32_t ctas = pair ? static_cast<uint32_t>(dev->sm_count) / 2u * 2u : static_cast<uint32_t>(dev->sm_count);
  if (sink != nullptr && sink_count < ctas) return fail(slot, "%s: sink holds %u floats, the launch writes %u", what, sink_count, ctas);
  cudaError_t err = pair ? cudaFuncSetAttribute(fp4_mma_peak_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kPeakSmem))
                         : cudaFuncSetAttribute(fp4_mma_peak_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kPeakSmem));
  if (err != cudaSuccess) return fail(slot, "%s: %s", what, cudaGetErrorString(err));
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(ctas, 1, 1);
  config.blockDim = dim3(128, 1, 1);
  config.dynamicSmemBytes = kPeakSmem;
  config.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = pair ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  err = pair ? cudaLaunchKernelEx(&config, fp4_mma_peak_kernel<true>, iterations, sink)
             : cudaLaunchKernelEx(&config, fp4_mma_peak_kernel<false>, iterations, sink);
  if (err != cudaSuccess) return fail(slot, "%s: launch failed: %s", what, cudaGetErrorString(err));
  // per CTA and stage: four MMAs of 2 x 128 x 256 x 64 (the pair's M 256 is 128 per CTA)
  if (flops != nullptr) *flops = static_cast<double>(ctas) * iterations * 4.0 * 2.0 * 128.0 * 256.0 * 64.0;
  return 0;
}

extern "C" int32_t b200q_nvfp4_mma_peak_status(void *stream, uint32_t *status) {
  ErrorSlot &slot = nvfp4_error();
  if (status == nullptr) return fail(slot, "b200q_nvfp4_mma_peak_status: status is NULL");
  cudaError_t err = cudaMemcpyFromSymbolAsync(status, g_peak_status, sizeof(uint32_t), 0, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (err == cudaSuccess) err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(slot, "b200q_nvfp4_mma_peak_status: %s", cudaGetErrorString(err));
  return 0;
}
