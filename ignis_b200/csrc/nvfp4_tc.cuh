// Device wrappers shared by the tensor-core NVFP4 kernels (mbarriers, TMA and bulk copies, tcgen05
// descriptors, MMAs and accumulator loads, cluster shared memory), the activation quantizer's
// 16-value block rule, and the host's tensor-map encoder entry.
#ifndef B200Q_NVFP4_TC_CUH
#define B200Q_NVFP4_TC_CUH

#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

namespace b200q {
namespace {

constexpr uint32_t kSpinLimit = 1u << 22;  // polls of an mbarrier before a wait gives up

// ---- activation quantizer: one block of 16 values (nvfp4_codec.cuh:81-110 of the reference) --------
// scale = E4M3_rn(d_in amax / 6); code_i = E2M1_rn((v_i d_in) / decoded scale), every operation a
// separately rounded fp32 one. The sixteen quotients share their divisor, so the division is one
// correctly rounded reciprocal and, per value, a product refined twice by its exact remainder
// (fused multiply-adds): the correctly rounded quotient for finite operands in the normal range,
// which is where a quotient that can reach a code boundary lies. Blocks with a non-finite
// d_in amax take IEEE divisions.
__device__ __forceinline__ uint32_t e2m1x2_byte(float lo, float hi) {
  uint32_t byte;
  asm("{ .reg .b8 b; cvt.rn.satfinite.e2m1x2.f32 b, %1, %2; cvt.u32.u8 %0, b; }" : "=r"(byte) : "f"(hi), "f"(lo));
  return byte;
}

__device__ __forceinline__ void quantize_block16(const uint4 lo, const uint4 hi, float d_in, uint2 &codes, uint8_t &scale) {
  const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  float v[16];
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    v[2 * j] = bf16_bits_to_f32(w[j] & 0xFFFFu);
    v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    amax = fmaxf(amax, fabsf(v[2 * j]));
    amax = fmaxf(amax, fabsf(v[2 * j + 1]));
  }
  const float top = __fmul_rn(d_in, amax);
  const float unencoded = __fdiv_rn(top, 6.0f);
  uint16_t s2;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(s2) : "f"(0.0f), "f"(unencoded));
  scale = static_cast<uint8_t>(s2 & 0xFFu);
  codes = make_uint2(0u, 0u);
  if (scale == 0) return;
  const uint32_t sh = e4m3x2_to_half2(scale);
  const float dec = __half2float(__ushort_as_half(static_cast<unsigned short>(sh & 0xFFFFu)));
  uint32_t packed[2] = {0u, 0u};
  if (top < __int_as_float(0x7F800000)) {
    const float r = __frcp_rn(dec);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float q[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float a = __fmul_rn(v[2 * j + i], d_in);
        float t = __fmul_rn(a, r);
        t = __fmaf_rn(__fmaf_rn(-dec, t, a), r, t);
        q[i] = __fmaf_rn(__fmaf_rn(-dec, t, a), r, t);
      }
      packed[j >> 2] |= e2m1x2_byte(q[0], q[1]) << (8 * (j & 3));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float q0 = __fdiv_rn(__fmul_rn(v[2 * j], d_in), dec);
      const float q1 = __fdiv_rn(__fmul_rn(v[2 * j + 1], d_in), dec);
      packed[j >> 2] |= e2m1x2_byte(q0, q1) << (8 * (j & 3));
    }
  }
  codes = make_uint2(packed[0], packed[1]);
}

// ---- mbarrier / TMA / tcgen05 wrappers ------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with `parity` to complete; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Shared-memory matrix descriptor: start address and byte offsets in 16-byte units, descriptor
// version 1 (bits 46..47), layout type in bits 61..63 (0 none, 2 the 128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t sbo_bytes, uint32_t layout) {
  return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) |
         (static_cast<uint64_t>(layout) << 61);
}

__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void mma_mxf4nvf4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                             uint32_t accumulate) {
  asm volatile("{ .reg .pred p; setp.ne.u32 p, %6, 0;\n"
               "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p; }"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 consecutive accumulator columns of this thread's lane (32x32b: one column per register).
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr)
      : "memory");
}

// One poll of the phase with `parity`.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(done)
               : "r"(bar), "r"(parity)
               : "memory");
  return done != 0u;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// ---- kind::f16 operands and cluster shared memory ------------------------------------------------
// K-major operand tile with the 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void mma_f16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{ .reg .pred p; setp.ne.u32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float *local_smem, uint32_t rank) {
  const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(local_smem));
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// ---- host: the driver's tensor-map encoder ----------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      return static_cast<EncodeTiledFn>(nullptr);
    }
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

}  // namespace
}  // namespace b200q

#endif
