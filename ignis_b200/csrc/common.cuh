// Shared host/device helpers of the library: the error channel, per-device state, launch helper
// with programmatic dependent launch, and the PTX wrappers the kernels use. sm_100a only.
#ifndef B200Q_COMMON_CUH
#define B200Q_COMMON_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

namespace b200q {

// ---- error channel ---------------------------------------------------------------------------
// One thread-local message per op family, as the reference keeps (trellis_linear.cu:29-44).
struct ErrorSlot {
  char text[512];
};
ErrorSlot &nvfp4_error();
ErrorSlot &trellis_error();
ErrorSlot &moe_error();

inline int32_t fail(ErrorSlot &slot, const char *fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(slot.text, sizeof(slot.text), fmt, args);
  va_end(args);
  return -1;
}

// ---- per-device state --------------------------------------------------------------------------
struct DeviceState {
  bool prepared = false;
  int sm_count = 0;
  int pdl = 1;           // programmatic dependent launch between the kernels of a call chain
  int gemv_rb = 0;       // B200Q_GEMV_RM: 32-row groups per CTA of the NVFP4 decode kernel (0: auto)
  int gemv_kc = 0;       // B200Q_GEMV_KC: its cluster size (0: auto)
  int gemv_ctas_per_sm = 2;
  int gemv_slots[9] = {};  // CTAs of the NVFP4 decode kernel resident at once, by cluster size (0: unknown)
  int a16_mma = 1;       // B200Q_A16_MMA: A16 calls of more than 8 tokens take the tensor-core kernel
  int a4_decode = 1;     // B200Q_A4_DECODE: AllowA4 calls of up to 32 tokens take the W4A4 decode kernel (0: the A16 route)
  int a4_slots[9] = {};      // CTAs of the W4A4 decode kernel placed at one per SM, by cluster size (0: unknown)
  int trellis_kc_max = 8;    // B200Q_TRELLIS_KC_MAX: largest cluster the trellis linear plans (measurement knob)
  int a4_decode_pair = -1;   // B200Q_A4_DECODE_PAIR: two row tiles per CTA of that kernel (-1: by the token count)
  int a4_decode_kc = 0;      // B200Q_A4_DECODE_KC: cluster size of that kernel (0: planned)
  int a4_decode_groups = 0;  // B200Q_A4_DECODE_GROUPS: quantizer groups per CTA of that kernel (0: chosen by the token count)
  int a4_decode_ctas = 2;  // B200Q_A4_DECODE_CTAS: CTAs of that kernel per SM (1: one CTA with a ring twice as deep)
  int a16_mma_wide = 1;  // B200Q_A16_MMA_WIDE: beyond 256 tokens the A16 tensor-core kernel takes token tiles of 512 (two accumulators per decoded stage)
  int w4a4_pair = 1;     // B200Q_W4A4_PAIR: the prefill GEMM on CTA pairs (cta_group::2, 256 x 256 tiles); 0: one CTA per 128 x 256 tile
  int gemv_xu = 8;       // B200Q_GEMV_XU: words per row of 8 decoded by the hardware E2M1 conversion
  int sm_cap = 0;        // IGNIS_TRELLIS_SM_CAP
  int moe_tc = 1;        // B200Q_MOE_TC: expert calls of more than 64 tokens take the tensor-core kernels
  int trellis_tc = 1;    // B200Q_TRELLIS_TC: dense trellis calls of more than 64 tokens with a workspace take the tensor-core route
  int peer_barrier_polls = 1 << 22;  // B200Q_PEER_BARRIER_POLLS: looks at a flag before b200q_peer_barrier gives up (400 ns apart)
};
// State of the current device, nullptr (and `slot` filled) when the device query fails.
DeviceState *device_state(ErrorSlot &slot);
// Prepares the current device once (thread-safe). 0 on success.
int32_t prepare_device(ErrorSlot &slot);
// Kernel attributes of one family each (defined beside the kernels), and all of them behind
// prepare_device: what every *_prepare entry point runs, so that a process that prepared through one
// family's entry can call the others' ops too.
int32_t prepare_nvfp4_kernels(ErrorSlot &slot);
int32_t prepare_trellis_kernels(ErrorSlot &slot);
int32_t prepare_moe_kernels(ErrorSlot &slot);
int32_t prepare_all(ErrorSlot &slot);

// The trellis tile decoder as a launch (trellis_linear.cu), shared by the dense and MoE entry points.
int32_t trellis_reconstruct_raw(ErrorSlot &slot, const char *what, const void *trellis, uint32_t k2, uint32_t in,
                                uint32_t out, uint32_t tile_stride, void *w_f16, void *stream);

// ---- launch helper -----------------------------------------------------------------------------
// Launches with the programmatic-stream-serialization attribute when `pdl` is set: the kernel may
// start while its predecessor in the stream drains, and orders itself with griddep_wait().
template <typename... KernelArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          bool pdl, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

#ifdef __CUDACC__
// ---- PTX wrappers ------------------------------------------------------------------------------

// Blocks until every grid this one depends on has completed and its writes are visible. A no-op
// when the grid was launched without a programmatic dependency.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next grid in the stream start its independent prologue.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// An L2 policy for data that is read once: first in line for eviction, so a weight stream does not
// push the (re-read) activations out of L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
// 32 bytes of a read-only stream that is touched once: no L1 allocation, evict-first in L2.
__device__ __forceinline__ void ldg256_stream(const void *p, uint32_t (&r)[8], uint64_t policy) {
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8], %9;"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "l"(p), "l"(policy));
}
__device__ __forceinline__ uint4 ldg128_stream(const void *p, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.b32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(policy));
  return v;
}
// 16 bytes of data an earlier kernel in the stream may have written while this grid was already
// resident (programmatic dependent launch): an ordinary coherent load, never the read-only path.
__device__ __forceinline__ uint4 ldg128_coherent(const void *p) {
  uint4 v;
  asm volatile("ld.global.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint2 ldg64_coherent(const void *p) {
  uint2 v;
  asm volatile("ld.global.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

// Four packed E2M1 pairs (one 32-bit word, eight codes) to four half2: word byte i -> h[i], the
// low nibble in the low half.
__device__ __forceinline__ void e2m1x8_to_half2x4(uint32_t word, uint32_t (&h)[4]) {
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}\n"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(word));
}

// Two E4M3 bytes (low 16 bits of `pair`) to half2, byte 0 in the low half.
__device__ __forceinline__ uint32_t e4m3x2_to_half2(uint32_t pair) {
  uint32_t h;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"(static_cast<uint16_t>(pair)));
  return h;
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  const __half2 r = __hmul2(*reinterpret_cast<const __half2 *>(&a), *reinterpret_cast<const __half2 *>(&b));
  return *reinterpret_cast<const uint32_t *>(&r);
}

// D += A(16x16, row) * B(16x8, col), fp16 operands, fp32 accumulate.
__device__ __forceinline__ void mma_f16_f32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The same with BF16 operands.
__device__ __forceinline__ void mma_bf16_f32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// ---- flags between the GPUs of a node ------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Lane s < peers of one warp waits, with a bound, until slot s of this rank's own flag array has
// reached `expected`; a wait that runs out records rank s in state[0] and returns.
__device__ __forceinline__ void peer_wait_flags(uint32_t *const *flags_peers, uint32_t *state, uint32_t peers, uint32_t rank,
                                                uint32_t polls, uint32_t expected, int lane) {
  if (static_cast<uint32_t>(lane) < peers) {
    const uint32_t *mine = flags_peers[rank] + lane;
    bool seen = false;
    for (uint32_t poll = 0; poll < polls; ++poll) {
      if (static_cast<int32_t>(ld_acquire_sys(mine) - expected) >= 0) {
        seen = true;
        break;
      }
      __nanosleep(poll < 4096u ? 250 : 1000);
    }
    if (!seen) atomicOr(state, 1u << lane);
  }
  __syncwarp();
}
#endif  // __CUDACC__

}  // namespace b200q

#endif  // B200Q_COMMON_CUH
