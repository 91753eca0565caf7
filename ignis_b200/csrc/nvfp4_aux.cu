// NVFP4 seams: the logical-weight dequantizer and the activation block quantizer as standalone
// kernels, each held bit for bit to the reference's definition by the parity tests.
#include "nvfp4_internal.cuh"

namespace b200q {

namespace {

// out[r][c] = float(E2M1(code) * E4M3(scale) / d_w): the product is exact in fp32 and the IEEE
// division rounds once, which equals the reference's fp64 division rounded to float
// (kernel/vendor/tests/ops/quantized_weight.h:684-688): 53 >= 2 * 24 + 2 bits make the double
// rounding harmless.
__global__ void __launch_bounds__(256) nvfp4_dequantize_kernel(const uint8_t *__restrict__ codes,
                                                               const uint8_t *__restrict__ scales, uint32_t n, uint32_t k,
                                                               float d_w, float *__restrict__ out) {
  // one thread per 16-weight group: 8 code bytes, one scale byte, 16 floats out
  const uint64_t groups = static_cast<uint64_t>(n) * (k / 16u);
  for (uint64_t gi = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; gi < groups;
       gi += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
    const uint32_t row = static_cast<uint32_t>(gi / (k / 16u));
    const uint32_t grp = static_cast<uint32_t>(gi % (k / 16u));
    const uint32_t m_tile = row >> 7, inner = row & 127u;
    const uint64_t so = (static_cast<uint64_t>(m_tile) * (k / 64u) + (grp >> 2)) * 512u + (inner & 31u) * 16u +
                        (inner >> 5) * 4u + (grp & 3u);
    const uint32_t sbyte = scales[so];
    const uint32_t sh = e4m3x2_to_half2(sbyte);
    const float s = __half2float(__ushort_as_half(static_cast<unsigned short>(sh & 0xFFFFu)));
    const uint2 packed = *reinterpret_cast<const uint2 *>(codes + static_cast<uint64_t>(row) * (k / 2u) + grp * 8u);
    const uint32_t words[2] = {packed.x, packed.y};
    float4 *dst = reinterpret_cast<float4 *>(out + static_cast<uint64_t>(row) * k + grp * 16u);
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      uint32_t h[4];
      e2m1x8_to_half2x4(words[w], h);
      float v[8];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const __half2 hh = *reinterpret_cast<const __half2 *>(&h[b]);
        v[2 * b] = __fdiv_rn(__low2float(hh) * s, d_w);
        v[2 * b + 1] = __fdiv_rn(__high2float(hh) * s, d_w);
      }
      dst[2 * w] = make_float4(v[0], v[1], v[2], v[3]);
      dst[2 * w + 1] = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
}

// One 16-value block of activations to NVFP4: scale = E4M3_satfinite(rn(d_in * amax) / 6),
// codes = E2M1_satfinite_rn(rn(x * d_in) / decoded scale), zero scale gives zero codes; the even
// element in the low nibble. kernel/vendor/src/ops/linear/nvfp4/nvfp4_codec.cuh:81-110.
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
  const float unencoded = __fdiv_rn(__fmul_rn(d_in, amax), 6.0f);
  uint16_t s2;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(s2) : "f"(0.0f), "f"(unencoded));
  scale = static_cast<uint8_t>(s2 & 0xFFu);
  codes = make_uint2(0u, 0u);
  if (scale == 0) return;
  const uint32_t sh = e4m3x2_to_half2(scale);
  const float dec = __half2float(__ushort_as_half(static_cast<unsigned short>(sh & 0xFFFFu)));
  uint32_t packed[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float q0 = __fdiv_rn(__fmul_rn(v[2 * j], d_in), dec);
    const float q1 = __fdiv_rn(__fmul_rn(v[2 * j + 1], d_in), dec);
    uint32_t byte;
    asm("{ .reg .b8 b; cvt.rn.satfinite.e2m1x2.f32 b, %1, %2; cvt.u32.u8 %0, b; }" : "=r"(byte) : "f"(q1), "f"(q0));
    packed[j >> 2] |= byte << (8 * (j & 3));
  }
  codes = make_uint2(packed[0], packed[1]);
}

__global__ void __launch_bounds__(256) nvfp4_quantize_activations_kernel(const uint16_t *__restrict__ x, uint32_t tokens,
                                                                         uint32_t k, float d_in, uint8_t *__restrict__ codes,
                                                                         uint8_t *__restrict__ scales) {
  const uint64_t blocks = static_cast<uint64_t>(tokens) * (k / 16u);
  for (uint64_t bi = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; bi < blocks;
       bi += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
    const uint4 *src = reinterpret_cast<const uint4 *>(x + bi * 16u);
    uint2 c;
    uint8_t s;
    quantize_block16(src[0], src[1], d_in, c, s);
    *reinterpret_cast<uint2 *>(codes + bi * 8u) = c;
    scales[bi] = s;
  }
}

}  // namespace

int32_t dequantize_launch(ErrorSlot &slot, const uint8_t *codes, const uint8_t *scales, uint32_t n, uint32_t k, float d_w,
                          float *out, cudaStream_t stream) {
  const uint64_t groups = static_cast<uint64_t>(n) * (k / 16u);
  const uint32_t grid = static_cast<uint32_t>(groups / 256u < 148u * 16u ? (groups + 255u) / 256u : 148u * 16u);
  nvfp4_dequantize_kernel<<<grid, 256, 0, stream>>>(codes, scales, n, k, d_w, out);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(slot, "nvfp4 dequantize launch: %s", cudaGetErrorString(err));
  return 0;
}

int32_t quantize_activations_launch(ErrorSlot &slot, const uint16_t *x, uint32_t tokens, uint32_t k, float d_in,
                                    uint8_t *codes, uint8_t *scales, cudaStream_t stream) {
  const uint64_t blocks = static_cast<uint64_t>(tokens) * (k / 16u);
  const uint32_t grid = static_cast<uint32_t>(blocks / 256u < 148u * 16u ? (blocks + 255u) / 256u : 148u * 16u);
  nvfp4_quantize_activations_kernel<<<grid, 256, 0, stream>>>(x, tokens, k, d_in, codes, scales);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(slot, "nvfp4 activation quantizer launch: %s", cudaGetErrorString(err));
  return 0;
}

}  // namespace b200q
