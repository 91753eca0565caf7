// Device-side pieces shared by the dense trellis linear and the MoE expert kernels: the tile
// decode (format: kernel/src/trellis_decode.cuh:6-24 of the reference), the warp Hadamard, the
// cluster helpers and a warp's walk over its 128-input blocks.
#ifndef B200Q_TRELLIS_DEVICE_CUH
#define B200Q_TRELLIS_DEVICE_CUH

#include "common.cuh"

namespace b200q {
namespace trellis_dev {

constexpr uint32_t kMul1 = 0x83DCD12Du;

// Exclusive end bit of step p in a tile of class k2 = 2 K.
__host__ __device__ constexpr int step_end(int k2, int p) {
  return k2 == 5 ? 3 * ((p + 1) / 2) + 2 * (p / 2 + 1) : (k2 / 2) * (p + 1);
}

struct LaneWindow {
  uint32_t w0, w1, w2;  // word indices inside the tile
  uint32_t off;         // bit offset of the lane's first window bit inside word w0
};

__device__ __forceinline__ LaneWindow lane_window(uint32_t k2, int lane) {
  const int words = 4 * static_cast<int>(k2), bits = 128 * static_cast<int>(k2);
  int first = 4 * static_cast<int>(k2) * lane + static_cast<int>(k2 >> 1) - 16;  // end of step 8 lane, minus 16
  if (first < 0) first += bits;
  LaneWindow w;
  w.w0 = static_cast<uint32_t>(first >> 5);
  w.off = static_cast<uint32_t>(first & 31);
  w.w1 = w.w0 + 1 == static_cast<uint32_t>(words) ? 0u : w.w0 + 1;
  w.w2 = w.w1 + 1 == static_cast<uint32_t>(words) ? 0u : w.w1 + 1;
  return w;
}

// The lane's eight weights from its three words: four half2 in step order (steps 0,1 | 2,3 | 4,5 |
// 6,7), i.e. tile elements (r0, c0) (r0+1, c0) | (r0+8, c0) (r0+9, c0) | the same rows at c0 + 8,
// r0 = 2 (lane % 4), c0 = lane / 4.
template <int K2>
__device__ __forceinline__ void decode8(uint32_t a, uint32_t b, uint32_t c, uint32_t off, uint32_t (&frag)[4]) {
  const uint32_t hi = __funnelshift_l(b, a, off);
  const uint32_t mid = __funnelshift_l(c, b, off);
  uint32_t code[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    constexpr int base = step_end(K2, 0);
    const int d = step_end(K2, j) - base;  // constant after unrolling
    const uint32_t x = d == 0 ? hi : (d < 32 ? __funnelshift_l(mid, hi, d) : mid << (d - 32));
    code[j] = __dp4a((x >> 16) * kMul1, 0x01010101u, 0x6400u);
  }
  const __half2 k_inv = __halves2half2(__ushort_as_half(0x1EEE), __ushort_as_half(0x1EEE));
  const __half2 k_bias = __halves2half2(__ushort_as_half(0xC931), __ushort_as_half(0xC931));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t packed = __byte_perm(code[2 * i], code[2 * i + 1], 0x5410);
    const __half2 v = __hfma2(*reinterpret_cast<const __half2 *>(&packed), k_inv, k_bias);
    frag[i] = *reinterpret_cast<const uint32_t *>(&v);
  }
}

__device__ __forceinline__ void decode8_any(uint32_t k2, uint32_t a, uint32_t b, uint32_t c, uint32_t off,
                                            uint32_t (&frag)[4]) {
  switch (k2) {
    case 4: decode8<4>(a, b, c, off, frag); break;
    case 5: decode8<5>(a, b, c, off, frag); break;
    case 6: decode8<6>(a, b, c, off, frag); break;
    case 8: decode8<8>(a, b, c, off, frag); break;
    case 10: decode8<10>(a, b, c, off, frag); break;
    default: decode8<12>(a, b, c, off, frag); break;
  }
}

// v holds elements 4 lane .. 4 lane + 3 of a 128-vector; on return the vector times the natural
// order Sylvester Hadamard / sqrt(128): two stages inside the lane, five across lanes.
__device__ __forceinline__ void hadamard128(float (&v)[4], int lane) {
  const float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c;
  v[1] = b + d;
  v[2] = a - c;
  v[3] = b - d;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    // the upper lane of a pair keeps (other - own), the lower (own + other): one fused multiply-add by
    // -1 or +1 gives either, rounded once like the subtraction or the addition it stands for
    const float sign = (lane & m) != 0 ? -1.0f : 1.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(0xFFFFFFFFu, v[i], m);
      v[i] = __fmaf_rn(sign, v[i], o);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] *= 0.08838834764831845f;
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_barrier() {
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

struct TileWords {
  uint32_t w[8][3];
};

// The lane's three words of each of the 8 tiles of one 16-input step. `p0/p1/p2` point at the
// lane's words w0/w1/w2 of the step's first tile; tiles are 4 K2 words apart (a compile-time
// distance, so the loads carry immediate offsets).
template <int K2>
__device__ __forceinline__ void load_step(TileWords &tw, const uint32_t *p0, const uint32_t *p1, const uint32_t *p2) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    tw.w[j][0] = __ldg(p0 + j * 4 * K2);
    tw.w[j][1] = __ldg(p1 + j * 4 * K2);
    tw.w[j][2] = __ldg(p2 + j * 4 * K2);
  }
}

// One step of 16 inputs: the 8 tiles of the column block, decoded and multiplied.
template <int K2>
__device__ __forceinline__ void step_tiles(const TileWords &tw, uint32_t off, const uint2 bfrag, float (&acc)[8][4]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint32_t frag[4];
    decode8<K2>(tw.w[j][0], tw.w[j][1], tw.w[j][2], off, frag);
    mma_f16_f32(acc[j], frag[0], frag[2], frag[1], frag[3], bfrag.x, bfrag.y);
  }
}

// A warp's walk over its 128-input blocks [blk, b1) in strides of `stride` blocks: 8 steps per
// block, the words of the next step in flight while the current one is decoded (two register
// buffers, alternating). Accumulators live in the units of the current block's per-token scale
// and are carried into the next block's units by an exact power-of-two factor.
template <int K2>
__device__ __forceinline__ void walk_blocks(const uint32_t *col_base, uint64_t tk_stride, const LaneWindow &win, uint32_t blk,
                                            uint32_t b0, uint32_t b1, uint32_t stride, const uint2 *xs_side,
                                            const float *inv_side, const float *scale_side, int lane, float (&tot)[8][4]) {
  if (blk >= b1) return;
  const int t2 = (lane & 3) * 2;
  // Three running pointers (the lane's words w0, w1, w2 of the step to load next); every load is
  // pointer + compile-time offset. Inside a block the next step is one tile row further; after a
  // block's last step the pointers jump to the warp's next block.
  const uint32_t *q0 = col_base + win.w0 + static_cast<uint64_t>(blk) * 8u * tk_stride;
  const uint32_t *q1 = q0 + (static_cast<int64_t>(win.w1) - static_cast<int64_t>(win.w0));
  const uint32_t *q2 = q0 + (static_cast<int64_t>(win.w2) - static_cast<int64_t>(win.w0));
  const int64_t step = static_cast<int64_t>(tk_stride);
  const int64_t jump = static_cast<int64_t>(static_cast<uint64_t>(stride) * 8u - 7u) * step;
  TileWords even, odd;
  load_step<K2>(even, q0, q1, q2);
  q0 += step, q1 += step, q2 += step;
  float carry0 = 0.0f, carry1 = 0.0f;
  for (; blk < b1; blk += stride) {
    const uint32_t bl = blk - b0;
    const float f0 = carry0 * scale_side[bl * 8 + t2], f1 = carry1 * scale_side[bl * 8 + t2 + 1];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      tot[j][0] *= f0;
      tot[j][1] *= f1;
      tot[j][2] *= f0;
      tot[j][3] *= f1;
    }
    // after this block's last step: on to the next block, or (last block) back one step, so the
    // final prefetch re-reads the last step instead of running past the tensor
    const int64_t after = blk + stride < b1 ? jump : -step;
    const uint2 *xb = xs_side + static_cast<size_t>(bl) * 8 * 32 + lane;
#pragma unroll
    for (int kt = 0; kt < 8; kt += 2) {
      load_step<K2>(odd, q0, q1, q2);  // step kt + 1
      {
        const int64_t d = kt + 1 == 7 ? after : step;
        q0 += d, q1 += d, q2 += d;
      }
      step_tiles<K2>(even, win.off, xb[kt * 32], tot);
      load_step<K2>(even, q0, q1, q2);  // step kt + 2, or the first step of the next block
      q0 += step, q1 += step, q2 += step;
      step_tiles<K2>(odd, win.off, xb[(kt + 1) * 32], tot);
    }
    carry0 = inv_side[bl * 8 + t2];
    carry1 = inv_side[bl * 8 + t2 + 1];
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    tot[j][0] *= carry0;
    tot[j][1] *= carry1;
    tot[j][2] *= carry0;
    tot[j][3] *= carry1;
  }
}

}  // namespace trellis_dev
}  // namespace b200q

#endif
