// NVFP4 decode route: y[t][r] = sum_k w[r][k] x[t][k] for 1..32 tokens, the weights streamed from
// HBM exactly once for all tokens. One kernel per call, no workspace.
//
// Stands where the reference runs nvfp4_gemv_kernel (T = 1) and nvfp4_small_t_kernel (T = 2..32)
// (kernel/vendor/src/ops/linear/nvfp4/nvfp4_gemv.cuh:199, nvfp4_small_t.cuh:211-377) under the A16
// policy; the design is not theirs:
//
//  * A warp owns 32 output rows {base + g + 32 q : g = lane / 4, q = 0..3}, the four rows whose
//    scales share one 16-byte word of the swizzled scale plane, and walks K in steps of 256. Per
//    step a lane loads 32 contiguous bytes of codes per row (one 256-bit load each: the 64
//    weights of one scale tile) and the 16 scale bytes of those 4 rows x 4 groups.
//  * Codes become fp16 and are multiplied by their E4M3 scale in fp16 (exact: at most 6
//    significant bits). The products are the A fragments of mma.sync m16n8k16 (fp16 in, fp32
//    accumulate); the tokens are the MMA's N, so 1 and 8 tokens cost the same weight traffic and
//    the same decode. The order of k inside an MMA is permuted (lane t supplies the k of its own
//    64-weight chunk): a sum does not care, and both operands use the same permutation.
//  * The CTA first rewrites its K slice of the BF16 activations as fp16 B fragments in shared
//    memory, scaled per (token, slice) by a power of two so the largest magnitude sits in
//    [2^13, 2^14): every BF16 value within 2^-27 of the slice's maximum converts exactly. The
//    inverse scale is applied to the slice's fp32 partial sums.
//  * K is split over the warps of a CTA and over the CTAs of a thread-block cluster; partial sums
//    meet in distributed shared memory and are added in a fixed order, so results are
//    bit-reproducible and the call needs no global scratch.
//  * Programmatic dependent launch: the first weight loads are issued before the grid waits for
//    its predecessor, so in a chain of layers the weight stream does not stop between kernels.
#include "nvfp4_internal.cuh"

namespace b200q {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;

// A build with -DB200Q_GEMV_TRACE (python -m ignis_b200.build --trace: a second library, never the
// shipped one) stamps the global timer at the phase boundaries of every CTA, for the timeline of a
// chain of calls: [0] entry, [1] first weight loads issued, [2] predecessor complete, [3]
// activations rewritten, [4] K loop done, [5] partial sums written, [6] cluster met, [7] SM and
// grid size, [8] the first chunk's maximum known (first pass over the activations done), [9] its
// fragments stored (before the CTA's barrier). The host numbers the launches (modulo 128) in bits 16..22 of the epilogue word, which
// the kernel otherwise reads through single-bit masks.
#ifdef B200Q_GEMV_TRACE
constexpr int kTraceLaunches = 128, kTraceCtas = 512, kTraceWords = 10;
__device__ unsigned long long g_trace[kTraceLaunches][kTraceCtas][kTraceWords];
__device__ __forceinline__ void trace_stamp(int launch, int word) {
  if (launch < 0 || blockIdx.x >= kTraceCtas) return;
  unsigned long long now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
  g_trace[launch][blockIdx.x][word] = now;
}
#define GEMV_TRACE_BEGIN(word)                                                   \
  const int trace_launch = threadIdx.x == 0 ? static_cast<int>(((word) >> 16) & 127u) : -1; \
  if (trace_launch >= 0 && blockIdx.x < kTraceCtas) {                            \
    unsigned int sm;                                                             \
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));                              \
    g_trace[trace_launch][blockIdx.x][7] = sm | (static_cast<unsigned long long>(gridDim.x) << 32); \
  }                                                                              \
  trace_stamp(trace_launch, 0)
#define GEMV_TRACE(word) trace_stamp(trace_launch, word)
#else
#define GEMV_TRACE_BEGIN(word) constexpr int trace_launch = -1
#define GEMV_TRACE(word) ((void)trace_launch)
#endif

struct Stage {
  uint32_t c[4][8];  // 32 bytes of codes for each of the lane's four rows
  uint4 sc;          // scales: .x .y .z .w = rows q = 0..3, byte j = group j of the lane's scale tile
};

__device__ __forceinline__ void zero_stage(Stage &st) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
#pragma unroll
    for (int i = 0; i < 8; ++i) st.c[q][i] = 0u;
  }
  st.sc = make_uint4(0u, 0u, 0u, 0u);
}

struct WarpRows {
  const uint8_t *codes;   // row (base + g), byte 32 t
  const uint8_t *scales;  // scale tile (m_tile, 0), byte 16 (J 8 + g)
  size_t row_stride32;    // bytes between rows 32 apart
  uint64_t policy;        // L2 eviction policy of the weight stream
  bool active;
};

__device__ __forceinline__ void load_stage(Stage &st, const WarpRows &rows, int step, int c1, int lane_t,
                                           uint32_t scale_tiles) {
  const uint32_t tile = static_cast<uint32_t>(step) * 4u + static_cast<uint32_t>(lane_t);
  if (rows.active && step < c1 && tile < scale_tiles) {
    const uint8_t *c = rows.codes + static_cast<size_t>(step) * 128u;
#pragma unroll
    for (int q = 0; q < 4; ++q) ldg256_stream(c + q * rows.row_stride32, st.c[q], rows.policy);
    st.sc = ldg128_stream(rows.scales + static_cast<size_t>(tile) * 512u, rows.policy);
  } else {
    zero_stage(st);
  }
}

// Eight E2M1 codes (one word) to four half2 on the integer pipe alone. A code's three magnitude
// bits and its sign are placed in a byte as [s 0 0 0 e1 e0 m 0]: read as the high byte of an fp16
// (low byte zero) that is the code's value times 2^-14 exactly, the subnormal code 0.5 included.
// The registers pair the codes (0,2) (4,6) (1,3) (5,7); the activation fragments of such a word
// are stored in the same order.
__device__ __forceinline__ void e2m1x8_to_half2x4_alu(uint32_t w, uint32_t (&h)[4]) {
  const uint32_t even = ((w << 1) & 0x0E0E0E0Eu) | ((w << 4) & 0x80808080u);  // codes 0,2,4,6
  const uint32_t odd = ((w >> 3) & 0x0E0E0E0Eu) | (w & 0x80808080u);          // codes 1,3,5,7
  h[0] = __byte_perm(even, 0u, 0x1404);
  h[1] = __byte_perm(even, 0u, 0x3424);
  h[2] = __byte_perm(odd, 0u, 0x1404);
  h[3] = __byte_perm(odd, 0u, 0x3424);
}

// One K step of a warp: 4 rows x 64 weights per lane against the prepared activations of the
// step (`xs_step`: [8 words][NT tiles][32 slots] uint4, slot = lane ^ (word << 2) ^ ((word >> 1) & 3)).
//
// The hardware E2M1 conversion runs on the quarter-rate special-function pipe, which alone would
// cap the kernel below the HBM rate, so only the first XU of a row's 8 words take it; the others
// are decoded with integer operations. Both kinds end as (code * scale * 2^-7) in fp16: the
// converted words are multiplied by scale * 2^-7, the integer-decoded ones (already times 2^-14)
// by scale * 2^7, all exact; the epilogue multiplies by 2^7.
template <int NT, int XU>
__device__ __forceinline__ void compute_stage(const Stage &st, const uint4 *xs_step, int lane, float (&acc)[2][NT][4]) {
  uint32_t sp_lo[4][2], sp_hi[4][2];
  {
    const uint32_t w[4] = {st.sc.x, st.sc.y, st.sc.z, st.sc.w};
    const uint32_t down = 0x20002000u;  // half2(2^-7, 2^-7)
    const uint32_t up = 0x58005800u;    // half2(2^7, 2^7)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t a = e4m3x2_to_half2(w[q] & 0xFFFFu), b = e4m3x2_to_half2(w[q] >> 16);
      sp_lo[q][0] = hmul2_u32(a, down);
      sp_lo[q][1] = hmul2_u32(b, down);
      sp_hi[q][0] = hmul2_u32(a, up);
      sp_hi[q][1] = hmul2_u32(b, up);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint32_t h[4][4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t pair;
      if (i < XU) {
        e2m1x8_to_half2x4(st.c[q][i], h[q]);
        pair = sp_lo[q][i >> 2];
      } else {
        e2m1x8_to_half2x4_alu(st.c[q][i], h[q]);
        pair = sp_hi[q][i >> 2];
      }
      const __half2 p2 = *reinterpret_cast<const __half2 *>(&pair);
      const __half2 sb = ((i >> 1) & 1) ? __high2half2(p2) : __low2half2(p2);
      const uint32_t sbu = *reinterpret_cast<const uint32_t *>(&sb);
#pragma unroll
      for (int b = 0; b < 4; ++b) h[q][b] = hmul2_u32(h[q][b], sbu);
    }
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) {
      const uint4 v = xs_step[(i * NT + tt) * 32 + ((lane ^ (i << 2)) ^ ((i >> 1) & 3))];
      mma_f16_f32(acc[0][tt], h[0][0], h[1][0], h[0][1], h[1][1], v.x, v.y);
      mma_f16_f32(acc[1][tt], h[2][0], h[3][0], h[2][1], h[3][1], v.x, v.y);
      mma_f16_f32(acc[0][tt], h[0][2], h[1][2], h[0][3], h[1][3], v.z, v.w);
      mma_f16_f32(acc[1][tt], h[2][2], h[3][2], h[2][3], h[3][3], v.z, v.w);
    }
  }
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
// float4 at the same shared-memory offset in CTA `rank` of this cluster.
__device__ __forceinline__ float4 ld_cluster_f4(const void *local_smem, uint32_t rank) {
  const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(local_smem));
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

__device__ __forceinline__ float silu_f32(float v) { return v / (1.0f + __expf(-v)); }

// Eight BF16 values (one 16-byte chunk) times a power of two, as fp16, in the order the MMA
// fragments of word `i` want: natural pairs for a hardware-converted word, the pairs (0,2) (4,6)
// (1,3) (5,7) for an integer-decoded one.
template <int XU>
__device__ __forceinline__ uint4 convert_chunk(const uint4 v, float scale, int i) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  float f[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = bf16_bits_to_f32(w[j] & 0xFFFFu) * scale;
    f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u) * scale;
  }
  __half2 r[4];
  if (i < XU) {
    r[0] = __floats2half2_rn(f[0], f[1]);
    r[1] = __floats2half2_rn(f[2], f[3]);
    r[2] = __floats2half2_rn(f[4], f[5]);
    r[3] = __floats2half2_rn(f[6], f[7]);
  } else {
    r[0] = __floats2half2_rn(f[0], f[2]);
    r[1] = __floats2half2_rn(f[4], f[6]);
    r[2] = __floats2half2_rn(f[1], f[3]);
    r[3] = __floats2half2_rn(f[5], f[7]);
  }
  return make_uint4(*reinterpret_cast<uint32_t *>(&r[0]), *reinterpret_cast<uint32_t *>(&r[1]),
                    *reinterpret_cast<uint32_t *>(&r[2]), *reinterpret_cast<uint32_t *>(&r[3]));
}

// The largest magnitude among eight BF16 values and a running pair of maxima, as bit patterns: the
// magnitudes of finite BF16 numbers order like their bits read as unsigned integers, so the maximum
// is two 16-bit integer maxima per word (infinities and NaNs come out on top and are caught by the
// caller). `run` holds one maximum per half.
__device__ __forceinline__ uint32_t chunk_amax_bits(const uint4 v, uint32_t run) {
  run = __vmaxu2(run, v.x & 0x7FFF7FFFu);
  run = __vmaxu2(run, v.y & 0x7FFF7FFFu);
  run = __vmaxu2(run, v.z & 0x7FFF7FFFu);
  run = __vmaxu2(run, v.w & 0x7FFF7FFFu);
  return run;
}

// The power of two that brings a token's largest magnitude (BF16 bits, sign cleared) into
// [2^13, 2^14): 14 minus the exponent frexp would report, held to what a float can carry; zero for
// an all-zero slice and for one that holds an infinity or a NaN.
__device__ __forceinline__ int amax_shift(uint32_t amax_bits) {
  if (amax_bits == 0u || amax_bits >= 0x7F80u) return 0;
  const int e8 = static_cast<int>(amax_bits >> 7);  // 0 for a subnormal maximum: far below every clamp
  return e8 == 0 ? 126 : max(-126, min(126, 140 - e8));
}
__device__ __forceinline__ float pow2f(int e) { return __uint_as_float(static_cast<uint32_t>(e + 127) << 23); }  // e in [-126, 127]

constexpr int kNoShiftYet = 1 << 20;  // a token whose chunks so far held nothing to scale
constexpr int kPrepRegs = 5;  // chunks a lane keeps in registers between the amax and the store

// Rewrites steps [cb, ce) of the activations as scaled fp16 B fragments. Warp w prepares token
// slots w, w + 8, ...; a lane owns one 16-byte chunk of every step (t: the lane quarter that will
// read it, i: the word it multiplies). The slot's inverse scale goes to
// inv_s, its scale to scale_s.
template <int NT, int XU, bool CHUNKED>
__device__ __forceinline__ void prepare_activations(const GemvParams &p, int cb, int ce, uint4 *xs, float *inv_s,
                                                    float *scale_s, int *low_s, bool first, int warp, int lane,
                                                    int trace_launch) {
  const int nsteps = ce - cb;
  // Lane l takes chunk l of a step: t = l / 8 is the lane quarter that will read it, i = l % 8 the
  // word it multiplies. (Dealing the chunks so that the fragment stores avoid their four-way bank
  // conflict scatters each quarter-warp's global load over four lines, and measured slower.)
  const int t = lane >> 3, i = lane & 7;
  const int chunk = lane;
  // Fragment slot of lane (g = warp, t), swizzled by the word i in both fields: the token by i (a
  // warp's 32 reads of one word fall in 32 different slots) and the lane quarter by bits 1..2 of i
  // (the eight lanes of one phase of this 16-byte store - one t, eight words - fall in the eight
  // different bank groups instead of two).
  const int slot = ((warp ^ i) << 2) | (t ^ ((i >> 1) & 3));
#pragma unroll
  for (int tt = 0; tt < NT; ++tt) {
    const uint32_t tok = static_cast<uint32_t>(tt * 8 + warp);
    const bool live = tok < p.tokens;
    const uint4 *src =
        reinterpret_cast<const uint4 *>(p.x + static_cast<size_t>(tok) * p.k + static_cast<size_t>(cb) * 256u) + chunk;
    // steps whose chunk for this lane lies inside K
    const int inside = (static_cast<int>(p.k / 8u) - cb * 32 - chunk + 31) / 32;
    const int valid = live ? min(nsteps, max(inside, 0)) : 0;
    uint4 *dst = xs + tt * 32 + slot + static_cast<size_t>(i) * NT * 32;
    uint32_t amax = 0u;  // one running maximum per 16-bit half
    int prov = 0;        // the provisional shift of a long slice
    uint4 held[kPrepRegs];
    const bool hold = nsteps <= kPrepRegs;
    if (hold) {
#pragma unroll
      for (int m = 0; m < kPrepRegs; ++m) {
        held[m] = make_uint4(0u, 0u, 0u, 0u);
        if (m < valid) held[m] = ldg128_coherent(src + m * 32);
      }
#pragma unroll
      for (int m = 0; m < kPrepRegs; ++m) amax = chunk_amax_bits(held[m], amax);
    } else {
      // A longer slice does not fit in registers beside the two weight stages. It is converted in
      // one pass at a provisional scale taken from its first four steps (their maximum brought into
      // [2^9, 2^10), which leaves the rest of the slice room to be 32 times larger), the slice's own
      // maximum being gathered on the way; only a slice whose maximum ends outside what fp16
      // carries well at that scale is converted again below.
      float pscale = 1.0f;
      for (int m0 = 0; m0 < nsteps; m0 += 4) {
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[j] = make_uint4(0u, 0u, 0u, 0u);
          if (m0 + j < valid) v[j] = ldg128_coherent(src + (m0 + j) * 32);
        }
        uint32_t bm = 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) bm = chunk_amax_bits(v[j], bm);
        amax = __vmaxu2(amax, bm);
        if (m0 == 0) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) bm = __vmaxu2(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, o));
          prov = max(-126, amax_shift(max(bm & 0xFFFFu, bm >> 16)) - 4);
          pscale = pow2f(prov);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (m0 + j < nsteps) dst[static_cast<size_t>(m0 + j) * 8 * NT * 32] = convert_chunk<XU>(v[j], pscale, i);
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = __vmaxu2(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if (tt == 0) GEMV_TRACE(8);
    const uint32_t top = max(amax & 0xFFFFu, amax >> 16);
    // The accumulators are carried from one chunk of a slice into the next chunk's units. A chunk
    // far smaller than an earlier one of its token must not pull them up by its whole ratio (the
    // sums gathered so far would leave the range of a float): its shift stays within 64 of the
    // lowest shift the token has had, and what it then loses lies 2^-50 below the earlier sums.
    int cap = 126, low = kNoShiftYet;
    if (CHUNKED && !first) {
      low = low_s[tt * 8 + warp];
      if (low != kNoShiftYet) cap = min(126, low + 64);
      __syncwarp();  // every lane has read the token's lowest shift before lane 0 replaces it
    }
    int shift = min(amax_shift(top), cap);
    bool again = false;
    if (!hold) {
      // the maximum lies in [2^e, 2^(e + 1)) at the provisional scale
      const int e = static_cast<int>(top >> 7) - 127 + prov;
      if (prov <= cap && (top == 0u || (top < 0x7F80u && e >= 5 && e <= 14))) shift = prov;
      else again = true;
    }
    if (CHUNKED && lane == 0) low_s[tt * 8 + warp] = (top == 0u || top >= 0x7F80u) ? low : min(low, shift);
    const float scale = pow2f(shift);
    if (lane == 0) {
      inv_s[tt * 8 + warp] = live ? pow2f(-shift) : 0.0f;
      scale_s[tt * 8 + warp] = scale;
    }
    if (hold) {
#pragma unroll
      for (int m = 0; m < kPrepRegs; ++m) {
        if (m < nsteps) dst[static_cast<size_t>(m) * 8 * NT * 32] = convert_chunk<XU>(held[m], scale, i);
      }
    } else if (again) {
      for (int m0 = 0; m0 < nsteps; m0 += 4) {
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[j] = make_uint4(0u, 0u, 0u, 0u);
          if (m0 + j < valid) v[j] = ldg128_coherent(src + (m0 + j) * 32);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (m0 + j < nsteps) dst[static_cast<size_t>(m0 + j) * 8 * NT * 32] = convert_chunk<XU>(v[j], scale, i);
        }
      }
    }
  }
}

template <int NT, int XU, bool CHUNKED>
__global__ void __launch_bounds__(kThreads, NT <= 2 ? 2 : 1) nvfp4_gemv_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  GEMV_TRACE_BEGIN(p.epilogue);
  const int rm = static_cast<int>(p.rm), kw_count = kWarps / rm;
  const int rgl = warp % rm, kw = warp / rm;
  const uint32_t kc = p.kc;
  const uint32_t rank = cluster_ctarank();

  // shared-memory carve-up (sizes fixed by the host from the same parameters)
  uint4 *xs = reinterpret_cast<uint4 *>(smem_raw);
  float4 *red = reinterpret_cast<float4 *>(smem_raw + static_cast<size_t>(p.xs_steps) * 4096u * NT);
  float4 *part = red + static_cast<size_t>(kw_count - 1) * rm * 2 * NT * 32;
  float *inv_s = reinterpret_cast<float *>(part + static_cast<size_t>(rm) * 2 * NT * 32);
  float *scale_s = inv_s + 8 * NT;
  int *low_s = reinterpret_cast<int *>(scale_s + 8 * NT);

  // which weight of the group this CTA serves
  uint32_t wi = 0;
#pragma unroll
  for (uint32_t i = 1; i < kMaxGroup; ++i) {
    if (i < p.count && blockIdx.x >= p.w[i].block_begin) wi = i;
  }
  const GemvWeight &W = p.w[wi];
  const uint32_t row_block = (blockIdx.x - W.block_begin) / kc;
  const bool swiglu = (p.epilogue & kEpilogueSwiglu) != 0u;
  const uint32_t groups_total = W.n / 32u;
  uint32_t group;  // 32-row group of this warp
  bool active;
  if (swiglu) {  // the first half of the CTA's groups are gate rows, the second half the matching up rows
    const uint32_t half = static_cast<uint32_t>(rm) / 2u;
    const uint32_t idx = row_block * half + (static_cast<uint32_t>(rgl) % half);
    active = idx < groups_total / 2u;
    group = static_cast<uint32_t>(rgl) < half ? idx : groups_total / 2u + idx;
  } else {
    group = row_block * rm + rgl;
    active = group < groups_total;
  }
  const uint32_t m_tile = group >> 2, jq = group & 3u;
  const uint32_t scale_tiles = p.k / 64u;

  WarpRows rows;
  rows.active = active;
  rows.policy = l2_evict_first_policy();
  const uint32_t row0 = m_tile * 128u + jq * 8u + g;
  rows.codes = W.codes + static_cast<size_t>(row0) * (p.k / 2u) + t * 32;
  rows.scales = W.scales + static_cast<size_t>(m_tile) * scale_tiles * 512u + (jq * 8u + g) * 16u;
  rows.row_stride32 = static_cast<size_t>(32u) * (p.k / 2u);

  // K slice of this CTA, steps interleaved over the CTA's kw_count warp columns
  const int c0 = static_cast<int>(static_cast<uint64_t>(p.ksteps) * rank / kc);
  const int c1 = static_cast<int>(static_cast<uint64_t>(p.ksteps) * (rank + 1) / kc);
  const int ch = static_cast<int>(p.xs_steps);
  Stage st0, st1;
  int s = c0 + kw;
  load_stage(st0, rows, s, c1, t, scale_tiles);
  load_stage(st1, rows, s + kw_count, c1, t, scale_tiles);

  // The weights above never depend on the previous kernel; the activations may.
  GEMV_TRACE(1);
  griddep_launch_dependents();
  griddep_wait();
  GEMV_TRACE(2);
  if (p.wait.flags_peers != nullptr) {
    // x lies in a buffer every rank's previous product stored its columns into. The barrier between
    // the ranks rides here, in the consumer's first instructions, instead of in a launch of its own:
    // this rank's product has finished and its stores (peer stores included) are complete - that is
    // what griddep_wait / stream order gives - so the grid's first CTA publishes barrier number
    // state[1] + 1 in this rank's slot of every rank's flag array, and every CTA waits until all
    // slots of its own rank's array have reached it. The last CTA through counts the barrier.
    if (warp == 0) {
      const uint32_t epoch = ld_acquire_gpu(p.wait.state + 1) + 1u;
      if (blockIdx.x == 0 && static_cast<uint32_t>(lane) < p.wait.peers) {
        __threadfence_system();
        st_release_sys(p.wait.flags_peers[lane] + p.wait.rank, epoch);
      }
      peer_wait_flags(p.wait.flags_peers, p.wait.state, p.wait.peers, p.wait.rank, p.wait.polls, epoch, lane);
      if (lane == 0 && atomicAdd(p.wait.state + 2, 1u) == gridDim.x - 1u) {   // every CTA has read state[1]
        atomicExch(p.wait.state + 2, 0u);
        atomicAdd(p.wait.state + 1, 1u);
      }
    }
    __syncthreads();
  }

  // Accumulators live in the units of the current chunk's per-token scale; at a chunk boundary
  // they are carried into the next chunk's units by an exact power-of-two factor.
  float tot[2][NT][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int tt = 0; tt < NT; ++tt)
#pragma unroll
      for (int e = 0; e < 4; ++e) tot[a][tt][e] = 0.0f;

  for (int cb = c0; cb < c1; cb += ch) {
    const int ce = min(cb + ch, c1);
    float carry[NT][2];
    if (CHUNKED && cb != c0) {
#pragma unroll
      for (int tt = 0; tt < NT; ++tt) {
        carry[tt][0] = inv_s[tt * 8 + 2 * t];
        carry[tt][1] = inv_s[tt * 8 + 2 * t + 1];
      }
      __syncthreads();  // the previous chunk's fragments and scales are no longer read
    }
    prepare_activations<NT, XU, CHUNKED>(p, cb, ce, xs, inv_s, scale_s, low_s, cb == c0, warp, lane, cb == c0 ? trace_launch : -1);
    if (cb == c0) GEMV_TRACE(9);
    __syncthreads();
    if (cb == c0) GEMV_TRACE(3);
    if (CHUNKED && cb != c0) {
#pragma unroll
      for (int tt = 0; tt < NT; ++tt) {
        const float f0 = carry[tt][0] * scale_s[tt * 8 + 2 * t], f1 = carry[tt][1] * scale_s[tt * 8 + 2 * t + 1];
#pragma unroll
        for (int a = 0; a < 2; ++a) {
          tot[a][tt][0] *= f0;
          tot[a][tt][1] *= f1;
          tot[a][tt][2] *= f0;
          tot[a][tt][3] *= f1;
        }
      }
    }
    while (s < ce) {
      compute_stage<NT, XU>(st0, xs + static_cast<size_t>(s - cb) * 8 * NT * 32, lane, tot);
      if (s + kw_count < ce) {
        load_stage(st0, rows, s + 2 * kw_count, c1, t, scale_tiles);
        compute_stage<NT, XU>(st1, xs + static_cast<size_t>(s + kw_count - cb) * 8 * NT * 32, lane, tot);
        load_stage(st1, rows, s + 3 * kw_count, c1, t, scale_tiles);
        s += 2 * kw_count;
      } else {
        st0 = st1;
        load_stage(st1, rows, s + 2 * kw_count, c1, t, scale_tiles);
        s += kw_count;
      }
    }
  }
  GEMV_TRACE(4);
  // back to the activations' own units
#pragma unroll
  for (int tt = 0; tt < NT; ++tt) {
    const float i0 = inv_s[tt * 8 + 2 * t], i1 = inv_s[tt * 8 + 2 * t + 1];
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      tot[a][tt][0] *= i0;
      tot[a][tt][1] *= i1;
      tot[a][tt][2] *= i0;
      tot[a][tt][3] *= i1;
    }
  }
  // ---- K reduction inside the CTA: columns kw = 1.. hand their sums to column 0, fixed order ----
  if (kw > 0) {
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int tt = 0; tt < NT; ++tt)
        red[(((kw - 1) * rm + rgl) * 2 + a) * NT * 32 + tt * 32 + lane] =
            make_float4(tot[a][tt][0], tot[a][tt][1], tot[a][tt][2], tot[a][tt][3]);
  }
  __syncthreads();
  if (kw == 0) {
    for (int k2 = 1; k2 < kw_count; ++k2) {
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) {
          const float4 v = red[(((k2 - 1) * rm + rgl) * 2 + a) * NT * 32 + tt * 32 + lane];
          tot[a][tt][0] += v.x;
          tot[a][tt][1] += v.y;
          tot[a][tt][2] += v.z;
          tot[a][tt][3] += v.w;
        }
    }
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int tt = 0; tt < NT; ++tt)
        part[((rgl * 2 + a) * NT + tt) * 32 + lane] = make_float4(tot[a][tt][0], tot[a][tt][1], tot[a][tt][2], tot[a][tt][3]);
  }

  // ---- K reduction across the cluster, then the epilogue, the items dealt over ranks and warps ----
  GEMV_TRACE(5);
  cluster_sync_all();
  GEMV_TRACE(6);
  const int out_groups = swiglu ? rm / 2 : rm;
  const int items = out_groups * 2 * NT;
  const float coef = W.inv_dw * 128.0f;  // the operands carried 2^-7
  for (int f = static_cast<int>(rank) + static_cast<int>(kc) * warp; f < items; f += static_cast<int>(kc) * kWarps) {
    const int og = f / (2 * NT), a = (f / NT) & 1, tt = f % NT;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f), sum_up = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t r = 0; r < kc; ++r) {
      const float4 v = ld_cluster_f4(&part[((og * 2 + a) * NT + tt) * 32 + lane], r);
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
      if (swiglu) {
        const float4 u = ld_cluster_f4(&part[(((og + out_groups) * 2 + a) * NT + tt) * 32 + lane], r);
        sum_up.x += u.x; sum_up.y += u.y; sum_up.z += u.z; sum_up.w += u.w;
      }
    }
    const uint32_t og_group = swiglu ? row_block * out_groups + og : row_block * rm + og;
    const uint32_t og_limit = swiglu ? groups_total / 2u : groups_total;
    if (og_group >= og_limit) continue;
    const uint32_t out_row = (og_group >> 2) * 128u + (og_group & 3u) * 8u + g + 64u * a;  // q = 2a, 2a + 1
    const uint32_t tok0 = tt * 8 + 2 * t;
    float v[4] = {sum.x * coef, sum.y * coef, sum.z * coef, sum.w * coef};
    if (swiglu) {
      const float u[4] = {sum_up.x * coef, sum_up.y * coef, sum_up.z * coef, sum_up.w * coef};
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = silu_f32(v[e]) * u[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t tok = tok0 + (e & 1);
      const uint32_t row = out_row + (e >> 1) * 32u;
      if (tok >= p.tokens) continue;
      const size_t at = static_cast<size_t>(tok) * W.ldy + row;
      // one buffer, or the same value into every rank's buffer (peer stores over NVLink)
      for (uint32_t pp = 0; pp < W.peers; ++pp) {
        if (p.epilogue & kEpilogueF32) {
          float *y = static_cast<float *>(W.y[pp]);
          y[at] = (p.epilogue & kEpilogueAdd) ? y[at] + v[e] : v[e];
        } else {
          __nv_bfloat16 *y = static_cast<__nv_bfloat16 *>(W.y[pp]);
          const float r = (p.epilogue & kEpilogueAdd) ? v[e] + __bfloat162float(y[at]) : v[e];
          y[at] = __float2bfloat16_rn(r);
        }
      }
    }
  }
  cluster_sync_all();  // no CTA leaves while a peer may still read its partial sums
}

constexpr size_t kGemvMaxSmem = 160 * 1024;

size_t gemv_smem_bytes(int nt, int rm, int xs_steps) {
  const int kw_count = kWarps / rm;
  return static_cast<size_t>(xs_steps) * 4096u * nt + static_cast<size_t>(kw_count - 1) * rm * 2 * nt * 32 * 16 +
         static_cast<size_t>(rm) * 2 * nt * 32 * 16 + static_cast<size_t>(24 * nt) * 4;
}

template <int NT, int XU, bool CHUNKED>
cudaError_t launch_gemv(const GemvParams &p, uint32_t ctas, size_t smem, cudaStream_t stream, bool pdl) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(ctas, 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.kc;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pdl ? 2 : 1;
  return cudaLaunchKernelEx(&config, nvfp4_gemv_kernel<NT, XU, CHUNKED>, p);
}

template <int NT, int XU>
cudaError_t set_smem_attr() {
  cudaError_t err = cudaFuncSetAttribute(nvfp4_gemv_kernel<NT, XU, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kGemvMaxSmem));
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(nvfp4_gemv_kernel<NT, XU, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kGemvMaxSmem));
  return err;
}

template <int XU>
cudaError_t set_smem_attrs() {
  cudaError_t err = set_smem_attr<1, XU>();
  if (err == cudaSuccess) err = set_smem_attr<2, XU>();
  if (err == cudaSuccess) err = set_smem_attr<4, XU>();
  return err;
}

template <int XU, bool CHUNKED>
cudaError_t launch_for_nt(int nt, const GemvParams &p, uint32_t ctas, size_t smem, cudaStream_t stream, bool pdl) {
  if (nt == 1) return launch_gemv<1, XU, CHUNKED>(p, ctas, smem, stream, pdl);
  if (nt == 2) return launch_gemv<2, XU, CHUNKED>(p, ctas, smem, stream, pdl);
  return launch_gemv<4, XU, CHUNKED>(p, ctas, smem, stream, pdl);
}

// `chunked`: some CTA's K slice is longer than the fragments the shared memory holds at a time.
template <int XU>
cudaError_t launch_for_slice(bool chunked, int nt, const GemvParams &p, uint32_t ctas, size_t smem, cudaStream_t stream, bool pdl) {
  return chunked ? launch_for_nt<XU, true>(nt, p, ctas, smem, stream, pdl) : launch_for_nt<XU, false>(nt, p, ctas, smem, stream, pdl);
}

}  // namespace

#ifdef B200Q_GEMV_TRACE
}  // namespace b200q
// Copies the stamps out ([128][512][8] u64) and clears them for the next window.
extern "C" int32_t b200q_debug_gemv_trace(void *out, uint64_t bytes) {
  if (out == nullptr || bytes != sizeof(b200q::g_trace)) return -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(out, b200q::g_trace, bytes) != cudaSuccess) return -1;
  void *stamps = nullptr;
  if (cudaGetSymbolAddress(&stamps, b200q::g_trace) != cudaSuccess) return -1;
  if (cudaMemset(stamps, 0, sizeof(b200q::g_trace)) != cudaSuccess) return -1;
  return 0;
}
namespace b200q {
#endif

int32_t gemv_prepare(ErrorSlot &slot) {
  cudaError_t err = set_smem_attrs<0>();
  if (err == cudaSuccess) err = set_smem_attrs<2>();
  if (err == cudaSuccess) err = set_smem_attrs<3>();
  if (err == cudaSuccess) err = set_smem_attrs<4>();
  if (err == cudaSuccess) err = set_smem_attrs<8>();
  if (err != cudaSuccess) return fail(slot, "nvfp4 decode kernel attributes: %s", cudaGetErrorString(err));
  // How many CTAs the device keeps resident for each cluster size: clusters are placed inside one
  // GPC, so the count is not simply slots / size. The plan uses it to tell one wave from two.
  DeviceState *dev = device_state(slot);
  if (dev == nullptr) return -1;
  for (int kc = 1; kc <= 8; ++kc) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(kc) * 1024u, 1, 1);
    config.blockDim = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = 56 * 1024;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(kc);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, nvfp4_gemv_kernel<1, 8, false>, &config) == cudaSuccess && clusters > 0) {
      dev->gemv_slots[kc] = clusters * kc;
    } else {
      dev->gemv_slots[kc] = 0;
      (void)cudaGetLastError();
    }
  }
  return 0;
}

// Chooses rows per CTA (rm groups of 32), the cluster size kc and the fragment buffer depth for a
// launch over `groups` 32-row groups and `ksteps` steps of 256 along K.
GemvPlan gemv_plan(const DeviceState &dev, uint32_t groups, uint32_t ksteps, int nt, bool swiglu) {
  const double slots = static_cast<double>(dev.sm_count) * (nt <= 2 ? dev.gemv_ctas_per_sm : 1);
  const int rm_min = swiglu ? 2 : 1;
  GemvPlan best = {};
  // pass 0 honours the B200Q_GEMV_RM / B200Q_GEMV_KC overrides; if they admit nothing for this
  // shape, pass 1 ignores them
  for (int pass = 0; pass < 2 && best.rm == 0; ++pass) {
    double best_cost = 1e30;
    for (int rm = 8; rm >= rm_min; rm >>= 1) {
      for (int kc = 1; kc <= 8; ++kc) {
        if (pass == 0 && dev.gemv_rb > 0 && rm != dev.gemv_rb) continue;
        if (pass == 0 && dev.gemv_kc > 0 && kc != dev.gemv_kc) continue;
        if (static_cast<uint32_t>(kc) > ksteps) continue;
        const int kwc = kWarps / rm;
        const uint32_t out_groups = swiglu ? groups / 2 : groups;
        const uint32_t rows_per_cta = swiglu ? rm / 2 : rm;
        const uint32_t row_blocks = (out_groups + rows_per_cta - 1) / rows_per_cta;
        const double ctas = static_cast<double>(row_blocks) * kc;
        const double resident = nt <= 2 && dev.gemv_slots[kc] > 0 ? static_cast<double>(dev.gemv_slots[kc]) : slots;
        const double waves = ceil(ctas / resident);
        const double slice = ceil(static_cast<double>(ksteps) / kc);
        const double steps = ceil(slice / kwc);
        // fitted on B200 (microseconds per launch): a warp's step costs about 1.6, a step of the
        // CTA's activation slice 0.3 per token tile, a wave of CTAs 3, the launch itself 2.4, and every
        // CTA of a cluster 0.35: clusters are placed inside one GPC, so the wider they are the more
        // SMs stay empty and the later the last CTA starts (phase stamps of the four configs[1] calls)
        const double cost = waves * (1.57 * steps + 0.3 * nt * slice + 3.0) + 2.4 + 0.35 * kc;
        if (cost < best_cost) {
          best_cost = cost;
          best.rm = rm;
          best.kc = kc;
          best.row_blocks = row_blocks;
        }
      }
    }
  }
  const uint32_t slice = (ksteps + best.kc - 1) / best.kc;
  const uint32_t cap = 16u / static_cast<uint32_t>(nt);  // 64 KB of fragments
  best.xs_steps = slice < cap ? slice : cap;
  return best;
}

int32_t gemv_launch(ErrorSlot &slot, const DeviceState &dev, GemvParams &p, int nt, const GemvPlan &plan, uint32_t ctas,
                    cudaStream_t stream) {
  p.rm = plan.rm;
  p.kc = plan.kc;
  p.xs_steps = plan.xs_steps;
#ifdef B200Q_GEMV_TRACE
  static uint32_t trace_counter = 0;
  p.epilogue = (p.epilogue & 0xFFFFu) | ((trace_counter++ & 127u) << 16);
#endif
  const size_t smem = gemv_smem_bytes(nt, plan.rm, plan.xs_steps);
  const bool chunked = (p.ksteps + plan.kc - 1u) / plan.kc > plan.xs_steps;
  if (smem > kGemvMaxSmem) return fail(slot, "nvfp4 decode: %zu bytes of shared memory exceed the kernel's limit", smem);
  cudaError_t err;
  const bool pdl = dev.pdl != 0;
  switch (dev.gemv_xu) {  // words per row of 8 that take the hardware E2M1 conversion
    case 0: err = launch_for_slice<0>(chunked, nt, p, ctas, smem, stream, pdl); break;
    case 2: err = launch_for_slice<2>(chunked, nt, p, ctas, smem, stream, pdl); break;
    case 4: err = launch_for_slice<4>(chunked, nt, p, ctas, smem, stream, pdl); break;
    case 8: err = launch_for_slice<8>(chunked, nt, p, ctas, smem, stream, pdl); break;
    default: err = launch_for_slice<3>(chunked, nt, p, ctas, smem, stream, pdl); break;
  }
  if (err != cudaSuccess) return fail(slot, "nvfp4 decode launch: %s", cudaGetErrorString(err));
  return 0;
}

}  // namespace b200q
