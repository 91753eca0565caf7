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
//  * Codes go to fp16 with the hardware E2M1 conversion and are multiplied by their E4M3 scale in
//    fp16 (exact: at most 6 significant bits, magnitude within [2^-10, 2688]). The products are
//    the A fragments of mma.sync m16n8k16 (fp16 in, fp32 accumulate); the tokens are the MMA's N,
//    so 1 and 8 tokens cost the same weight traffic and the same decode. The order of k inside an
//    MMA is permuted (lane t supplies the k of its own 64-weight chunk): a sum does not care, and
//    both operands use the same permutation.
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
  bool active;
};

__device__ __forceinline__ void load_stage(Stage &st, const WarpRows &rows, int step, int c1, int lane_t,
                                           uint32_t scale_tiles) {
  const uint32_t tile = static_cast<uint32_t>(step) * 4u + static_cast<uint32_t>(lane_t);
  if (rows.active && step < c1 && tile < scale_tiles) {
    const uint8_t *c = rows.codes + static_cast<size_t>(step) * 128u;
#pragma unroll
    for (int q = 0; q < 4; ++q) ldg256_stream(c + q * rows.row_stride32, st.c[q]);
    st.sc = ldg128_stream(rows.scales + static_cast<size_t>(tile) * 512u);
  } else {
    zero_stage(st);
  }
}

// One K step of a warp: 4 rows x 64 weights per lane against the prepared activations of the
// step (`xs_step`: [8 chunks][NT tiles][32 lanes] uint4).
template <int NT>
__device__ __forceinline__ void compute_stage(const Stage &st, const uint4 *xs_step, int lane, float (&acc)[2][NT][4]) {
  uint32_t sp[4][2];
  {
    const uint32_t w[4] = {st.sc.x, st.sc.y, st.sc.z, st.sc.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      sp[q][0] = e4m3x2_to_half2(w[q] & 0xFFFFu);
      sp[q][1] = e4m3x2_to_half2(w[q] >> 16);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint32_t h[4][4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      e2m1x8_to_half2x4(st.c[q][i], h[q]);
      const uint32_t pair = sp[q][i >> 2];
      const __half2 p2 = *reinterpret_cast<const __half2 *>(&pair);
      const __half2 sb = ((i >> 1) & 1) ? __high2half2(p2) : __low2half2(p2);
      const uint32_t sbu = *reinterpret_cast<const uint32_t *>(&sb);
#pragma unroll
      for (int b = 0; b < 4; ++b) h[q][b] = hmul2_u32(h[q][b], sbu);
    }
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) {
      const uint4 v = xs_step[(i * NT + tt) * 32 + lane];
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

// Rewrites steps [cb, ce) of the activations as scaled fp16 B fragments. Warp w prepares token
// slots w, w + 8, ...; the slot's inverse scale goes to inv_s.
template <int NT>
__device__ __forceinline__ void prepare_activations(const GemvParams &p, int cb, int ce, uint4 *xs, float *inv_s,
                                                    float *scale_s, int warp, int lane) {
  const int chunks = (ce - cb) * 32;  // 16-byte chunks of 8 values per token
#pragma unroll
  for (int tt = 0; tt < NT; ++tt) {
    const uint32_t tok = static_cast<uint32_t>(tt * 8 + warp);
    const bool live = tok < p.tokens;
    const uint4 *src = reinterpret_cast<const uint4 *>(p.x + static_cast<size_t>(tok) * p.k + static_cast<size_t>(cb) * 256u);
    const int valid_chunks = live ? min(chunks, static_cast<int>((p.k - static_cast<uint32_t>(cb) * 256u) / 8u)) : 0;
    float amax = 0.0f;
    for (int c = lane; c < valid_chunks; c += 32) {
      const uint4 v = ldg128_coherent(src + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        amax = fmaxf(amax, fabsf(bf16_bits_to_f32(w[j] & 0xFFFFu)));
        amax = fmaxf(amax, fabsf(__uint_as_float(w[j] & 0xFFFF0000u)));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    int shift = 0;
    if (amax > 0.0f && amax <= 3.0e38f) {
      int e;
      (void)frexpf(amax, &e);  // amax in [2^(e-1), 2^e)
      shift = max(-126, min(126, 14 - e));
    }
    const float scale = ldexpf(1.0f, shift);
    if (lane == 0) {
      inv_s[tt * 8 + warp] = live ? ldexpf(1.0f, -shift) : 0.0f;
      scale_s[tt * 8 + warp] = scale;
    }
    for (int c = lane; c < chunks; c += 32) {
      uint4 out = make_uint4(0u, 0u, 0u, 0u);
      if (c < valid_chunks) {
        const uint4 v = ldg128_coherent(src + c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = bf16_bits_to_f32(w[j] & 0xFFFFu) * scale;
          const float hi = __uint_as_float(w[j] & 0xFFFF0000u) * scale;
          const __half2 hh = __floats2half2_rn(lo, hi);
          r[j] = *reinterpret_cast<const uint32_t *>(&hh);
        }
        out = make_uint4(r[0], r[1], r[2], r[3]);
      }
      // chunk c = step 32 s + 8 t + i  ->  fragment slot [s][i][tt][g = warp][t]
      const int s = c >> 5, t = (c >> 3) & 3, i = c & 7;
      xs[((s * 8 + i) * NT + tt) * 32 + warp * 4 + t] = out;
    }
  }
}

template <int NT>
__global__ void __launch_bounds__(kThreads, NT <= 2 ? 2 : 1) nvfp4_gemv_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
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
  griddep_launch_dependents();
  griddep_wait();

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
    if (cb != c0) {
#pragma unroll
      for (int tt = 0; tt < NT; ++tt) {
        carry[tt][0] = inv_s[tt * 8 + 2 * t];
        carry[tt][1] = inv_s[tt * 8 + 2 * t + 1];
      }
      __syncthreads();  // the previous chunk's fragments and scales are no longer read
    }
    prepare_activations<NT>(p, cb, ce, xs, inv_s, scale_s, warp, lane);
    __syncthreads();
    if (cb != c0) {
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
      compute_stage<NT>(st0, xs + static_cast<size_t>(s - cb) * 8 * NT * 32, lane, tot);
      if (s + kw_count < ce) {
        load_stage(st0, rows, s + 2 * kw_count, c1, t, scale_tiles);
        compute_stage<NT>(st1, xs + static_cast<size_t>(s + kw_count - cb) * 8 * NT * 32, lane, tot);
        load_stage(st1, rows, s + 3 * kw_count, c1, t, scale_tiles);
        s += 2 * kw_count;
      } else {
        st0 = st1;
        load_stage(st1, rows, s + 2 * kw_count, c1, t, scale_tiles);
        s += kw_count;
      }
    }
  }
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
  cluster_sync_all();
  const int out_groups = swiglu ? rm / 2 : rm;
  const int items = out_groups * 2 * NT;
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
    float v[4] = {sum.x * W.inv_dw, sum.y * W.inv_dw, sum.z * W.inv_dw, sum.w * W.inv_dw};
    if (swiglu) {
      const float u[4] = {sum_up.x * W.inv_dw, sum_up.y * W.inv_dw, sum_up.z * W.inv_dw, sum_up.w * W.inv_dw};
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = silu_f32(v[e]) * u[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t tok = tok0 + (e & 1);
      const uint32_t row = out_row + (e >> 1) * 32u;
      if (tok >= p.tokens) continue;
      const size_t at = static_cast<size_t>(tok) * W.ldy + row;
      if (p.epilogue & kEpilogueF32) {
        float *y = static_cast<float *>(W.y);
        y[at] = (p.epilogue & kEpilogueAdd) ? y[at] + v[e] : v[e];
      } else {
        __nv_bfloat16 *y = static_cast<__nv_bfloat16 *>(W.y);
        const float r = (p.epilogue & kEpilogueAdd) ? v[e] + __bfloat162float(y[at]) : v[e];
        y[at] = __float2bfloat16_rn(r);
      }
    }
  }
  cluster_sync_all();  // no CTA leaves while a peer may still read its partial sums
}

size_t gemv_smem_bytes(int nt, int rm, int xs_steps) {
  const int kw_count = kWarps / rm;
  return static_cast<size_t>(xs_steps) * 4096u * nt + static_cast<size_t>(kw_count - 1) * rm * 2 * nt * 32 * 16 +
         static_cast<size_t>(rm) * 2 * nt * 32 * 16 + static_cast<size_t>(16 * nt) * 4;
}

template <int NT>
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
  return cudaLaunchKernelEx(&config, nvfp4_gemv_kernel<NT>, p);
}

}  // namespace

constexpr size_t kGemvMaxSmem = 160 * 1024;

int32_t gemv_prepare(ErrorSlot &slot) {
  cudaError_t err = cudaFuncSetAttribute(nvfp4_gemv_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kGemvMaxSmem));
  if (err == cudaSuccess) err = cudaFuncSetAttribute(nvfp4_gemv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kGemvMaxSmem));
  if (err == cudaSuccess) err = cudaFuncSetAttribute(nvfp4_gemv_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kGemvMaxSmem));
  if (err != cudaSuccess) return fail(slot, "nvfp4 decode kernel attributes: %s", cudaGetErrorString(err));
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
      for (int kc = 1; kc <= 8; kc <<= 1) {
        if (pass == 0 && dev.gemv_rb > 0 && rm != dev.gemv_rb) continue;
        if (pass == 0 && dev.gemv_kc > 0 && kc != dev.gemv_kc) continue;
        if (static_cast<uint32_t>(kc) > ksteps) continue;
        const int kwc = kWarps / rm;
        const uint32_t out_groups = swiglu ? groups / 2 : groups;
        const uint32_t rows_per_cta = swiglu ? rm / 2 : rm;
        const uint32_t row_blocks = (out_groups + rows_per_cta - 1) / rows_per_cta;
        const double ctas = static_cast<double>(row_blocks) * kc;
        const double waves = ceil(ctas / slots);
        const double slice = ceil(static_cast<double>(ksteps) / kc);
        const double steps = ceil(slice / kwc);
        // a step costs 1; preparing one step of activations costs about 0.09 per token tile; a
        // fixed 2 stands for the launch ramp and the reductions
        const double cost = waves * (steps + 0.09 * nt * slice + 2.0) + 0.02 * kc;
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
  const size_t smem = gemv_smem_bytes(nt, plan.rm, plan.xs_steps);
  if (smem > kGemvMaxSmem) return fail(slot, "nvfp4 decode: %zu bytes of shared memory exceed the kernel's limit", smem);
  cudaError_t err;
  if (nt == 1) {
    err = launch_gemv<1>(p, ctas, smem, stream, dev.pdl != 0);
  } else if (nt == 2) {
    err = launch_gemv<2>(p, ctas, smem, stream, dev.pdl != 0);
  } else {
    err = launch_gemv<4>(p, ctas, smem, stream, dev.pdl != 0);
  }
  if (err != cudaSuccess) return fail(slot, "nvfp4 decode launch: %s", cudaGetErrorString(err));
  return 0;
}

}  // namespace b200q
