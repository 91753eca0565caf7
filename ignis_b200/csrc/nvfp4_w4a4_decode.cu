// NVFP4 W4A4 at decode and verify widths (up to 32 tokens): out[t][r] = bf16(alpha * sum_k
// E2M1(a) E4M3(sa) E2M1(w) E4M3(sw)), alpha = 1 / (d_in d_w), with the weights going from HBM to
// the tensor cores untouched. Stands where the reference, under its default AllowA4 policy, leaves
// the A16 kernels from 4 / 5 / 8 tokens and runs its FP4 MMA on quantized activations
// (kernel/vendor/src/ops/linear/nvfp4/nvfp4_dispatch.cpp:31-39, nvfp4_w4a4_mma.cuh:203-436); the
// design is not theirs.
//
//  * The weights are the MMA's A operand: a CTA owns 128 weight rows (M) and walks its slice of K
//    in stages of 256 values. A producer thread brings a stage's 16 KB of codes (TMA, 128-byte
//    swizzle, evict-first) and its four 512-byte scale tiles (a bulk copy) into a ring; nothing in
//    the SM ever decodes a weight.
//  * The tokens are the B operand (N = 16 or 32). Quantizer warps turn the stage's activations into
//    NVFP4 themselves - 16 values per item, bit for bit the rule of the prefill quantizer
//    (nvfp4_codec.cuh:81-110) - straight into the stage's swizzled B tile and its scale tile, so a
//    call needs no workspace, no second launch and no pass over global memory. Every CTA repeats
//    this for its K slice from the L2. The warps work in groups of four that take the stages in
//    turn, so a group has several stage times for its stage.
//  * The producer thread also copies a stage's scale tiles of both operands to tensor memory
//    (tcgen05.cp) once everything of the stage is in place; the last warp owns tensor memory and
//    issues four tcgen05.mma kind::mxf4nvf4 block_scale scale_vec::4X (M 128, N, K 64) per stage.
//  * The fused SwiGLU (a gate|up parent) pairs a tile's 128 gate rows with their up rows: per K
//    stage two ring entries, each with its own weight tile, sharing the first one's token tile,
//    into two accumulators; the epilogue writes BF16(silu(BF16(g alpha)) * BF16(u alpha)).
//  * Narrow weights split K over the CTAs of a cluster, which meet in distributed shared memory and
//    add their partial sums in rank order (bit-reproducible, no global scratch).
//  * Every mbarrier wait is bounded; one that runs out sets a bit in the library's status word
//    (b200q_nvfp4_device_status), and the CTA falls through to the common exit and frees its
//    tensor memory.
#include "nvfp4_internal.cuh"
#include "nvfp4_tc.cuh"

namespace b200q {
namespace {

constexpr uint32_t kABytes = 128 * 128;   // one stage of weight codes: 128 rows x 256 values
constexpr uint32_t kSfBytes = 4 * 512;    // one stage of scales of a 128-row tile: four K-atoms
constexpr uint32_t kProducerTimeout = 0x100u, kMmaTimeout = 0x200u, kEpilogueTimeout = 0x400u, kQuantTimeout = 0x800u;
constexpr int kMaxQuantGroups = 2;
constexpr int kMaxItems = 4;              // 16-value items per quantizer thread and stage (32 tokens)

__device__ uint32_t g_a4_status = 0;

struct A4Weight {
  const uint8_t *scales;
  void *y;
  uint32_t n, ldy;
  float alpha;           // 1 / (d_in d_w)
  float d_in;
  uint32_t block_begin;  // first CTA of this weight
};

struct A4Maps {
  CUtensorMap m[kMaxGroup];  // the weights' code planes
};

struct A4Params {
  A4Weight w[kMaxGroup];
  const uint16_t *x;   // BF16 [tokens][k]
  uint32_t count;
  uint32_t k, tokens;
  uint32_t bn;         // token tile (MMA N): 16 or 32
  uint32_t stages;     // ring depth
  uint32_t pair;       // plain products: 1 = a CTA owns two consecutive row tiles, which share the quantized token tile
  uint32_t groups;     // quantizer groups of 128 threads; then the producer warp and the MMA warp
  uint32_t kc;         // cluster size: K slices
  uint32_t tmem_cols;  // accumulators (64) + 32 scale columns per ring entry, rounded up to a power of two
  uint32_t epilogue;   // STORE / ADD / OUT_F32, or the fused SwiGLU
};

__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t x, int32_t y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void bulk_load_hint(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                 "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(addr)
               : "memory");
}

struct RawItem {
  uint4 lo, hi;  // 16 BF16 activations
};

__global__ void __launch_bounds__(64 + 128 * kMaxQuantGroups, 2) w4a4_decode_kernel(const __grid_constant__ A4Maps maps, const __grid_constant__ A4Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw);
  // a stage: weight codes | token codes | weight scale tiles | token scale tiles
  const uint32_t b_bytes = p.bn * 128u;
  const uint32_t stage_bytes = kABytes + b_bytes + 2u * kSfBytes;
  const uint32_t bars = base + p.stages * stage_bytes;  // full[stages], empty[stages], accumulator full, scales ready[stages]; then the TMEM slot
  const uint32_t bar_sf_ready = bars + 8u * (2u * p.stages + 1u);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + p.stages * stage_bytes + 8u * (3u * p.stages + 1u) + 8u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int producer_warp = 4 * static_cast<int>(p.groups), mma_warp = producer_warp + 1;
  const uint32_t rank = cluster_ctarank(), kc = p.kc;

  uint32_t wi = 0;
#pragma unroll
  for (uint32_t i = 1; i < kMaxGroup; ++i) {
    if (i < p.count && blockIdx.x >= p.w[i].block_begin) wi = i;
  }
  const A4Weight &W = p.w[wi];
  const bool swiglu = (p.epilogue & kEpilogueSwiglu) != 0u;
  const bool two = swiglu || p.pair != 0u;
  const uint32_t halves = two ? 2u : 1u;   // ring entries per K stage: two weight tiles share a token tile
  const uint32_t m_tile = (blockIdx.x - W.block_begin) / kc;
  // first weight rows of the CTA's tiles: gate rows and their up rows (n / 2 further down), or two
  // consecutive tiles of a plain product, or one tile
  const uint32_t row_a = swiglu ? m_tile * 128u : m_tile * 128u * halves;
  const uint32_t row_b = swiglu ? W.n / 2u + m_tile * 128u : row_a + 128u;
  const uint32_t k_stages = p.k / 256u, k_atoms = p.k / 64u;
  const uint32_t s0 = static_cast<uint32_t>(static_cast<uint64_t>(k_stages) * rank / kc);
  const uint32_t s1 = static_cast<uint32_t>(static_cast<uint64_t>(k_stages) * (rank + 1) / kc);

  // One ring entry: a weight tile of K stage s0 + it / halves (entry 2 j is the first tile, 2 j + 1
  // the second when the CTA has two) and its scale tiles.
  const uint32_t entries = (s1 - s0) * halves;
  auto produce = [&](uint32_t it, uint64_t policy) {
    const uint32_t s = s0 + it / halves;
    const uint32_t row0 = (it % halves) != 0u ? row_b : row_a;
    const uint32_t slot = it % p.stages;
    const uint32_t full = bars + 8 * slot;
    const uint32_t stage = base + slot * stage_bytes;
    mbar_expect_tx(full, kABytes + kSfBytes);
    tma_load_2d_hint(stage, &maps.m[wi], full, static_cast<int32_t>(s * 128u), static_cast<int32_t>(row0), policy);
    bulk_load_hint(stage + kABytes + b_bytes, W.scales + (static_cast<size_t>(row0 / 128u) * k_atoms + s * 4u) * 512u, kSfBytes, full,
                   policy);
  };
  // (Requesting the first ring of weight tiles from here, before tensor memory is allocated, was
  // measured slower: the early loads take bandwidth from the previous kernel's last CTAs, which
  // this kernel's quantizers wait for.)
  if (warp == producer_warp && lane == 0) {
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_init(bars + 8 * s, 128 + 1);          // 128 quantizer threads and the producer's expect_tx arrival
      mbar_init(bars + 8 * (p.stages + s), 1);   // the MMA thread's commit
    }
    mbar_init(bars + 8 * 2 * p.stages, 1);
    for (uint32_t s = 0; s < p.stages; ++s) mbar_init(bar_sf_ready + 8 * s, 1);   // the copies' commit
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == mma_warp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(p.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp < 4) {
    // token rows past the call's tokens are never written again: zero codes and zero scales
    for (uint32_t s = 0; s < p.stages; ++s) {
      uint8_t *stage = base_ptr + s * stage_bytes;
      for (uint32_t i = threadIdx.x; i < b_bytes / 16u; i += 128u) reinterpret_cast<uint4 *>(stage + kABytes)[i] = make_uint4(0, 0, 0, 0);
      reinterpret_cast<uint4 *>(stage + kABytes + b_bytes + kSfBytes)[threadIdx.x] = make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp < producer_warp) {
    // ---- quantizers: item i of a stage = token i / 16, values [16 (i % 16), +16) of the stage;
    //      group g takes the CTA's stages g, g + groups, ... ----
    griddep_launch_dependents();
    griddep_wait();   // the activations may come from the previous kernel
    const uint32_t items = p.tokens * 16u;
    const uint32_t group = static_cast<uint32_t>(warp) >> 2, tid = threadIdx.x & 127u;
    const uint32_t first = s0 + group;
    uint32_t tok[kMaxItems], grp[kMaxItems];
    const uint16_t *src[kMaxItems];
#pragma unroll
    for (int j = 0; j < kMaxItems; ++j) {
      const uint32_t i = tid + 128u * j;
      tok[j] = i >> 4;
      grp[j] = i & 15u;
      src[j] = p.x + static_cast<size_t>(tok[j]) * p.k + grp[j] * 16u;
    }
    RawItem cur[kMaxItems];
#pragma unroll
    for (int j = 0; j < kMaxItems; ++j) {
      if (tid + 128u * j < items && first < s1) {
        cur[j].lo = ldg128_coherent(src[j] + static_cast<size_t>(first) * 256u);
        cur[j].hi = ldg128_coherent(src[j] + static_cast<size_t>(first) * 256u + 8);
      }
    }
    bool ok = true;
    for (uint32_t s = first; s < s1 && ok; s += p.groups) {
      const uint32_t it = (s - s0) * halves;   // the stage's (first) ring entry
      uint2 codes[kMaxItems];
      uint8_t scale[kMaxItems];
#pragma unroll
      for (int j = 0; j < kMaxItems; ++j) {
        if (tid + 128u * j < items) quantize_block16(cur[j].lo, cur[j].hi, W.d_in, codes[j], scale[j]);
      }
      if (s + p.groups < s1) {
#pragma unroll
        for (int j = 0; j < kMaxItems; ++j) {
          if (tid + 128u * j < items) {
            cur[j].lo = ldg128_coherent(src[j] + static_cast<size_t>(s + p.groups) * 256u);
            cur[j].hi = ldg128_coherent(src[j] + static_cast<size_t>(s + p.groups) * 256u + 8);
          }
        }
      }
      const uint32_t slot = it % p.stages;
      if (!mbar_wait(bars + 8 * (p.stages + slot), ((it / p.stages) & 1u) ^ 1u)) {
        if (lane == 0) atomicOr(&g_a4_status, kQuantTimeout);
        ok = false;
        break;
      }
      const uint32_t b_tile = base + slot * stage_bytes + kABytes;
      const uint32_t sf_tile = b_tile + b_bytes + kSfBytes;
#pragma unroll
      for (int j = 0; j < kMaxItems; ++j) {
        if (tid + 128u * j < items) {
          const uint32_t t = tok[j], g = grp[j];
          // 128-byte swizzle: row t of the tile, 16-byte unit g / 2 exchanged by the row's low bits
          const uint32_t at = b_tile + (t >> 3) * 1024u + (t & 7u) * 128u + (((g >> 1) ^ (t & 7u)) << 4) + (g & 1u) * 8u;
          asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(at), "r"(codes[j].x), "r"(codes[j].y) : "memory");
          // scale tile of K-atom g / 4: row t at (t % 32) * 16 + (t / 32) * 4, group g % 4 within it
          const uint32_t sat = sf_tile + (g >> 2) * 512u + (t & 31u) * 16u + (t >> 5) * 4u + (g & 3u);
          asm volatile("st.shared.u8 [%0], %1;" ::"r"(sat), "r"(static_cast<uint32_t>(scale[j])) : "memory");
        }
      }
      // the tiles are read by the tensor core (async proxy): order these writes before it
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(bars + 8 * slot);
      if (two) {   // the second entry reads this token tile: nothing to write, only its turn to take
        const uint32_t it2 = it + 1u, slot2 = it2 % p.stages;
        if (!mbar_wait(bars + 8 * (p.stages + slot2), ((it2 / p.stages) & 1u) ^ 1u)) {
          if (lane == 0) atomicOr(&g_a4_status, kQuantTimeout);
          ok = false;
          break;
        }
        mbar_arrive(bars + 8 * slot2);
      }
    }
  } else if (warp == producer_warp) {
    // ---- producer of the weight tiles: they never depend on the previous kernel ----
    griddep_launch_dependents();
    if (lane == 0) {
      // Two jobs, whichever is ready: a free ring entry gets its loads requested; an entry whose
      // operands are all in place (weights landed, tokens quantized) gets its scale tiles copied to
      // tensor memory, so that the MMA thread issues MMAs only (issuing a copy costs its thread
      // about as much as issuing an MMA, and there are twice as many).
      const uint64_t policy = l2_evict_first_policy();
      uint32_t loaded = 0, copied = 0, idle = 0;
      while (copied < entries) {
        bool did = false;
        if (loaded < entries && mbar_test(bars + 8 * (p.stages + loaded % p.stages), ((loaded / p.stages) & 1u) ^ 1u)) {
          produce(loaded, policy);
          ++loaded;
          did = true;
        }
        if (copied < loaded && mbar_test(bars + 8 * (copied % p.stages), (copied / p.stages) & 1u)) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t half = copied % halves, slot = copied % p.stages;
          const uint32_t stage = base + slot * stage_bytes;
          const uint32_t sf_cols = tmem + 64u + slot * 32u;  // 16 columns of weight scales, 16 of token scales
          const uint32_t sfa_smem = stage + kABytes + b_bytes, sfb_smem = sfa_smem + kSfBytes;
#pragma unroll
          for (uint32_t kb = 0; kb < 4; ++kb) {
            tmem_cp_sf(sf_cols + kb * 4u, smem_desc(sfa_smem + kb * 512u, 128u, 0u));
            if (half == 0u) tmem_cp_sf(sf_cols + 16u + kb * 4u, smem_desc(sfb_smem + kb * 512u, 128u, 0u));
          }
          mma_commit(bar_sf_ready + 8 * slot);
          ++copied;
          did = true;
        }
        if (did) {
          idle = 0;
        } else if (++idle > kSpinLimit) {
          atomicOr(&g_a4_status, kProducerTimeout);
          break;
        }
      }
    }
  } else {
    // ---- MMA issuer ----
    griddep_launch_dependents();
    if (lane == 0) {
      // instruction descriptor: E2M1 x E2M1 (format 1 at bits 7 and 10), both K-major, N >> 3 at bit
      // 17, UE4M3 scales (bit 23 clear), M >> 4 at bit 24
      const uint32_t idesc = (1u << 7) | (1u << 10) | ((p.bn >> 3) << 17) | ((128u >> 4) << 24);
      bool ok = true;
      for (uint32_t it = 0; it < entries; ++it) {
        const uint32_t half = it % halves;
        const uint32_t slot = it % p.stages;
        if (!mbar_wait(bar_sf_ready + 8 * slot, (it / p.stages) & 1u)) {   // operands in place and scales copied
          atomicOr(&g_a4_status, kMmaTimeout);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // the token tile and its scales are those of the stage's first entry
        const uint32_t b_slot = (it - half) % p.stages;
        const uint32_t stage = base + slot * stage_bytes, b_stage = base + b_slot * stage_bytes;
        const uint32_t sf_cols = tmem + 64u + slot * 32u;  // 16 columns of weight scales, 16 of token scales
        const uint32_t sfb_cols = tmem + 64u + b_slot * 32u + 16u;
        const uint64_t a_desc = smem_desc(stage, 1024u, 2u);
        const uint64_t b_desc = smem_desc(b_stage + kABytes, 1024u, 2u);
#pragma unroll
        for (uint32_t kb = 0; kb < 4; ++kb) {   // 64 values along K are 32 bytes: two 16-byte units further
          mma_mxf4nvf4(tmem + half * p.bn, a_desc + 2u * kb, b_desc + 2u * kb, idesc, sf_cols + kb * 4u, sfb_cols + kb * 4u,
                       (it >= halves || kb != 0u) ? 1u : 0u);
        }
        if (half + 1u == halves) {   // the stage's entries go back to their writers together
          if (two) mma_commit(bars + 8 * (p.stages + b_slot));
          mma_commit(bars + 8 * (p.stages + slot));
        }
      }
      if (ok) mma_commit(bars + 8 * 2 * p.stages);
    }
  }

  // ---- epilogue: thread r of warps 0-3 owns accumulator lane r = weight row r of the tile ----
  const uint32_t out_elem_f32 = p.epilogue & kEpilogueF32;
  float *part = reinterpret_cast<float *>(base_ptr);   // [half][token][128] partial sums, over the (then idle) stage ring
  bool have = false;
  uint32_t v[32], u[32];
  if (warp < 4) {
    have = mbar_wait(bars + 8 * 2 * p.stages, 0u);
    if (!have && lane == 0) atomicOr(&g_a4_status, kEpilogueTimeout);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (have) {
      const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
      if (p.bn == 16u) {
        tmem_ld16(lane_base, v);
        if (two) tmem_ld16(lane_base + 16u, u);
      } else {
        tmem_ld32(lane_base, v);
        if (two) tmem_ld32(lane_base + 32u, u);
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    }
  }
  // token tl, row r of the CTA's tile(s), from the accumulator sums (the second only with two tiles)
  auto store = [&](size_t at, float acc) {
    const float val = __fmul_rn(acc, W.alpha);   // not contracted into the residual add: one value for every epilogue
    if (out_elem_f32) {
      float *y = static_cast<float *>(W.y);
      y[at] = (p.epilogue & kEpilogueAdd) ? y[at] + val : val;
    } else {
      __nv_bfloat16 *y = static_cast<__nv_bfloat16 *>(W.y);
      y[at] = __float2bfloat16_rn((p.epilogue & kEpilogueAdd) ? val + __bfloat162float(y[at]) : val);
    }
  };
  auto emit = [&](uint32_t tl, uint32_t r, float acc, float acc_b) {
    const size_t at = static_cast<size_t>(tl) * W.ldy + r;
    if (swiglu) {
      const float gv = __bfloat162float(__float2bfloat16_rn(__fmul_rn(acc, W.alpha)));
      const float uv = __bfloat162float(__float2bfloat16_rn(__fmul_rn(acc_b, W.alpha)));
      static_cast<__nv_bfloat16 *>(W.y)[at + row_a] = __float2bfloat16_rn(gv / (1.0f + __expf(-gv)) * uv);
    } else {
      store(at + row_a, acc);
      if (two) store(at + row_b, acc_b);
    }
  };
  if (kc == 1u) {
    if (warp < 4 && have) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (static_cast<uint32_t>(j) >= p.tokens) break;
        emit(static_cast<uint32_t>(j), threadIdx.x, __uint_as_float(v[j]), two ? __uint_as_float(u[j]) : 0.0f);
      }
    }
  } else {
    __syncthreads();   // every role is done with the stage ring: the partial sums take its place
    float *part_up = part + p.bn * 128u;
    if (warp < 4) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (static_cast<uint32_t>(j) < p.bn) {
          part[static_cast<size_t>(j) * 128u + threadIdx.x] = have ? __uint_as_float(v[j]) : 0.0f;
          if (two) part_up[static_cast<size_t>(j) * 128u + threadIdx.x] = have ? __uint_as_float(u[j]) : 0.0f;
        }
      }
    }
    __syncwarp();
    cluster_sync_all();
    if (warp < 4) {
      // tokens dealt over the cluster's CTAs in turn; a thread requests the kc partial sums of its
      // output together and adds them in rank order
      for (uint32_t tl = rank; tl < p.tokens; tl += kc) {
        float pg[8], pu[8];
#pragma unroll
        for (uint32_t q = 0; q < 8u; ++q) {
          pg[q] = q < kc ? ld_cluster_f32(part + static_cast<size_t>(tl) * 128u + threadIdx.x, q) : 0.0f;
          pu[q] = q < kc && two ? ld_cluster_f32(part_up + static_cast<size_t>(tl) * 128u + threadIdx.x, q) : 0.0f;
        }
        float sum = pg[0], sum_up = pu[0];
#pragma unroll
        for (uint32_t q = 1; q < 8u; ++q) {
          if (q < kc) {
            sum += pg[q];
            sum_up += pu[q];
          }
        }
        emit(tl, threadIdx.x, sum, sum_up);
      }
    }
    __syncwarp();
    cluster_sync_all();   // no CTA leaves while a peer may still read its partial sums
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == mma_warp) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(p.tmem_cols) : "memory");
  }
}

constexpr size_t kA4MaxSmem = 220 * 1024;

// Ring depth: what fits beside the other CTAs of the SM, at most 8 stages and no more than the K slice has.
uint32_t a4_ring_depth(uint32_t ctas_per_sm, uint32_t bn, uint32_t k_stages) {
  const uint32_t stage_bytes = kABytes + bn * 128u + 2u * kSfBytes;
  uint32_t stages = (static_cast<uint32_t>(kA4MaxSmem / ctas_per_sm) - 2048u) / stage_bytes;
  if (stages > 8u) stages = 8u;
  return stages < k_stages ? stages : k_stages;
}

size_t a4_smem_bytes(uint32_t bn, uint32_t stages) {
  return static_cast<size_t>(stages) * (kABytes + bn * 128u + 2u * kSfBytes) + 8u * (3u * stages + 1u) + 16u + 1024u;
}

}  // namespace

int32_t w4a4_decode_prepare(ErrorSlot &slot) {
  const cudaError_t err = cudaFuncSetAttribute(w4a4_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kA4MaxSmem));
  if (err != cudaSuccess) return fail(slot, "nvfp4 W4A4 decode kernel attributes: %s", cudaGetErrorString(err));
  if (encode_tiled_fn() == nullptr) return fail(slot, "cuTensorMapEncodeTiled is not available from this driver");
  // How many clusters of each size the device places at one CTA per SM (clusters stay inside one
  // GPC, so sizes 7 and 8 leave many SMs out). The occupancy query counts one CTA per SM for this
  // kernel whatever its shared memory; the plan scales the count by the CTAs that do share an SM.
  DeviceState *dev = device_state(slot);
  if (dev == nullptr) return -1;
  for (int kc = 1; kc <= 8; ++kc) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(kc) * 1024u, 1, 1);
    config.blockDim = dim3(64 + 128 * 2, 1, 1);
    config.dynamicSmemBytes = a4_smem_bytes(16, a4_ring_depth(1, 16, 64));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(kc);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, w4a4_decode_kernel, &config) == cudaSuccess && clusters > 0) {
      dev->a4_slots[kc] = clusters * kc;
    } else {
      dev->a4_slots[kc] = 0;
      (void)cudaGetLastError();
    }
  }
  return 0;
}

bool w4a4_decode_takes(uint32_t n, uint32_t k, uint32_t tokens, uint32_t epilogue) {
  if ((epilogue & kEpilogueSwiglu) != 0u && ((n % 256u) != 0 || (epilogue & (kEpilogueAdd | kEpilogueF32)) != 0u)) return false;
  return tokens >= 1u && tokens <= kA4DecodeMaxTokens && (k % 256u) == 0 && (n % 128u) == 0;
}

int32_t w4a4_decode_launch(ErrorSlot &slot, const DeviceState &dev, const A4Item *items, uint32_t count, const uint16_t *x,
                           uint32_t k, uint32_t tokens, uint32_t epilogue, cudaStream_t stream) {
  A4Params p = {};
  A4Maps maps = {};
  p.x = x;
  p.count = count;
  p.k = k;
  p.tokens = tokens;
  p.bn = tokens <= 16u ? 16u : 32u;
  p.epilogue = epilogue;
  const uint32_t ctas_per_sm = dev.a4_decode_ctas == 1 ? 1u : 2u;
  const bool swiglu = (epilogue & kEpilogueSwiglu) != 0u;
  const uint32_t k_stages = k / 256u;
  // cluster size for `tiles` CTA rows: the largest K split that still runs as one wave (clusters are
  // placed inside one GPC: sizes 7 and 8 leave many slots empty)
  auto plan_kc = [&](uint32_t tiles) {
    uint32_t best = 1;
    for (uint32_t c = 2; c <= 8u && k_stages / c >= 2u; ++c) {
      const int known = dev.a4_slots[c];
      const uint32_t resident = (known > 0 ? static_cast<uint32_t>(known) : static_cast<uint32_t>(dev.sm_count) * 3u / 4u) * ctas_per_sm;
      if (tiles * c <= resident) best = c;
    }
    return best;
  };
  uint32_t row_tiles = 0;
  bool even = true;
  for (uint32_t i = 0; i < count; ++i) {
    row_tiles += (swiglu ? items[i].n / 2u : items[i].n) / 128u;
    even = even && (items[i].n % 256u) == 0;
  }
  uint32_t kc = plan_kc(row_tiles);
  // Two row tiles per CTA halve the quantizers' work per weight byte, K being split twice as often to
  // keep the CTA count. Worth it where the quantizers bound the kernel and K is hardly split yet:
  // wide weights at more than 8 tokens.
  const bool pair = !swiglu && even && k_stages >= 4u && (dev.a4_decode_pair >= 0 ? dev.a4_decode_pair != 0 : tokens > 8u && kc <= 2u);
  if (pair) {
    row_tiles /= 2u;
    kc = plan_kc(row_tiles);
  }
  p.pair = pair ? 1u : 0u;
  const bool two = swiglu || pair;
  uint32_t stages = a4_ring_depth(ctas_per_sm, p.bn, two ? 2u * k_stages : k_stages);
  if (two) stages &= ~1u;   // a K stage takes two ring entries
  p.stages = stages;
  // quantizer groups: two, so that two CTAs still share an SM's registers
  p.groups = dev.a4_decode_groups > 0 ? static_cast<uint32_t>(dev.a4_decode_groups) : 2u;
  if (p.groups > static_cast<uint32_t>(kMaxQuantGroups)) p.groups = kMaxQuantGroups;
  const uint32_t cols = 64u + 32u * stages;
  p.tmem_cols = cols <= 128u ? 128u : (cols <= 256u ? 256u : 512u);
  if (dev.a4_decode_kc > 0 && static_cast<uint32_t>(dev.a4_decode_kc) <= 8u && k_stages / dev.a4_decode_kc >= 1u) kc = dev.a4_decode_kc;
  p.kc = kc;
  EncodeTiledFn encode = encode_tiled_fn();
  uint32_t ctas = 0;
  for (uint32_t i = 0; i < count; ++i) {
    A4Weight &g = p.w[i];
    g.scales = items[i].scales;
    g.y = items[i].y;
    g.n = items[i].n;
    g.ldy = items[i].ldy;
    g.alpha = 1.0f / (items[i].d_in * items[i].d_w);
    g.d_in = items[i].d_in;
    g.block_begin = ctas;
    ctas += (two ? items[i].n / 2u : items[i].n) / 128u * kc;
    const cuuint64_t dims[2] = {k / 2u, items[i].n};
    const cuuint64_t strides[1] = {k / 2u};
    const cuuint32_t box[2] = {128u, 128u};
    const cuuint32_t elem[2] = {1, 1};
    if (encode == nullptr ||
        encode(&maps.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(items[i].codes), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return fail(slot, "nvfp4 W4A4 decode route: tensor map encoding failed");
    }
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(ctas, 1, 1);
  config.blockDim = dim3(64 + 128 * p.groups, 1, 1);
  config.dynamicSmemBytes = a4_smem_bytes(p.bn, stages);
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
  const cudaError_t err = cudaLaunchKernelEx(&config, w4a4_decode_kernel, maps, p);
  if (err != cudaSuccess) return fail(slot, "nvfp4 W4A4 decode launch: %s", cudaGetErrorString(err));
  return 0;
}

int32_t w4a4_decode_status(ErrorSlot &slot, cudaStream_t stream, uint32_t *status) {
  cudaError_t err = cudaMemcpyFromSymbolAsync(status, g_a4_status, sizeof(uint32_t), 0, cudaMemcpyDeviceToHost, stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
  if (err != cudaSuccess) return fail(slot, "b200q_nvfp4_device_status: %s", cudaGetErrorString(err));
  return 0;
}

}  // namespace b200q
