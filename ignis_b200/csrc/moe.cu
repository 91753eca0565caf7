// Flash-Next mixture-of-experts ops: the entry points of include/ignis_moe.h and their kernels.
//
// Routed experts (the reference's ignis_moe_experts_prefill / _decode, kernel/src/moe_prefill.cu:
// 41-492 and moe_decode.cu:325-399): the (token, rank) assignments are grouped by expert on the
// device (count, scan, scatter) and cut into work items of at most 64 rows of one expert (8 from
// the decode entry) made of row tiles of 8. Every row is rotated once into MMA B fragments in the
// workspace (x o suh, Hadamard, power-of-two scale per row and 128 inputs, fp16); a grouped launch
// multiplies each item with its expert's gate|up record, one CTA per 128 output columns, warp j
// walking tile column j: every tile is decoded once in registers and used for all the item's row
// tiles. silu(g) u is rotated the same way and the down launch adds the weighted result to `acc`
// in 64-bit fixed point (2^-32), so the sum does not depend on arrival order. No CTA waits for
// another; a row's arithmetic does not depend on the item it is in, so the decode and prefill
// entries give the same bits.
//
// Nothing here traps or spins: a bad expert id, an absent record or an out-of-range contribution
// is skipped and recorded in the workspace's status word.
#include "../../include/ignis_moe.h"

#include "moe_internal.cuh"
#include "trellis_device.cuh"

#include <mutex>

namespace b200q {
namespace {

using namespace trellis_dev;

constexpr int kThreads = 256;
constexpr int kWarps = 8;

using Geometry = b200q_moe_geometry;
// The geometry the reference's own entry points (no geometry argument) work at: the reference
// compiles it in; here it starts at the reference's and b200q_moe_set_geometry replaces it.
Geometry g_default = {IGNIS_MOE_HIDDEN, IGNIS_MOE_INTERMEDIATE, IGNIS_MOE_EXPERTS, IGNIS_MOE_TOP_K};

int32_t check_geometry(ErrorSlot &slot, const Geometry *g, const char *what) {
  if (g == nullptr) return fail(slot, "%s: geometry is NULL", what);
  if (g->hidden == 0 || (g->hidden % 128u) != 0 || g->inter == 0 || (g->inter % 128u) != 0) {
    return fail(slot, "%s: hidden and inter must be positive multiples of 128", what);
  }
  if (g->experts == 0 || g->experts > 4096u || g->top_k == 0 || g->top_k > 32u || g->top_k > g->experts) {
    return fail(slot, "%s: experts must lie in 1..4096 and top_k in 1..min(32, experts)", what);
  }
  if (g->hidden / 128u > 8u * 40u || g->inter / 128u > 8u * 40u) return fail(slot, "%s: dimension too long", what);
  return 0;
}

// Workspace regions for `tokens_max` tokens.
struct Layout {
  uint64_t status, counts, cursor, offsets, n_items, sorted, items, tiles, frag_in, scale_in, gu, frag_h, scale_h, down_rows, total;
  uint32_t rows_max, items_max, tiles_max;
};

uint64_t align256(uint64_t v) { return (v + 255u) & ~static_cast<uint64_t>(255u); }

uint32_t items_bound(const Geometry &g, uint32_t rows, uint32_t item_rows) {
  return rows / item_rows + (g.experts < rows ? g.experts : rows);
}

Layout layout_for(const Geometry &g, uint32_t tokens_max) {
  Layout l = {};
  l.rows_max = tokens_max * g.top_k;
  l.items_max = items_bound(g, l.rows_max, 8u);  // the bound for 8-row items covers 64-row items too
  l.tiles_max = items_bound(g, l.rows_max, 8u);
  const uint64_t nblk_h = g.hidden / 128u, nblk_i = g.inter / 128u;
  uint64_t at = 0;
  l.status = at; at += 256;
  l.counts = at; at = align256(at + 4ull * g.experts);
  l.cursor = at; at = align256(at + 4ull * g.experts);
  l.offsets = at; at = align256(at + 4ull * (g.experts + 1));
  l.n_items = at; at += 256;  // [0] items, [1] tiles
  l.sorted = at; at = align256(at + 4ull * l.rows_max);
  l.items = at; at = align256(at + 16ull * l.items_max);
  l.tiles = at; at = align256(at + 16ull * l.tiles_max);
  l.frag_in = at; at = align256(at + 2048ull * l.tiles_max * nblk_h);   // rotated x, fragment order
  l.scale_in = at; at = align256(at + 64ull * l.tiles_max * nblk_h);    // (inverse scale, scale) x 8 rows
  l.gu = at; at = align256(at + 8ull * l.rows_max * g.inter);           // fp32 [rows][2 inter]
  l.frag_h = at; at = align256(at + 2048ull * l.tiles_max * nblk_i);    // rotated silu(g) u
  l.scale_h = at; at = align256(at + 64ull * l.tiles_max * nblk_i);
  l.down_rows = at; at = align256(at + (tokens_max > 8u ? 4ull * l.rows_max * g.hidden : 0ull));   // wide calls only (the tensor-core route)
  l.total = at;
  return l;
}

// ---- grouping ------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_count_kernel(const int32_t *ids, uint32_t rows, uint32_t experts,
                                                        uint32_t *counts, uint32_t *status) {
  griddep_launch_dependents();
  griddep_wait();
  for (uint32_t a = blockIdx.x * blockDim.x + threadIdx.x; a < rows; a += gridDim.x * blockDim.x) {
    const int32_t e = ids[a];
    if (e < 0 || static_cast<uint32_t>(e) >= experts) {
      if (e != IGNIS_MOE_NO_EXPERT) atomicOr(status, kStatusBadExpert);  // -1 is "no expert for this choice": skipped, not an error
    } else {
      atomicAdd(&counts[e], 1u);
    }
  }
}

// One CTA: exclusive scans of the per-expert row, item and tile counts, then the item and tile lists.
__global__ void __launch_bounds__(1024) moe_scan_kernel(const uint32_t *counts, uint32_t experts, uint32_t item_rows,
                                                        uint32_t *offsets, uint32_t *n_items, Item *items, Tile *tiles) {
  griddep_launch_dependents();
  griddep_wait();
  __shared__ uint32_t row_sum[1024], item_sum[1024], tile_sum[1024];
  const uint32_t per = (experts + 1023u) / 1024u;  // experts per thread, consecutive
  const uint32_t e0 = threadIdx.x * per;
  uint32_t rows = 0, its = 0, tls = 0;
  for (uint32_t e = e0; e < e0 + per && e < experts; ++e) {
    rows += counts[e];
    its += (counts[e] + item_rows - 1u) / item_rows;
    tls += (counts[e] + 7u) / 8u;
  }
  row_sum[threadIdx.x] = rows;
  item_sum[threadIdx.x] = its;
  tile_sum[threadIdx.x] = tls;
  __syncthreads();
  for (uint32_t d = 1; d < 1024; d <<= 1) {  // Hillis-Steele inclusive scan
    const uint32_t r = threadIdx.x >= d ? row_sum[threadIdx.x - d] : 0u;
    const uint32_t i = threadIdx.x >= d ? item_sum[threadIdx.x - d] : 0u;
    const uint32_t t = threadIdx.x >= d ? tile_sum[threadIdx.x - d] : 0u;
    __syncthreads();
    row_sum[threadIdx.x] += r;
    item_sum[threadIdx.x] += i;
    tile_sum[threadIdx.x] += t;
    __syncthreads();
  }
  uint32_t row_at = row_sum[threadIdx.x] - rows, item_at = item_sum[threadIdx.x] - its, tile_at = tile_sum[threadIdx.x] - tls;
  for (uint32_t e = e0; e < e0 + per && e < experts; ++e) {
    offsets[e] = row_at;
    const uint32_t c = counts[e];
    for (uint32_t j = 0; j < c; j += item_rows) {
      items[item_at++] = Item{e, row_at + j, c - j < item_rows ? c - j : item_rows, tile_at + j / 8u};
    }
    for (uint32_t j = 0; j < c; j += 8) tiles[tile_at++] = Tile{e, row_at + j, c - j < 8u ? c - j : 8u, 0u};
    row_at += c;
  }
  if (threadIdx.x == 1023) {
    offsets[experts] = row_sum[1023];
    n_items[0] = item_sum[1023];
    n_items[1] = tile_sum[1023];
  }
}

__global__ void __launch_bounds__(256) moe_scatter_kernel(const int32_t *ids, uint32_t rows, uint32_t experts,
                                                          const uint32_t *offsets, uint32_t *cursor, uint32_t *sorted) {
  griddep_launch_dependents();
  griddep_wait();
  for (uint32_t a = blockIdx.x * blockDim.x + threadIdx.x; a < rows; a += gridDim.x * blockDim.x) {
    const int32_t e = ids[a];
    if (e < 0 || static_cast<uint32_t>(e) >= experts) continue;
    // rows of one expert are independent of each other, so their order inside the group does
    // not change any output bit
    sorted[offsets[e] + atomicAdd(&cursor[e], 1u)] = a;
  }
}

// Count, scan and scatter in one CTA for calls of a few rows (the decode widths): the three launches
// above cost more than their work there. Counts and cursors live in shared memory.
constexpr uint32_t kSmallRows = 4096, kSmallExperts = 4096;

__global__ void __launch_bounds__(1024) moe_group_small_kernel(const int32_t *ids, uint32_t rows, uint32_t experts, uint32_t item_rows,
                                                               uint32_t *offsets, uint32_t *n_items, Item *items, Tile *tiles,
                                                               uint32_t *sorted, uint32_t *status) {
  griddep_launch_dependents();
  griddep_wait();
  __shared__ uint32_t counts[kSmallExperts], start[kSmallExperts];
  __shared__ uint32_t row_sum[1024], item_sum[1024], tile_sum[1024];
  for (uint32_t e = threadIdx.x; e < experts; e += 1024) counts[e] = 0u;
  __syncthreads();
  for (uint32_t a = threadIdx.x; a < rows; a += 1024) {
    const int32_t e = ids[a];
    if (e < 0 || static_cast<uint32_t>(e) >= experts) {
      if (e != IGNIS_MOE_NO_EXPERT) atomicOr(status, kStatusBadExpert);  // -1 is "no expert for this choice": skipped, not an error
    } else {
      atomicAdd(&counts[e], 1u);
    }
  }
  __syncthreads();
  const uint32_t per = (experts + 1023u) / 1024u;
  const uint32_t e0 = threadIdx.x * per;
  uint32_t nrows = 0, its = 0, tls = 0;
  for (uint32_t e = e0; e < e0 + per && e < experts; ++e) {
    nrows += counts[e];
    its += (counts[e] + item_rows - 1u) / item_rows;
    tls += (counts[e] + 7u) / 8u;
  }
  row_sum[threadIdx.x] = nrows;
  item_sum[threadIdx.x] = its;
  tile_sum[threadIdx.x] = tls;
  __syncthreads();
  for (uint32_t d = 1; d < 1024; d <<= 1) {
    const uint32_t r = threadIdx.x >= d ? row_sum[threadIdx.x - d] : 0u;
    const uint32_t i = threadIdx.x >= d ? item_sum[threadIdx.x - d] : 0u;
    const uint32_t t = threadIdx.x >= d ? tile_sum[threadIdx.x - d] : 0u;
    __syncthreads();
    row_sum[threadIdx.x] += r;
    item_sum[threadIdx.x] += i;
    tile_sum[threadIdx.x] += t;
    __syncthreads();
  }
  uint32_t row_at = row_sum[threadIdx.x] - nrows, item_at = item_sum[threadIdx.x] - its, tile_at = tile_sum[threadIdx.x] - tls;
  for (uint32_t e = e0; e < e0 + per && e < experts; ++e) {
    offsets[e] = row_at;
    start[e] = row_at;
    const uint32_t c = counts[e];
    for (uint32_t j = 0; j < c; j += item_rows) {
      items[item_at++] = Item{e, row_at + j, c - j < item_rows ? c - j : item_rows, tile_at + j / 8u};
    }
    for (uint32_t j = 0; j < c; j += 8) tiles[tile_at++] = Tile{e, row_at + j, c - j < 8u ? c - j : 8u, 0u};
    row_at += c;
  }
  if (threadIdx.x == 1023) {
    offsets[experts] = row_sum[1023];
    n_items[0] = item_sum[1023];
    n_items[1] = tile_sum[1023];
  }
  __syncthreads();
  for (uint32_t a = threadIdx.x; a < rows; a += 1024) {
    const int32_t e = ids[a];
    if (e < 0 || static_cast<uint32_t>(e) >= experts) continue;
    sorted[atomicAdd(&start[e], 1u)] = a;  // rows of one expert are independent: their order changes no output bit
  }
}

// ---- the expert kernels ----------------------------------------------------------------------
// Rotates the rows of one tile into B fragments, once per row: PHASE 0 x o suh of the gate/up
// record, PHASE 1 silu(g) u o suh of the down record; then the 128-wide Hadamard in fp32, a
// power-of-two scale per (row, block) (largest value in [2^13, 2^14)) and fp16. One CTA per tile,
// warp r = row r; a block's fragment (2 KB) is put together in shared memory and written out whole.
template <int PHASE>
__global__ void __launch_bounds__(kThreads) moe_rotate_kernel(const __grid_constant__ ExpertParams p) {
  __shared__ __align__(16) uint2 frag[2][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  griddep_launch_dependents();
  griddep_wait();
  const uint32_t tile_index = blockIdx.x;
  if (tile_index >= p.n_items[1]) return;
  const Tile tile = p.tiles[tile_index];
  const ignis_moe_slot slot = p.slots[tile.expert * 2u + PHASE];
  if (slot.record == nullptr || !(slot.k2 == 4 || slot.k2 == 5 || slot.k2 == 6 || slot.k2 == 8)) return;  // flagged by the walk
  const uint32_t in = PHASE == 0 ? p.hidden : p.inter;
  const uint32_t out_plane = PHASE == 0 ? 2u * p.inter : p.hidden;
  const uint64_t trellis_bytes = static_cast<uint64_t>(in) * out_plane * slot.k2 / 16u;
  const uint16_t *suh = reinterpret_cast<const uint16_t *>(static_cast<const uint8_t *>(slot.record) + trellis_bytes);
  const uint32_t nblk = in / 128u;
  const bool live = static_cast<uint32_t>(warp) < tile.count;
  const uint32_t row = tile.first + static_cast<uint32_t>(warp);
  uint32_t token = 0;
  if (live && PHASE == 0) token = p.sorted[row] / p.top_k;
  uint2 *dst_frag = (PHASE == 0 ? p.frag_in : p.frag_h) + static_cast<size_t>(tile_index) * nblk * 256u;
  float2 *dst_scale = (PHASE == 0 ? p.scale_in : p.scale_h) + static_cast<size_t>(tile_index) * nblk * 8u;
  for (uint32_t bl = 0; bl < nblk; ++bl) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
      const size_t k0 = static_cast<size_t>(bl) * 128u + 4u * lane;
      const uint2 sb = *reinterpret_cast<const uint2 *>(suh + k0);
      const __half2 s01 = *reinterpret_cast<const __half2 *>(&sb.x), s23 = *reinterpret_cast<const __half2 *>(&sb.y);
      if (PHASE == 0) {
        const uint2 xb = ldg64_coherent(p.x + static_cast<size_t>(token) * p.hidden + k0);
        v[0] = bf16_bits_to_f32(xb.x & 0xFFFFu) * __low2float(s01);
        v[1] = __uint_as_float(xb.x & 0xFFFF0000u) * __high2float(s01);
        v[2] = bf16_bits_to_f32(xb.y & 0xFFFFu) * __low2float(s23);
        v[3] = __uint_as_float(xb.y & 0xFFFF0000u) * __high2float(s23);
      } else {
        const float *g = p.gu + static_cast<size_t>(row) * 2u * p.inter + k0;
        const uint4 gb = ldg128_coherent(g), ub = ldg128_coherent(g + p.inter);
        const float gv[4] = {__uint_as_float(gb.x), __uint_as_float(gb.y), __uint_as_float(gb.z), __uint_as_float(gb.w)};
        const float uv[4] = {__uint_as_float(ub.x), __uint_as_float(ub.y), __uint_as_float(ub.z), __uint_as_float(ub.w)};
        const float sv[4] = {__low2float(s01), __high2float(s01), __low2float(s23), __high2float(s23)};
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = gv[i] / (1.0f + __expf(-gv[i])) * uv[i] * sv[i];
      }
    }
    hadamard128(v, lane);
    float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    int shift = 0;
    if (m > 0.0f && m <= 3.0e38f) {
      int e;
      (void)frexpf(m, &e);
      shift = max(-126, min(126, 14 - e));
    }
    const float scale = ldexpf(1.0f, shift);
    const __half2 h01 = __floats2half2_rn(v[0] * scale, v[1] * scale);
    const __half2 h23 = __floats2half2_rn(v[2] * scale, v[3] * scale);
    // element e = 4 lane + i of the block: step kt = e / 16, inside it k16 = e % 16; the reader
    // lane (g = row, t) keeps k16 in {2t, 2t+1} in .x and {2t+8, 2t+9} in .y
    const int kt = lane >> 2, k16 = (lane & 3) * 4;
    const int t_first = (k16 & 7) >> 1, reg = k16 >> 3;
    uint32_t *dst = reinterpret_cast<uint32_t *>(&frag[bl & 1][kt * 32 + warp * 4]);
    dst[t_first * 2 + reg] = *reinterpret_cast<const uint32_t *>(&h01);
    dst[(t_first + 1) * 2 + reg] = *reinterpret_cast<const uint32_t *>(&h23);
    if (lane == 0) dst_scale[bl * 8u + warp] = make_float2(live ? ldexpf(1.0f, -shift) : 0.0f, scale);
    __syncthreads();  // the block's fragment is whole; the other buffer is free for the next block
    dst_frag[static_cast<size_t>(bl) * 256u + threadIdx.x] = frag[bl & 1][threadIdx.x];
  }
}

// The lane's words of the 8 steps of one 128-input block of one tile column.
struct BlockWords {
  uint32_t w[8][3];
};

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *src) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// The item's fragments and scales of one 128-input block, copied asynchronously into the CTA's
// staging buffers: 2 KB per live row tile and 64 bytes of (inverse scale, scale) pairs.
template <int NT>
__device__ __forceinline__ void stage_block(uint2 *frag_buf, float2 *scale_buf, const uint2 *frag, const float2 *scales,
                                            uint32_t nblk, uint32_t bl, uint32_t ntiles) {
  for (uint32_t c = threadIdx.x; c < ntiles * 128u; c += kThreads) {
    const uint32_t tt = c >> 7, off = c & 127u;  // 16-byte chunk `off` of tile tt's fragment
    cp_async16(frag_buf + tt * 256u + off * 2u, frag + (static_cast<size_t>(tt) * nblk + bl) * 256u + off * 2u);
  }
  if (threadIdx.x < ntiles * 4u) {
    const uint32_t tt = threadIdx.x >> 2, off = threadIdx.x & 3u;
    cp_async16(scale_buf + tt * 8u + off * 2u, scales + (static_cast<size_t>(tt) * nblk + bl) * 8u + off * 2u);
  }
  cp_async_commit();
}

// Warp j of the CTA walks tile column j of the item's column block down all the inputs: one tile
// per 16 inputs, decoded once and multiplied with every live row tile of the item (up to NT tiles
// of 8 rows). The words of the next 128-input block are requested as the current block's are
// consumed; the rows' fragments and scales of the next block are copied to shared memory while
// the current block is multiplied (one CTA barrier per block). Sums are in the units of the
// current block's per-row scale and carried exactly into the next block's.
template <int K2, int NT>
__device__ __forceinline__ void walk_tile_column(const uint32_t *tile_base, int64_t step_words, uint32_t nblk, const uint2 *frag,
                                                 const float2 *scales, uint32_t ntiles, int lane, uint2 (*frag_buf)[NT * 256],
                                                 float2 (*scale_buf)[NT * 8], float (&tot)[NT][4]) {
  const LaneWindow win = lane_window(K2, lane);
  const uint32_t *q0 = tile_base + win.w0, *q1 = tile_base + win.w1, *q2 = tile_base + win.w2;
  BlockWords bw;
#pragma unroll
  for (int kt = 0; kt < 8; ++kt) {
    bw.w[kt][0] = __ldg(q0 + kt * step_words);
    bw.w[kt][1] = __ldg(q1 + kt * step_words);
    bw.w[kt][2] = __ldg(q2 + kt * step_words);
  }
  stage_block<NT>(frag_buf[0], scale_buf[0], frag, scales, nblk, 0, ntiles);
  const int t2 = (lane & 3) * 2;
  for (uint32_t bl = 0; bl < nblk; ++bl) {
    const bool more = bl + 1 < nblk;
    cp_async_wait_all();
    __syncthreads();  // this block's copies are visible; nobody still reads the buffers refilled next
    if (more) stage_block<NT>(frag_buf[(bl + 1) & 1], scale_buf[(bl + 1) % 3], frag, scales, nblk, bl + 1, ntiles);
    const uint2 *fb = frag_buf[bl & 1] + lane;
    const float2 *cur = scale_buf[bl % 3] + t2, *prev = scale_buf[(bl + 2) % 3] + t2;
    // into this block's units: the sums so far are in the previous block's (inverse scale of the
    // previous block times scale of this one, an exact power of two; nothing to carry at block 0)
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) {
      float f0 = 0.0f, f1 = 0.0f;
      if (bl > 0 && static_cast<uint32_t>(tt) < ntiles) {
        const float4 c = *reinterpret_cast<const float4 *>(cur + tt * 8), pv = *reinterpret_cast<const float4 *>(prev + tt * 8);
        f0 = pv.x * c.y;
        f1 = pv.z * c.w;
      }
      tot[tt][0] *= f0;
      tot[tt][1] *= f1;
      tot[tt][2] *= f0;
      tot[tt][3] *= f1;
    }
    if (more) q0 += 8 * step_words, q1 += 8 * step_words, q2 += 8 * step_words;
#pragma unroll
    for (int kt = 0; kt < 8; ++kt) {
      uint32_t a[4];
      decode8<K2>(bw.w[kt][0], bw.w[kt][1], bw.w[kt][2], win.off, a);
      if (more) {
        bw.w[kt][0] = __ldg(q0 + kt * step_words);
        bw.w[kt][1] = __ldg(q1 + kt * step_words);
        bw.w[kt][2] = __ldg(q2 + kt * step_words);
      }
#pragma unroll
      for (int tt = 0; tt < NT; ++tt) {
        if (static_cast<uint32_t>(tt) < ntiles) {  // uniform over the CTA
          const uint2 b = fb[tt * 256 + kt * 32];
          mma_f16_f32(tot[tt], a[0], a[2], a[1], a[3], b.x, b.y);
        }
      }
    }
  }
  // back to the rows' own units
  const float2 *last = scale_buf[(nblk - 1u) % 3] + t2;
#pragma unroll
  for (int tt = 0; tt < NT; ++tt) {
    float i0 = 0.0f, i1 = 0.0f;
    if (static_cast<uint32_t>(tt) < ntiles) {
      const float4 c = *reinterpret_cast<const float4 *>(last + tt * 8);
      i0 = c.x;
      i1 = c.z;
    }
    tot[tt][0] *= i0;
    tot[tt][1] *= i1;
    tot[tt][2] *= i0;
    tot[tt][3] *= i1;
  }
}

// PHASE 0: gate | up products of an item into gu. PHASE 1: down, weighted, into acc.
// One CTA per (item, block of 128 output columns); no CTA waits for another.
template <int PHASE, int NT>
__global__ void __launch_bounds__(kThreads, NT <= 2 ? 3 : 2) moe_experts_kernel(const __grid_constant__ ExpertParams p) {
  // staging for two blocks of fragments, aliased after the walk by the partial sums
  // [tile column 8][row tile NT][lane 32]; three blocks of scales
  __shared__ __align__(16) uint2 frag_buf[2][NT * 256];
  __shared__ __align__(16) float2 scale_buf[3][NT * 8];
  float4 *part = reinterpret_cast<float4 *>(&frag_buf[0][0]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t in = PHASE == 0 ? p.hidden : p.inter;
  const uint32_t out_plane = PHASE == 0 ? 2u * p.inter : p.hidden;   // columns of the stored plane
  const uint32_t col_blocks = out_plane / 128u;
  const uint32_t item_index = blockIdx.x / col_blocks;
  const uint32_t col_block = blockIdx.x % col_blocks;

  griddep_launch_dependents();
  griddep_wait();  // the item list and the fragments come from the kernels before

  if (item_index >= p.n_items[0]) return;
  const Item item = p.items[item_index];
  const ignis_moe_slot slot = p.slots[item.expert * 2u + PHASE];
  const uint32_t k2 = slot.k2;
  if (slot.record == nullptr || !(k2 == 4 || k2 == 5 || k2 == 6 || k2 == 8)) {
    if (threadIdx.x == 0 && col_block == 0) atomicOr(p.status, kStatusAbsentRecord);
    return;
  }
  const uint32_t *trellis = static_cast<const uint32_t *>(slot.record);
  const uint64_t trellis_bytes = static_cast<uint64_t>(in) * out_plane * k2 / 16u;
  const uint16_t *svh = reinterpret_cast<const uint16_t *>(static_cast<const uint8_t *>(slot.record) + trellis_bytes) + in;
  const uint32_t nblk = in / 128u;
  const uint32_t ntiles = (item.count + 7u) / 8u;
  const uint2 *frag = (PHASE == 0 ? p.frag_in : p.frag_h) + static_cast<size_t>(item.tile_first) * nblk * 256u;
  const float2 *scales = (PHASE == 0 ? p.scale_in : p.scale_h) + static_cast<size_t>(item.tile_first) * nblk * 8u;

  float tot[NT][4];
#pragma unroll
  for (int tt = 0; tt < NT; ++tt)
#pragma unroll
    for (int e = 0; e < 4; ++e) tot[tt][e] = 0.0f;
  {
    const uint32_t tile_words = 4u * k2;
    const uint32_t *tile_base = trellis + (static_cast<uint64_t>(col_block) * 8u + static_cast<uint32_t>(warp)) * tile_words;
    const int64_t step_words = static_cast<int64_t>(out_plane / 16u) * tile_words;
    switch (k2) {
      case 4: walk_tile_column<4, NT>(tile_base, step_words, nblk, frag, scales, ntiles, lane, frag_buf, scale_buf, tot); break;
      case 5: walk_tile_column<5, NT>(tile_base, step_words, nblk, frag, scales, ntiles, lane, frag_buf, scale_buf, tot); break;
      case 6: walk_tile_column<6, NT>(tile_base, step_words, nblk, frag, scales, ntiles, lane, frag_buf, scale_buf, tot); break;
      default: walk_tile_column<8, NT>(tile_base, step_words, nblk, frag, scales, ntiles, lane, frag_buf, scale_buf, tot); break;
    }
  }
  __syncthreads();  // every warp is done with the staging buffers: the partial sums take their place
#pragma unroll
  for (int tt = 0; tt < NT; ++tt) part[(warp * NT + tt) * 32 + lane] = make_float4(tot[tt][0], tot[tt][1], tot[tt][2], tot[tt][3]);
  __syncthreads();

  // ---- finish: rows dealt to the warps; lane = 4 output columns of the block ----
  for (uint32_t r = static_cast<uint32_t>(warp); r < item.count; r += kWarps) {
    const uint32_t tt = r >> 3, rs = r & 7u;
    const int tq = static_cast<int>(rs >> 1), te = static_cast<int>(rs & 1u);
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = 4 * lane + i, j = c >> 4, cc = c & 15;
      v[i] = *(reinterpret_cast<const float *>(&part[(j * NT + tt) * 32 + (cc & 7) * 4 + tq]) + te + 2 * (cc >> 3));
    }
    hadamard128(v, lane);
    const uint2 sv = *reinterpret_cast<const uint2 *>(svh + static_cast<size_t>(col_block) * 128u + 4u * lane);
    const __half2 s01 = *reinterpret_cast<const __half2 *>(&sv.x), s23 = *reinterpret_cast<const __half2 *>(&sv.y);
    v[0] *= __low2float(s01);
    v[1] *= __high2float(s01);
    v[2] *= __low2float(s23);
    v[3] *= __high2float(s23);
    const uint32_t row = item.first + r;
    if (PHASE == 0) {
      *reinterpret_cast<float4 *>(p.gu + static_cast<size_t>(row) * 2u * p.inter + col_block * 128u + 4u * lane) =
          make_float4(v[0], v[1], v[2], v[3]);
    } else {
      const uint32_t a = p.sorted[row];
      const uint32_t token = a / p.top_k;
      const float wr = p.weights[a];
      long long *dst = p.acc + static_cast<size_t>(token) * p.hidden + col_block * 128u + 4u * lane;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float c = wr * v[i];
        if (!(fabsf(c) < 2147483648.0f)) {  // also catches NaN
          atomicOr(p.status, kStatusRange);
        } else {
          atomicAdd(reinterpret_cast<unsigned long long *>(dst + i),
                    static_cast<unsigned long long>(__double2ll_rn(static_cast<double>(c) * 4294967296.0)));
        }
      }
    }
  }
}

// ---- router ----------------------------------------------------------------------------------
// One CTA per token: the token's activations in shared memory, each warp takes experts
// warp, warp + 8, ...; fp32 accumulation in a fixed order (lane-strided, then a butterfly).
__global__ void __launch_bounds__(256) moe_router_logits_kernel(const uint16_t *x, const uint16_t *w, uint32_t hidden,
                                                                uint32_t experts, float *logits) {
  extern __shared__ float xs[];
  griddep_launch_dependents();
  griddep_wait();
  const uint32_t t = blockIdx.x;
  for (uint32_t k = threadIdx.x; k < hidden; k += blockDim.x) xs[k] = bf16_bits_to_f32(x[static_cast<size_t>(t) * hidden + k]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (uint32_t e = warp; e < experts; e += 8) {
    const uint16_t *row = w + static_cast<size_t>(e) * hidden;
    float acc = 0.0f;
    for (uint32_t k = lane * 2; k < hidden; k += 64) {
      const uint32_t pair = *reinterpret_cast<const uint32_t *>(row + k);
      acc = fmaf(bf16_bits_to_f32(pair & 0xFFFFu), xs[k], acc);
      acc = fmaf(__uint_as_float(pair & 0xFFFF0000u), xs[k + 1], acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if (lane == 0) logits[static_cast<size_t>(t) * experts + e] = acc;
  }
}

// One warp per token: the top_k largest BF16-rounded logits, ties to the lower id, then the
// softmax over the selected ones in fp32, rounded to BF16 and stored as fp32.
__global__ void __launch_bounds__(256) moe_router_select_kernel(const float *logits, uint32_t tokens, uint32_t experts,
                                                                uint32_t top_k, int32_t *ids, float *weights) {
  griddep_launch_dependents();
  griddep_wait();
  const uint32_t t = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const float *row = logits + static_cast<size_t>(t) * experts;
  float sel[32];
  float prev_v = INFINITY;
  int prev_id = -1;
  for (uint32_t r = 0; r < top_k; ++r) {
    // the largest (value, then lowest id) strictly after the previous pick in that order
    float best_v = -INFINITY;
    int best_id = 0x7FFFFFFF;
    for (uint32_t e = lane; e < experts; e += 32) {
      const float v = __bfloat162float(__float2bfloat16_rn(row[e]));
      const bool after_prev = v < prev_v || (v == prev_v && static_cast<int>(e) > prev_id);
      const bool better = v > best_v || (v == best_v && static_cast<int>(e) < best_id);
      if (after_prev && better) {
        best_v = v;
        best_id = static_cast<int>(e);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, best_v, o);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, best_id, o);
      if (ov > best_v || (ov == best_v && oi < best_id)) {
        best_v = ov;
        best_id = oi;
      }
    }
    prev_v = best_v;
    prev_id = best_id;
    sel[r] = best_v;
    if (lane == 0) ids[static_cast<size_t>(t) * top_k + r] = best_id;
  }
  if (lane == 0) {
    const float mx = sel[0];
    float sum = 0.0f;
    for (uint32_t r = 0; r < top_k; ++r) {
      sel[r] = expf(sel[r] - mx);
      sum += sel[r];
    }
    for (uint32_t r = 0; r < top_k; ++r) {
      weights[static_cast<size_t>(t) * top_k + r] = __bfloat162float(__float2bfloat16_rn(sel[r] / sum));
    }
  }
}

// ---- shared expert (FP8 row-scale) and combine ---------------------------------------------------
// y[t][r] = scale[r] * sum_c e4m3(code[r][c]) * x[t][c]: one warp per output row, up to 8 tokens a
// pass. MODE 0: two weights, BF16 SwiGLU output; MODE 1: one weight, fp32 output from BF16 input.
template <int MODE>
__global__ void __launch_bounds__(256) moe_fp8_rows_kernel(const uint8_t *w0, const uint8_t *w1, uint32_t rows, uint32_t cols,
                                                           const uint16_t *x, uint32_t tokens, void *y) {
  griddep_launch_dependents();
  griddep_wait();
  const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint64_t scale_off = (static_cast<uint64_t>(rows) * cols + 255u) & ~static_cast<uint64_t>(255u);
  const uint8_t *weights[2] = {w0, w1};
  for (uint32_t t0 = 0; t0 < tokens; t0 += 8) {
    float acc[2][8];
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int t = 0; t < 8; ++t) acc[s][t] = 0.0f;
    for (uint32_t c = lane * 4; c < cols; c += 128) {
      float wv[2][4];
#pragma unroll
      for (int s = 0; s < (MODE == 0 ? 2 : 1); ++s) {
        const uint32_t codes = *reinterpret_cast<const uint32_t *>(weights[s] + static_cast<uint64_t>(row) * cols + c);
        const uint32_t lo = e4m3x2_to_half2(codes & 0xFFFFu), hi = e4m3x2_to_half2(codes >> 16);
        const __half2 l2 = *reinterpret_cast<const __half2 *>(&lo), h2 = *reinterpret_cast<const __half2 *>(&hi);
        wv[s][0] = __low2float(l2);
        wv[s][1] = __high2float(l2);
        wv[s][2] = __low2float(h2);
        wv[s][3] = __high2float(h2);
      }
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        if (t0 + t >= tokens) break;
        const uint2 xb = *reinterpret_cast<const uint2 *>(x + static_cast<uint64_t>(t0 + t) * cols + c);
        const float xv[4] = {bf16_bits_to_f32(xb.x & 0xFFFFu), __uint_as_float(xb.x & 0xFFFF0000u),
                             bf16_bits_to_f32(xb.y & 0xFFFFu), __uint_as_float(xb.y & 0xFFFF0000u)};
#pragma unroll
        for (int s = 0; s < (MODE == 0 ? 2 : 1); ++s)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[s][t] = fmaf(wv[s][i], xv[i], acc[s][t]);
      }
    }
#pragma unroll
    for (int s = 0; s < (MODE == 0 ? 2 : 1); ++s)
#pragma unroll
      for (int t = 0; t < 8; ++t)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[s][t] += __shfl_xor_sync(0xFFFFFFFFu, acc[s][t], o);
    if (lane == 0) {
      const float s0 = bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(w0 + scale_off)[row]);
      const float s1 = MODE == 0 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(w1 + scale_off)[row]) : 0.0f;
      for (int t = 0; t < 8 && t0 + t < tokens; ++t) {
        if (MODE == 0) {
          const float g = acc[0][t] * s0, u = acc[1][t] * s1;
          static_cast<__nv_bfloat16 *>(y)[static_cast<uint64_t>(t0 + t) * rows + row] = __float2bfloat16_rn(g / (1.0f + __expf(-g)) * u);
        } else {
          static_cast<float *>(y)[static_cast<uint64_t>(t0 + t) * rows + row] = acc[0][t] * s0;
        }
      }
    }
  }
}

// Two E4M3 codes (the low 16 bits of `pair`) as BF16 x 2, exactly: every E4M3 value has a BF16.
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2(uint32_t pair) {
  const uint32_t h = e4m3x2_to_half2(pair);
  const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&h));
  const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
  return *reinterpret_cast<const uint32_t *>(&b);
}

// The same products for many tokens, on the tensor cores: a warp owns 16 weight rows (of both
// weights in MODE 0) and 64 tokens, a CTA 128 rows. Weights are widened E4M3 -> BF16 (exact) into A
// fragments, the activations are the B fragments as they lie in memory: inside a chunk of 64
// columns the MMA's k slots are dealt so that a lane needs 16 contiguous codes of its two rows
// and 16 contiguous activations of its token. FP32 accumulation, the row scale applied at the end.
template <int MODE>
__global__ void __launch_bounds__(256) moe_fp8_gemm_kernel(const uint8_t *w0, const uint8_t *w1, uint32_t rows, uint32_t cols,
                                                           const uint16_t *x, uint32_t tokens, void *y) {
  griddep_launch_dependents();
  griddep_wait();
  constexpr int S = MODE == 0 ? 2 : 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t row0 = (blockIdx.x * 8u + static_cast<uint32_t>(warp)) * 16u;
  const uint32_t tok0 = blockIdx.y * 64u;
  if (row0 >= rows) return;
  const uint8_t *weights[2] = {w0, w1};
  float acc[S][8][4];
#pragma unroll
  for (int s = 0; s < S; ++s)
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[s][nt][e] = 0.0f;
  for (uint32_t kb = 0; kb < cols; kb += 64) {
    uint32_t a[S][4][4];  // [weight][MMA j][a0..a3]
#pragma unroll
    for (int s = 0; s < S; ++s) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint4 cw = *reinterpret_cast<const uint4 *>(weights[s] + static_cast<uint64_t>(row0 + g + 8 * half) * cols + kb + 16 * t);
        const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          a[s][j][half] = e4m3x2_to_bf16x2(w[j] & 0xFFFFu);      // k slots 2t, 2t + 1
          a[s][j][2 + half] = e4m3x2_to_bf16x2(w[j] >> 16);       // k slots 2t + 8, 2t + 9
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const uint32_t token = tok0 + nt * 8 + g;
      uint4 x0 = make_uint4(0u, 0u, 0u, 0u), x1 = x0;
      if (token < tokens) {
        const uint4 *src = reinterpret_cast<const uint4 *>(x + static_cast<uint64_t>(token) * cols + kb + 16 * t);
        x0 = ldg128_coherent(src);
        x1 = ldg128_coherent(src + 1);
      }
      const uint32_t b[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int s = 0; s < S; ++s) mma_bf16_f32(acc[s][nt], a[s][j][0], a[s][j][1], a[s][j][2], a[s][j][3], b[2 * j], b[2 * j + 1]);
    }
  }
  const uint64_t scale_off = (static_cast<uint64_t>(rows) * cols + 255u) & ~static_cast<uint64_t>(255u);
  float sc[S][2];
#pragma unroll
  for (int s = 0; s < S; ++s)
#pragma unroll
    for (int half = 0; half < 2; ++half)
      sc[s][half] = bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(weights[s] + scale_off)[row0 + g + 8 * half]);
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t token = tok0 + nt * 8 + 2 * t + (e & 1);
      const int half = e >> 1;
      if (token >= tokens) continue;
      const uint64_t at = static_cast<uint64_t>(token) * rows + row0 + g + 8 * half;
      if (MODE == 0) {
        const float gv = acc[0][nt][e] * sc[0][half], uv = acc[S - 1][nt][e] * sc[S - 1][half];
        static_cast<__nv_bfloat16 *>(y)[at] = __float2bfloat16_rn(gv / (1.0f + __expf(-gv)) * uv);
      } else {
        static_cast<float *>(y)[at] = acc[0][nt][e] * sc[0][half];
      }
    }
  }
}

// One CTA per token: out = BF16(acc * 2^-32 + sigmoid(x . w_gate) * shared), acc zeroed behind it.
__global__ void __launch_bounds__(256) moe_combine_kernel(long long *acc, const float *shared, const uint16_t *x,
                                                          const uint16_t *w_gate, uint32_t hidden, uint16_t *out) {
  griddep_launch_dependents();
  griddep_wait();
  __shared__ float partial[8];
  const uint32_t t = blockIdx.x;
  float dot = 0.0f;
  for (uint32_t k = threadIdx.x; k < hidden; k += blockDim.x) {
    dot = fmaf(bf16_bits_to_f32(x[static_cast<size_t>(t) * hidden + k]), bf16_bits_to_f32(w_gate[k]), dot);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, o);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = dot;
  __syncthreads();
  float total = 0.0f;
  for (int i = 0; i < 8; ++i) total += partial[i];
  const float gate = 1.0f / (1.0f + __expf(-total));
  for (uint32_t k = threadIdx.x; k < hidden; k += blockDim.x) {
    const size_t at = static_cast<size_t>(t) * hidden + k;
    const float routed = static_cast<float>(static_cast<double>(acc[at]) * (1.0 / 4294967296.0));
    const __nv_bfloat16 o = __float2bfloat16_rn(routed + gate * shared[at]);
    out[at] = *reinterpret_cast<const uint16_t *>(&o);
    acc[at] = 0;
  }
}

bool aligned(const void *p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

const DeviceState *prepared(ErrorSlot &slot, const char *what) {
  const DeviceState *dev = device_state(slot);
  if (dev == nullptr) return nullptr;
  if (!dev->prepared) {
    fail(slot, "%s: the device was not prepared (call ignis_moe_prepare at load)", what);
    return nullptr;
  }
  return dev;
}

int32_t run_experts(const Geometry &g, const void *x, uint32_t tokens, const int32_t *ids, const float *weights, const ignis_moe_slot *slots,
                    const ignis_moe_workspace *workspace, int64_t *acc, void *stream_v, uint32_t limit, uint32_t item_rows,
                    const char *what) {
  ErrorSlot &slot = moe_error();
  if (x == nullptr || ids == nullptr || weights == nullptr || slots == nullptr || workspace == nullptr || acc == nullptr ||
      workspace->base == nullptr) {
    return fail(slot, "%s: NULL argument", what);
  }
  if (tokens == 0 || tokens > limit) return fail(slot, "%s: %u tokens are outside 1..%u", what, tokens, limit);
  if (!aligned(x, 16) || !aligned(workspace->base, 256)) return fail(slot, "%s: x must be 16-byte and the workspace 256-byte aligned", what);
  const DeviceState *dev = prepared(slot, what);
  if (dev == nullptr) return -1;
  const uint32_t tokens_max = workspace->decode_tokens > workspace->prefill_tokens ? workspace->decode_tokens : workspace->prefill_tokens;
  const Layout l = layout_for(g, tokens_max);
  uint8_t *base = static_cast<uint8_t *>(workspace->base);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const uint32_t rows = tokens * g.top_k;
  uint32_t *counts = reinterpret_cast<uint32_t *>(base + l.counts);
  uint32_t *cursor = reinterpret_cast<uint32_t *>(base + l.cursor);
  uint32_t *offsets = reinterpret_cast<uint32_t *>(base + l.offsets);
  uint32_t *n_items = reinterpret_cast<uint32_t *>(base + l.n_items);
  uint32_t *sorted = reinterpret_cast<uint32_t *>(base + l.sorted);
  Item *items = reinterpret_cast<Item *>(base + l.items);
  uint32_t *status = reinterpret_cast<uint32_t *>(base + l.status);
  const bool pdl = dev->pdl != 0;
  cudaError_t err = cudaSuccess;
  if (rows <= kSmallRows && g.experts <= kSmallExperts) {
    err = launch(moe_group_small_kernel, dim3(1), dim3(1024), 0, stream, false, ids, rows, g.experts, item_rows, offsets, n_items, items,
                 reinterpret_cast<Tile *>(base + l.tiles), sorted, status);
    if (err != cudaSuccess) return fail(slot, "%s: grouping launch failed: %s", what, cudaGetErrorString(err));
  } else {
  err = cudaMemsetAsync(counts, 0, l.offsets - l.counts, stream);  // counts and cursor
  if (err != cudaSuccess) return fail(slot, "%s: %s", what, cudaGetErrorString(err));
  const uint32_t grid_rows = (rows + 255u) / 256u < 1184u ? (rows + 255u) / 256u : 1184u;
  err = launch(moe_count_kernel, dim3(grid_rows), dim3(256), 0, stream, false, ids, rows, g.experts, counts, status);
  if (err == cudaSuccess) err = launch(moe_scan_kernel, dim3(1), dim3(1024), 0, stream, pdl, static_cast<const uint32_t *>(counts), g.experts, item_rows, offsets, n_items, items, reinterpret_cast<Tile *>(base + l.tiles));
  if (err == cudaSuccess) err = launch(moe_scatter_kernel, dim3(grid_rows), dim3(256), 0, stream, pdl, ids, rows, g.experts, static_cast<const uint32_t *>(offsets), cursor, sorted);
  if (err != cudaSuccess) return fail(slot, "%s: grouping launch failed: %s", what, cudaGetErrorString(err));
  }

  ExpertParams p = {};
  p.ids = ids;
  p.slots = slots;
  p.items = items;
  p.tiles = reinterpret_cast<const Tile *>(base + l.tiles);
  p.n_items = n_items;
  p.sorted = sorted;
  p.x = static_cast<const uint16_t *>(x);
  p.weights = weights;
  p.frag_in = reinterpret_cast<uint2 *>(base + l.frag_in);
  p.scale_in = reinterpret_cast<float2 *>(base + l.scale_in);
  p.gu = reinterpret_cast<float *>(base + l.gu);
  p.frag_h = reinterpret_cast<uint2 *>(base + l.frag_h);
  p.scale_h = reinterpret_cast<float2 *>(base + l.scale_h);
  p.down_rows = reinterpret_cast<float *>(base + l.down_rows);
  p.acc = reinterpret_cast<long long *>(acc);
  p.status = status;
  p.hidden = g.hidden;
  p.inter = g.inter;
  p.top_k = g.top_k;
  p.experts = g.experts;
  // Grids are sized for the worst case the host can know (the grouping happened on the device);
  // CTAs beyond the item or tile count return at once.
  const uint32_t items_max = items_bound(g, rows, item_rows);
  if (item_rows == kMoeTcItemRows) {   // the tensor-core route: items of up to 256 rows
    return moe_tc_experts(slot, *dev, p, rows, items_max, offsets, stream, what);
  }
  const uint32_t tiles_max = items_bound(g, rows, 8u);
  const bool wide = item_rows > 8u;
  for (int phase = 0; phase < 2; ++phase) {
    const uint32_t col_blocks = (phase == 0 ? 2u * g.inter : g.hidden) / 128u;
    err = phase == 0 ? launch(moe_rotate_kernel<0>, dim3(tiles_max), dim3(kThreads), 0, stream, pdl, p)
                     : launch(moe_rotate_kernel<1>, dim3(tiles_max), dim3(kThreads), 0, stream, pdl, p);
    if (err != cudaSuccess) return fail(slot, "%s: rotation launch failed: %s", what, cudaGetErrorString(err));
    const dim3 grid(items_max * col_blocks);
    if (phase == 0) {
      err = wide ? launch(moe_experts_kernel<0, 8>, grid, dim3(kThreads), 0, stream, pdl, p)
                 : launch(moe_experts_kernel<0, 1>, grid, dim3(kThreads), 0, stream, pdl, p);
    } else {
      err = wide ? launch(moe_experts_kernel<1, 8>, grid, dim3(kThreads), 0, stream, pdl, p)
                 : launch(moe_experts_kernel<1, 1>, grid, dim3(kThreads), 0, stream, pdl, p);
    }
    if (err != cudaSuccess) return fail(slot, "%s: expert launch failed: %s", what, cudaGetErrorString(err));
  }
  return 0;
}

}  // namespace

int32_t prepare_moe_kernels(ErrorSlot &slot) {
  const cudaError_t err = cudaFuncSetAttribute(moe_router_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
  if (err != cudaSuccess) return fail(slot, "ignis_moe_prepare: %s", cudaGetErrorString(err));
  if (moe_tc_prepare(slot) != 0) return -1;
  return moe_fp8_tc_prepare(slot);
}
}  // namespace b200q

using namespace b200q;

extern "C" {

int32_t b200q_moe_set_geometry(uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t top_k) {
  const Geometry g = {hidden, inter, experts, top_k};
  if (check_geometry(moe_error(), &g, "b200q_moe_set_geometry") != 0) return -1;
  g_default = g;
  return 0;
}

int32_t b200q_moe_record_bytes(const b200q_moe_geometry *geometry, uint32_t projection, uint32_t k2, uint64_t *bytes) {
  ErrorSlot &slot = moe_error();
  if (check_geometry(slot, geometry, "ignis_moe_record_bytes") != 0) return -1;
  const Geometry &g_geo = *geometry;
  if (bytes == nullptr) return fail(slot, "ignis_moe_record_bytes: bytes is NULL");
  if (projection > IGNIS_MOE_PROJ_DOWN) return fail(slot, "ignis_moe_record_bytes: unknown projection %u", projection);
  if (!(k2 == 4 || k2 == 5 || k2 == 6 || k2 == 8)) return fail(slot, "ignis_moe_record_bytes: k2 = %u is not one of 4, 5, 6, 8", k2);
  const uint64_t in = projection == IGNIS_MOE_PROJ_GATE_UP ? g_geo.hidden : g_geo.inter;
  const uint64_t out = projection == IGNIS_MOE_PROJ_GATE_UP ? 2ull * g_geo.inter : g_geo.hidden;
  const uint64_t data = in * out * k2 / 16u + 2u * in + 2u * out;
  *bytes = (data + 4095u) & ~static_cast<uint64_t>(4095u);
  return 0;
}

int32_t ignis_moe_trellis_reconstruct(const void *trellis, uint32_t k2, uint32_t in, uint32_t out, void *w_f16, void *stream) {
  return trellis_reconstruct_raw(moe_error(), "ignis_moe_trellis_reconstruct", trellis, k2, in, out, 0, w_f16, stream);
}

int32_t ignis_moe_prepare(void) { return prepare_all(moe_error()); }

uint64_t b200q_moe_workspace_bytes(const b200q_moe_geometry *geometry, uint32_t decode_tokens, uint32_t prefill_tokens) {
  if (check_geometry(moe_error(), geometry, "ignis_moe_workspace_bytes") != 0) return 0;
  const Geometry &g_geo = *geometry;
  const uint32_t tokens_max = decode_tokens > prefill_tokens ? decode_tokens : prefill_tokens;
  if (tokens_max == 0 || decode_tokens > IGNIS_MOE_DECODE_MAX_TOKENS) return 0;
  return layout_for(g_geo, tokens_max).total;
}

int32_t b200q_moe_workspace_init(const b200q_moe_geometry *geometry, const struct ignis_moe_workspace *workspace, int64_t *acc, void *stream) {
  ErrorSlot &slot = moe_error();
  if (check_geometry(slot, geometry, "ignis_moe_workspace_init") != 0) return -1;
  const Geometry &g_geo = *geometry;
  if (workspace == nullptr || workspace->base == nullptr || acc == nullptr) return fail(slot, "ignis_moe_workspace_init: NULL argument");
  if (!aligned(workspace->base, 256)) return fail(slot, "ignis_moe_workspace_init: base is not 256-byte aligned");
  if (ignis_moe_prepare() != 0) return -1;
  const uint32_t tokens_max = workspace->decode_tokens > workspace->prefill_tokens ? workspace->decode_tokens : workspace->prefill_tokens;
  if (tokens_max == 0) return fail(slot, "ignis_moe_workspace_init: the workspace describes no tokens");
  const Layout l = layout_for(g_geo, tokens_max);
  cudaError_t err = cudaMemsetAsync(workspace->base, 0, l.sorted, static_cast<cudaStream_t>(stream));  // status, counters
  if (err == cudaSuccess) err = cudaMemsetAsync(acc, 0, sizeof(int64_t) * tokens_max * g_geo.hidden, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(slot, "ignis_moe_workspace_init: %s", cudaGetErrorString(err));
  return 0;
}

int32_t b200q_moe_plan_bytes(const b200q_moe_geometry *geometry, uint32_t decode_tokens, uint32_t prefill_tokens, struct ignis_moe_plan *plan) {
  ErrorSlot &slot = moe_error();
  if (plan == nullptr) return fail(slot, "ignis_moe_plan_bytes: plan is NULL");
  if (check_geometry(slot, geometry, "ignis_moe_plan_bytes") != 0) return -1;
  const Geometry &g_geo = *geometry;
  const uint64_t ws = b200q_moe_workspace_bytes(geometry, decode_tokens, prefill_tokens);
  if (ws == 0) return fail(slot, "ignis_moe_plan_bytes: no tokens, or more than %d decode tokens", IGNIS_MOE_DECODE_MAX_TOKENS);
  const uint64_t mx = decode_tokens > prefill_tokens ? decode_tokens : prefill_tokens;
  plan->workspace = ws;
  plan->acc = mx * g_geo.hidden * 8u;
  plan->router = mx * g_geo.top_k * 4u + mx * g_geo.top_k * 4u + mx * g_geo.experts * 4u;
  plan->shared = mx * g_geo.inter * 2u + mx * g_geo.hidden * 4u;
  plan->total = align256(plan->workspace) + align256(plan->acc) + align256(plan->router) + align256(plan->shared);
  return 0;
}

int32_t b200q_moe_router_logits(const b200q_moe_geometry *geometry, const void *x, uint32_t tokens, const void *w_router, float *logits,
                                void *stream) {
  ErrorSlot &slot = moe_error();
  if (check_geometry(slot, geometry, "ignis_moe_router_logits") != 0) return -1;
  const Geometry &g_geo = *geometry;
  if (x == nullptr || w_router == nullptr || logits == nullptr) return fail(slot, "ignis_moe_router_logits: NULL argument");
  if (tokens == 0) return fail(slot, "ignis_moe_router_logits: tokens must be positive");
  if (!aligned(x, 16) || !aligned(w_router, 16)) return fail(slot, "ignis_moe_router_logits: x and w_router must be 16-byte aligned");
  const DeviceState *dev = prepared(slot, "ignis_moe_router_logits");
  if (dev == nullptr) return -1;
  const cudaError_t err = launch(moe_router_logits_kernel, dim3(tokens), dim3(256), g_geo.hidden * sizeof(float),
                                 static_cast<cudaStream_t>(stream), dev->pdl != 0, static_cast<const uint16_t *>(x),
                                 static_cast<const uint16_t *>(w_router), g_geo.hidden, g_geo.experts, logits);
  if (err != cudaSuccess) return fail(slot, "ignis_moe_router_logits: launch failed: %s", cudaGetErrorString(err));
  return 0;
}

int32_t b200q_moe_router(const b200q_moe_geometry *geometry, const void *x, uint32_t tokens, const void *w_router, int32_t *ids,
                         float *weights, float *logits, void *stream) {
  ErrorSlot &slot = moe_error();
  if (ids == nullptr || weights == nullptr) return fail(slot, "ignis_moe_router: NULL argument");
  if (b200q_moe_router_logits(geometry, x, tokens, w_router, logits, stream) != 0) return -1;
  const Geometry &g_geo = *geometry;
  const DeviceState *dev = prepared(slot, "ignis_moe_router");
  if (dev == nullptr) return -1;
  const cudaError_t err = launch(moe_router_select_kernel, dim3((tokens + 7u) / 8u), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                 dev->pdl != 0, static_cast<const float *>(logits), tokens, g_geo.experts, g_geo.top_k, ids, weights);
  if (err != cudaSuccess) return fail(slot, "ignis_moe_router: launch failed: %s", cudaGetErrorString(err));
  return 0;
}

int32_t b200q_moe_experts_decode(const b200q_moe_geometry *geometry, const void *x, uint32_t tokens, const int32_t *ids,
                                 const float *weights, const struct ignis_moe_slot *slots,
                                 const struct ignis_moe_workspace *workspace, int64_t *acc, void *stream) {
  if (check_geometry(moe_error(), geometry, "ignis_moe_experts_decode") != 0) return -1;
  const uint32_t limit = workspace != nullptr ? workspace->decode_tokens : 0u;
  return run_experts(*geometry, x, tokens, ids, weights, slots, workspace, acc, stream, limit, 8u, "ignis_moe_experts_decode");
}

int32_t b200q_moe_experts_prefill(const b200q_moe_geometry *geometry, const void *x, uint32_t tokens, const int32_t *ids,
                                  const float *weights, const struct ignis_moe_slot *slots,
                                  const struct ignis_moe_workspace *workspace, int64_t *acc, void *stream) {
  if (check_geometry(moe_error(), geometry, "ignis_moe_experts_prefill") != 0) return -1;
  const uint32_t limit = workspace != nullptr ? workspace->prefill_tokens : 0u;
  // up to 8 tokens the decode entry's item size; up to 64 tokens items of 64 rows on the warp-level
  // MMAs; beyond, items of 256 rows on the tensor cores (B200Q_MOE_TC = 0 keeps the warp-level kernels)
  const DeviceState *dev = device_state(moe_error());
  const bool tc = dev != nullptr && dev->prepared && dev->moe_tc != 0 && tokens > 64u;
  return run_experts(*geometry, x, tokens, ids, weights, slots, workspace, acc, stream, limit, tokens > 8u ? (tc ? kMoeTcItemRows : 64u) : 8u,
                     "ignis_moe_experts_prefill");
}

int32_t ignis_moe_decode_cluster_size(void) { return 0; }

int32_t b200q_moe_shared_expert(const b200q_moe_geometry *geometry, const void *gate, const void *up, const void *down, const void *x,
                                uint32_t tokens, void *h, float *shared, void *stream) {
  ErrorSlot &slot = moe_error();
  if (check_geometry(slot, geometry, "ignis_moe_shared_expert") != 0) return -1;
  const Geometry &g_geo = *geometry;
  if (gate == nullptr || up == nullptr || down == nullptr || x == nullptr || h == nullptr || shared == nullptr) {
    return fail(slot, "ignis_moe_shared_expert: NULL argument");
  }
  if (tokens == 0) return fail(slot, "ignis_moe_shared_expert: tokens must be positive");
  if (!aligned(gate, 16) || !aligned(up, 16) || !aligned(down, 16) || !aligned(x, 16) || !aligned(h, 8)) {
    return fail(slot, "ignis_moe_shared_expert: weights and x must be 16-byte aligned, h 8-byte aligned");
  }
  const DeviceState *dev = prepared(slot, "ignis_moe_shared_expert");
  if (dev == nullptr) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err;
  if (moe_fp8_tc_takes(*dev, g_geo.hidden, g_geo.inter, tokens, x, h)) {  // wide calls: tcgen05
    err = moe_fp8_tc_shared_expert(*dev, static_cast<const uint8_t *>(gate), static_cast<const uint8_t *>(up),
                                   static_cast<const uint8_t *>(down), static_cast<const uint16_t *>(x), tokens, g_geo.hidden, g_geo.inter, h,
                                   shared, s);
  } else if (tokens > 8u) {  // some tokens: warp-level MMAs, 64 tokens a CTA
    const uint32_t token_blocks = (tokens + 63u) / 64u;
    err = launch(moe_fp8_gemm_kernel<0>, dim3((g_geo.inter + 127u) / 128u, token_blocks), dim3(256), 0, s, dev->pdl != 0,
                 static_cast<const uint8_t *>(gate), static_cast<const uint8_t *>(up), g_geo.inter, g_geo.hidden,
                 static_cast<const uint16_t *>(x), tokens, h);
    if (err == cudaSuccess) {
      err = launch(moe_fp8_gemm_kernel<1>, dim3((g_geo.hidden + 127u) / 128u, token_blocks), dim3(256), 0, s, dev->pdl != 0,
                   static_cast<const uint8_t *>(down), static_cast<const uint8_t *>(down), g_geo.hidden, g_geo.inter,
                   static_cast<const uint16_t *>(h), tokens, static_cast<void *>(shared));
    }
  } else {
    err = launch(moe_fp8_rows_kernel<0>, dim3((g_geo.inter + 7u) / 8u), dim3(256), 0, s, dev->pdl != 0,
                 static_cast<const uint8_t *>(gate), static_cast<const uint8_t *>(up), g_geo.inter, g_geo.hidden,
                 static_cast<const uint16_t *>(x), tokens, h);
    if (err == cudaSuccess) {
      err = launch(moe_fp8_rows_kernel<1>, dim3((g_geo.hidden + 7u) / 8u), dim3(256), 0, s, dev->pdl != 0,
                   static_cast<const uint8_t *>(down), static_cast<const uint8_t *>(down), g_geo.hidden, g_geo.inter,
                   static_cast<const uint16_t *>(h), tokens, static_cast<void *>(shared));
    }
  }
  if (err != cudaSuccess) return fail(slot, "ignis_moe_shared_expert: launch failed: %s", cudaGetErrorString(err));
  return 0;
}

int32_t b200q_moe_combine(const b200q_moe_geometry *geometry, int64_t *acc, const float *shared, const void *x, const void *w_gate,
                          uint32_t tokens, void *out, void *stream) {
  ErrorSlot &slot = moe_error();
  if (check_geometry(slot, geometry, "ignis_moe_combine") != 0) return -1;
  const Geometry &g_geo = *geometry;
  if (acc == nullptr || shared == nullptr || x == nullptr || w_gate == nullptr || out == nullptr) {
    return fail(slot, "ignis_moe_combine: NULL argument");
  }
  if (tokens == 0) return fail(slot, "ignis_moe_combine: tokens must be positive");
  const DeviceState *dev = prepared(slot, "ignis_moe_combine");
  if (dev == nullptr) return -1;
  const cudaError_t err = launch(moe_combine_kernel, dim3(tokens), dim3(256), 0, static_cast<cudaStream_t>(stream), dev->pdl != 0,
                                 reinterpret_cast<long long *>(acc), shared, static_cast<const uint16_t *>(x),
                                 static_cast<const uint16_t *>(w_gate), g_geo.hidden, static_cast<uint16_t *>(out));
  if (err != cudaSuccess) return fail(slot, "ignis_moe_combine: launch failed: %s", cudaGetErrorString(err));
  return 0;
}

// ---- the reference's own entry points: the same calls at the default geometry -----------------------
int32_t ignis_moe_record_bytes(uint32_t projection, uint32_t k2, uint64_t *bytes) {
  return b200q_moe_record_bytes(&g_default, projection, k2, bytes);
}
uint64_t ignis_moe_workspace_bytes(uint32_t decode_tokens, uint32_t prefill_tokens) {
  return b200q_moe_workspace_bytes(&g_default, decode_tokens, prefill_tokens);
}
int32_t ignis_moe_workspace_init(const struct ignis_moe_workspace *workspace, int64_t *acc, void *stream) {
  return b200q_moe_workspace_init(&g_default, workspace, acc, stream);
}
int32_t ignis_moe_plan_bytes(uint32_t decode_tokens, uint32_t prefill_tokens, struct ignis_moe_plan *plan) {
  return b200q_moe_plan_bytes(&g_default, decode_tokens, prefill_tokens, plan);
}
int32_t ignis_moe_router_logits(const void *x, uint32_t tokens, const void *w_router, float *logits, void *stream) {
  return b200q_moe_router_logits(&g_default, x, tokens, w_router, logits, stream);
}
int32_t ignis_moe_router(const void *x, uint32_t tokens, const void *w_router, int32_t *ids, float *weights, float *logits,
                         void *stream) {
  return b200q_moe_router(&g_default, x, tokens, w_router, ids, weights, logits, stream);
}
int32_t ignis_moe_experts_decode(const void *x, uint32_t tokens, const int32_t *ids, const float *weights,
                                 const struct ignis_moe_slot *slots, const struct ignis_moe_workspace *workspace,
                                 int64_t *acc, void *stream) {
  return b200q_moe_experts_decode(&g_default, x, tokens, ids, weights, slots, workspace, acc, stream);
}
int32_t ignis_moe_experts_prefill(const void *x, uint32_t tokens, const int32_t *ids, const float *weights,
                                  const struct ignis_moe_slot *slots, const struct ignis_moe_workspace *workspace,
                                  int64_t *acc, void *stream) {
  return b200q_moe_experts_prefill(&g_default, x, tokens, ids, weights, slots, workspace, acc, stream);
}
int32_t ignis_moe_shared_expert(const void *gate, const void *up, const void *down, const void *x, uint32_t tokens, void *h,
                                float *shared, void *stream) {
  return b200q_moe_shared_expert(&g_default, gate, up, down, x, tokens, h, shared, stream);
}
int32_t ignis_moe_combine(int64_t *acc, const float *shared, const void *x, const void *w_gate, uint32_t tokens, void *out,
                          void *stream) {
  return b200q_moe_combine(&g_default, acc, shared, x, w_gate, tokens, out, stream);
}

int32_t ignis_moe_stream_sync(void *stream) {
  const cudaError_t err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(moe_error(), "ignis_moe_stream_sync: %s", cudaGetErrorString(err));
  return 0;
}

int32_t ignis_moe_workspace_status(const struct ignis_moe_workspace *workspace, void *stream, uint32_t *status) {
  ErrorSlot &slot = moe_error();
  if (workspace == nullptr || workspace->base == nullptr || status == nullptr) return fail(slot, "ignis_moe_workspace_status: NULL argument");
  uint32_t words[2] = {0u, 0u};   // [0] the expert kernels' bits, [1] bounded waits of the tensor-core kernels that ran out
  uint32_t shared_expert = 0u;    // the same for the shared expert's tensor-core kernels (no workspace of their own)
  cudaError_t err = cudaMemcpyAsync(words, workspace->base, sizeof(words), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (err == cudaSuccess) err = moe_fp8_tc_status(&shared_expert, static_cast<cudaStream_t>(stream));
  if (err == cudaSuccess) err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(slot, "ignis_moe_workspace_status: %s", cudaGetErrorString(err));
  *status = words[0] | ((words[1] | shared_expert) != 0u ? kStatusTcWait : 0u);
  return 0;
}

const char *ignis_moe_last_error(void) { return moe_error().text; }

}  // extern "C"
