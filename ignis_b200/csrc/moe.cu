// Flash-Next mixture-of-experts ops: the entry points of include/ignis_moe.h and their kernels.
//
// Routed experts (the reference's ignis_moe_experts_prefill / _decode, kernel/src/moe_prefill.cu:
// 41-492 and moe_decode.cu:325-399): the (token, rank) assignments are grouped by expert on the
// device (count, scan, scatter), cut into work items of at most 8 rows of one expert, and two
// grouped launches follow - gate/up with the SwiGLU epilogue into h (fp32 [rows][inter]), then
// down with the routing weight applied and the result added to `acc` in 64-bit fixed point
// (2^-32), so the sum does not depend on arrival order. Each item's CTA cluster runs the dense
// trellis linear's machinery (trellis_device.cuh): rotation of the rows into fp16 fragments,
// tiles decoded in registers straight into MMA fragments, fp32 accumulation, shared-memory and
// distributed-shared-memory reductions, output Hadamard and svh.
//
// Nothing here traps or spins: a bad expert id, an absent record or an out-of-range contribution
// is skipped and recorded in the workspace's status word.
#include "../../include/ignis_moe.h"

#include "trellis_device.cuh"

#include <mutex>

namespace b200q {
namespace {

using namespace trellis_dev;

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr uint32_t kStatusBadExpert = 1u, kStatusAbsentRecord = 2u, kStatusRange = 4u;

struct Geometry {
  uint32_t hidden = IGNIS_MOE_HIDDEN, inter = IGNIS_MOE_INTERMEDIATE, experts = IGNIS_MOE_EXPERTS, top_k = IGNIS_MOE_TOP_K;
};
Geometry g_geo;

struct Item {
  uint32_t expert, first, count, pad;
};

// Workspace regions for `tokens_max` tokens.
struct Layout {
  uint64_t status, counts, cursor, offsets, n_items, sorted, items, h, total;
  uint32_t rows_max, items_max;
};

uint64_t align256(uint64_t v) { return (v + 255u) & ~static_cast<uint64_t>(255u); }

Layout layout_for(const Geometry &g, uint32_t tokens_max) {
  Layout l = {};
  l.rows_max = tokens_max * g.top_k;
  l.items_max = (l.rows_max + 7u) / 8u + (g.experts < l.rows_max ? g.experts : l.rows_max);
  uint64_t at = 0;
  l.status = at; at += 256;
  l.counts = at; at = align256(at + 4ull * g.experts);
  l.cursor = at; at = align256(at + 4ull * g.experts);
  l.offsets = at; at = align256(at + 4ull * (g.experts + 1));
  l.n_items = at; at += 256;
  l.sorted = at; at = align256(at + 4ull * l.rows_max);
  l.items = at; at = align256(at + 16ull * l.items_max);
  l.h = at; at = align256(at + 4ull * l.rows_max * g.inter);
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
      atomicOr(status, kStatusBadExpert);
    } else {
      atomicAdd(&counts[e], 1u);
    }
  }
}

// One CTA: exclusive scans of the per-expert row counts and item counts, then the item list.
__global__ void __launch_bounds__(1024) moe_scan_kernel(const uint32_t *counts, uint32_t experts, uint32_t *offsets,
                                                        uint32_t *n_items, Item *items) {
  griddep_launch_dependents();
  griddep_wait();
  __shared__ uint32_t row_sum[1024], item_sum[1024];
  const uint32_t per = (experts + 1023u) / 1024u;  // experts per thread, consecutive
  const uint32_t e0 = threadIdx.x * per;
  uint32_t rows = 0, its = 0;
  for (uint32_t e = e0; e < e0 + per && e < experts; ++e) {
    rows += counts[e];
    its += (counts[e] + 7u) / 8u;
  }
  row_sum[threadIdx.x] = rows;
  item_sum[threadIdx.x] = its;
  __syncthreads();
  for (uint32_t d = 1; d < 1024; d <<= 1) {  // Hillis-Steele inclusive scan
    const uint32_t r = threadIdx.x >= d ? row_sum[threadIdx.x - d] : 0u;
    const uint32_t i = threadIdx.x >= d ? item_sum[threadIdx.x - d] : 0u;
    __syncthreads();
    row_sum[threadIdx.x] += r;
    item_sum[threadIdx.x] += i;
    __syncthreads();
  }
  uint32_t row_at = row_sum[threadIdx.x] - rows, item_at = item_sum[threadIdx.x] - its;
  for (uint32_t e = e0; e < e0 + per && e < experts; ++e) {
    offsets[e] = row_at;
    const uint32_t c = counts[e];
    for (uint32_t j = 0; j < c; j += 8) {
      items[item_at++] = Item{e, row_at + j, c - j < 8u ? c - j : 8u, 0u};
    }
    row_at += c;
  }
  if (threadIdx.x == 1023) {
    offsets[experts] = row_sum[1023];
    *n_items = item_sum[1023];
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

// ---- the grouped expert kernel ---------------------------------------------------------------
struct ExpertParams {
  const ignis_moe_slot *slots;
  const Item *items;
  const uint32_t *n_items;
  const uint32_t *sorted;   // row -> assignment index (token * top_k + rank)
  const uint16_t *x;        // BF16 [tokens][hidden]
  const float *weights;     // routing weights [tokens][top_k]
  float *h;                 // fp32 [rows][inter]
  long long *acc;           // int64 [tokens][hidden]
  uint32_t *status;
  uint32_t hidden, inter, top_k, experts;
  uint32_t kc;              // cluster size
  uint32_t slice_cap;       // 128-input blocks of fragments a CTA holds
};

// PHASE 0: gate/up with SwiGLU into h. PHASE 1: down, weighted, into acc.
template <int PHASE>
__global__ void __launch_bounds__(kThreads, 2) moe_experts_kernel(const __grid_constant__ ExpertParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank(), kc = p.kc;
  const uint32_t in = PHASE == 0 ? p.hidden : p.inter;
  const uint32_t out_plane = PHASE == 0 ? 2u * p.inter : p.hidden;   // columns of the stored plane
  const uint32_t col_blocks = (PHASE == 0 ? p.inter : p.hidden) / 128u;
  const uint32_t item_index = blockIdx.x / (col_blocks * kc);
  const uint32_t col_block = (blockIdx.x / kc) % col_blocks;

  griddep_launch_dependents();
  griddep_wait();  // the item list comes from the grouping kernels

  if (item_index >= *p.n_items) return;  // every CTA of a cluster shares the item: a uniform exit
  const Item item = p.items[item_index];
  const ignis_moe_slot slot = p.slots[item.expert * 2u + PHASE];
  const uint32_t k2 = slot.k2;
  if (slot.record == nullptr || !(k2 == 4 || k2 == 5 || k2 == 6 || k2 == 8)) {
    if (threadIdx.x == 0 && rank == 0 && col_block == 0) atomicOr(p.status, kStatusAbsentRecord);
    return;  // uniform over the cluster as well
  }
  const uint32_t *trellis = static_cast<const uint32_t *>(slot.record);
  const uint64_t trellis_bytes = static_cast<uint64_t>(in) * out_plane * k2 / 16u;
  const uint16_t *suh = reinterpret_cast<const uint16_t *>(static_cast<const uint8_t *>(slot.record) + trellis_bytes);
  const uint16_t *svh = suh + in;

  constexpr int sides = PHASE == 0 ? 2 : 1;             // gate and up column blocks share one rotation
  const int side = PHASE == 0 ? warp >> 2 : 0;
  const int warps_per_side = PHASE == 0 ? 4 : 8;
  const int wslot = PHASE == 0 ? (warp & 3) : warp;
  const uint32_t side_col_block = col_block + (side == 1 ? p.inter / 128u : 0u);

  const uint32_t nblk = in / 128u;
  const uint32_t b0 = static_cast<uint32_t>(static_cast<uint64_t>(nblk) * rank / kc);
  const uint32_t b1 = static_cast<uint32_t>(static_cast<uint64_t>(nblk) * (rank + 1) / kc);
  const uint32_t slice = b1 - b0;

  const size_t frag_bytes = static_cast<size_t>(p.slice_cap) * 2048u;
  const size_t red_bytes = static_cast<size_t>(kWarps - sides) * 8 * 32 * 16;
  const size_t region = frag_bytes > red_bytes ? frag_bytes : red_bytes;
  uint2 *xs = reinterpret_cast<uint2 *>(smem_raw);
  float4 *red = reinterpret_cast<float4 *>(smem_raw);
  float4 *part = reinterpret_cast<float4 *>(smem_raw + region);
  float *inv_s = reinterpret_cast<float *>(smem_raw + region + 2 * 8 * 32 * 16);
  float *scale_s = inv_s + static_cast<size_t>(p.slice_cap) * 8;
  __shared__ uint32_t row_assign[8];
  if (threadIdx.x < 8) row_assign[threadIdx.x] = threadIdx.x < item.count ? p.sorted[item.first + threadIdx.x] : 0u;
  __syncthreads();

  // ---- rotate the item's rows into B fragments ----
  {
    const uint32_t units = slice * 8u;
    for (uint32_t u = static_cast<uint32_t>(warp); u < units; u += kWarps) {
      const uint32_t r = u & 7u, bl = u >> 3;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (r < item.count) {
        const size_t k0 = static_cast<size_t>(b0 + bl) * 128u + 4u * lane;
        const uint2 sb = *reinterpret_cast<const uint2 *>(suh + k0);
        const __half2 s01 = *reinterpret_cast<const __half2 *>(&sb.x), s23 = *reinterpret_cast<const __half2 *>(&sb.y);
        if (PHASE == 0) {
          const uint32_t token = row_assign[r] / p.top_k;
          const uint2 xb = ldg64_coherent(p.x + static_cast<size_t>(token) * p.hidden + k0);
          v[0] = bf16_bits_to_f32(xb.x & 0xFFFFu) * __low2float(s01);
          v[1] = __uint_as_float(xb.x & 0xFFFF0000u) * __high2float(s01);
          v[2] = bf16_bits_to_f32(xb.y & 0xFFFFu) * __low2float(s23);
          v[3] = __uint_as_float(xb.y & 0xFFFF0000u) * __high2float(s23);
        } else {
          const uint4 hb = ldg128_coherent(p.h + static_cast<size_t>(item.first + r) * p.inter + k0);
          v[0] = __uint_as_float(hb.x) * __low2float(s01);
          v[1] = __uint_as_float(hb.y) * __high2float(s01);
          v[2] = __uint_as_float(hb.z) * __low2float(s23);
          v[3] = __uint_as_float(hb.w) * __high2float(s23);
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
      const int kt = lane >> 2, k16 = (lane & 3) * 4;
      const int t_first = (k16 & 7) >> 1, reg = k16 >> 3;
      uint32_t *dst = reinterpret_cast<uint32_t *>(xs + (static_cast<size_t>(bl) * 8 + kt) * 32 + r * 4);
      dst[t_first * 2 + reg] = *reinterpret_cast<const uint32_t *>(&h01);
      dst[(t_first + 1) * 2 + reg] = *reinterpret_cast<const uint32_t *>(&h23);
      if (lane == 0) {
        inv_s[bl * 8 + r] = r < item.count ? ldexpf(1.0f, -shift) : 0.0f;
        scale_s[bl * 8 + r] = scale;
      }
    }
  }
  __syncthreads();

  // ---- main loop ----
  float tot[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) tot[j][e] = 0.0f;
  {
    const LaneWindow win = lane_window(k2, lane);
    const uint32_t tile_words = 4u * k2;
    const uint32_t *col_base = trellis + static_cast<uint64_t>(side_col_block) * 8u * tile_words;
    const uint64_t tk_stride = static_cast<uint64_t>(out_plane / 16u) * tile_words;
    const uint32_t blk_first = b0 + static_cast<uint32_t>(wslot);
    switch (k2) {
      case 4: walk_blocks<4>(col_base, tk_stride, win, blk_first, b0, b1, warps_per_side, xs, inv_s, scale_s, lane, tot); break;
      case 5: walk_blocks<5>(col_base, tk_stride, win, blk_first, b0, b1, warps_per_side, xs, inv_s, scale_s, lane, tot); break;
      case 6: walk_blocks<6>(col_base, tk_stride, win, blk_first, b0, b1, warps_per_side, xs, inv_s, scale_s, lane, tot); break;
      default: walk_blocks<8>(col_base, tk_stride, win, blk_first, b0, b1, warps_per_side, xs, inv_s, scale_s, lane, tot); break;
    }
  }

  // ---- reduce the warps of each side, then the cluster ----
  __syncthreads();
  if (wslot > 0) {
    const int rslot = side * (warps_per_side - 1) + (wslot - 1);
#pragma unroll
    for (int j = 0; j < 8; ++j) red[(rslot * 8 + j) * 32 + lane] = make_float4(tot[j][0], tot[j][1], tot[j][2], tot[j][3]);
  }
  __syncthreads();
  if (wslot == 0) {
    for (int o = 1; o < warps_per_side; ++o) {
      const int rslot = side * (warps_per_side - 1) + (o - 1);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 v = red[(rslot * 8 + j) * 32 + lane];
        tot[j][0] += v.x;
        tot[j][1] += v.y;
        tot[j][2] += v.z;
        tot[j][3] += v.w;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) part[(side * 8 + j) * 32 + lane] = make_float4(tot[j][0], tot[j][1], tot[j][2], tot[j][3]);
  }
  cluster_barrier();

  // ---- the first CTA finishes: warp = row of the item, lane = 4 output columns ----
  if (rank == 0 && static_cast<uint32_t>(warp) < item.count) {
    const int r = warp, tq = r >> 1, te = r & 1;
    float v[2][4];
#pragma unroll
    for (int sd = 0; sd < 2; ++sd)
#pragma unroll
      for (int i = 0; i < 4; ++i) v[sd][i] = 0.0f;
#pragma unroll
    for (int sd = 0; sd < sides; ++sd) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 4 * lane + i, j = c >> 4, cc = c & 15;
        const float *src = reinterpret_cast<const float *>(&part[(sd * 8 + j) * 32 + (cc & 7) * 4 + tq]) + te + 2 * (cc >> 3);
        float sum = 0.0f;
        for (uint32_t q = 0; q < kc; ++q) sum += ld_cluster_f32(src, q);
        v[sd][i] = sum;
      }
      hadamard128(v[sd], lane);
      const uint32_t plane_col = (col_block + (sd == 1 ? p.inter / 128u : 0u)) * 128u + 4u * lane;
      const uint2 sv = *reinterpret_cast<const uint2 *>(svh + plane_col);
      const __half2 s01 = *reinterpret_cast<const __half2 *>(&sv.x), s23 = *reinterpret_cast<const __half2 *>(&sv.y);
      v[sd][0] *= __low2float(s01);
      v[sd][1] *= __high2float(s01);
      v[sd][2] *= __low2float(s23);
      v[sd][3] *= __high2float(s23);
    }
    if (PHASE == 0) {
      float4 o;
      o.x = v[0][0] / (1.0f + __expf(-v[0][0])) * v[1][0];
      o.y = v[0][1] / (1.0f + __expf(-v[0][1])) * v[1][1];
      o.z = v[0][2] / (1.0f + __expf(-v[0][2])) * v[1][2];
      o.w = v[0][3] / (1.0f + __expf(-v[0][3])) * v[1][3];
      *reinterpret_cast<float4 *>(p.h + static_cast<size_t>(item.first + r) * p.inter + col_block * 128u + 4u * lane) = o;
    } else {
      const uint32_t a = row_assign[r];
      const uint32_t token = a / p.top_k;
      const float wr = p.weights[a];
      long long *dst = p.acc + static_cast<size_t>(token) * p.hidden + col_block * 128u + 4u * lane;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float c = wr * v[0][i];
        if (!(fabsf(c) < 2147483648.0f)) {  // also catches NaN
          atomicOr(p.status, kStatusRange);
        } else {
          atomicAdd(reinterpret_cast<unsigned long long *>(dst + i),
                    static_cast<unsigned long long>(__double2ll_rn(static_cast<double>(c) * 4294967296.0)));
        }
      }
    }
  }
  cluster_barrier();
}

size_t experts_smem_bytes(uint32_t slice_cap, int sides) {
  const size_t frag_bytes = static_cast<size_t>(slice_cap) * 2048u;
  const size_t red_bytes = static_cast<size_t>(kWarps - sides) * 8 * 32 * 16;
  return (frag_bytes > red_bytes ? frag_bytes : red_bytes) + 2 * 8 * 32 * 16 + static_cast<size_t>(slice_cap) * 8 * 4 * 2;
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

int32_t run_experts(const void *x, uint32_t tokens, const int32_t *ids, const float *weights, const ignis_moe_slot *slots,
                    const ignis_moe_workspace *workspace, int64_t *acc, void *stream_v, uint32_t limit, const char *what) {
  ErrorSlot &slot = moe_error();
  if (x == nullptr || ids == nullptr || weights == nullptr || slots == nullptr || workspace == nullptr || acc == nullptr ||
      workspace->base == nullptr) {
    return fail(slot, "%s: NULL argument", what);
  }
  if (tokens == 0 || tokens > limit) return fail(slot, "%s: %u tokens are outside 1..%u", what, tokens, limit);
  if (!aligned(x, 16) || !aligned(workspace->base, 256)) return fail(slot, "%s: x must be 16-byte and the workspace 256-byte aligned", what);
  const DeviceState *dev = prepared(slot, what);
  if (dev == nullptr) return -1;
  const Geometry g = g_geo;
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
  cudaError_t err = cudaMemsetAsync(counts, 0, l.offsets - l.counts, stream);  // counts and cursor
  if (err != cudaSuccess) return fail(slot, "%s: %s", what, cudaGetErrorString(err));
  const bool pdl = dev->pdl != 0;
  const uint32_t grid_rows = (rows + 255u) / 256u < 1184u ? (rows + 255u) / 256u : 1184u;
  err = launch(moe_count_kernel, dim3(grid_rows), dim3(256), 0, stream, false, ids, rows, g.experts, counts, status);
  if (err == cudaSuccess) err = launch(moe_scan_kernel, dim3(1), dim3(1024), 0, stream, pdl, static_cast<const uint32_t *>(counts), g.experts, offsets, n_items, items);
  if (err == cudaSuccess) err = launch(moe_scatter_kernel, dim3(grid_rows), dim3(256), 0, stream, pdl, ids, rows, g.experts, static_cast<const uint32_t *>(offsets), cursor, sorted);
  if (err != cudaSuccess) return fail(slot, "%s: grouping launch failed: %s", what, cudaGetErrorString(err));

  ExpertParams p = {};
  p.slots = slots;
  p.items = items;
  p.n_items = n_items;
  p.sorted = sorted;
  p.x = static_cast<const uint16_t *>(x);
  p.weights = weights;
  p.h = reinterpret_cast<float *>(base + l.h);
  p.acc = reinterpret_cast<long long *>(acc);
  p.status = status;
  p.hidden = g.hidden;
  p.inter = g.inter;
  p.top_k = g.top_k;
  p.experts = g.experts;
  const uint32_t items_max = (rows + 7u) / 8u + (g.experts < rows ? g.experts : rows);
  for (int phase = 0; phase < 2; ++phase) {
    const uint32_t in = phase == 0 ? g.hidden : g.inter;
    const uint32_t col_blocks = (phase == 0 ? g.inter : g.hidden) / 128u;
    const uint32_t warps = phase == 0 ? 4u : 8u;
    const uint32_t nblk = in / 128u;
    uint32_t kc = (nblk + 2u * warps - 1u) / (2u * warps);  // about two blocks per warp
    if (kc < 1u) kc = 1u;
    if (kc > 8u) kc = 8u;
    p.kc = kc;
    p.slice_cap = (nblk + kc - 1u) / kc;
    const size_t smem = experts_smem_bytes(p.slice_cap, phase == 0 ? 2 : 1);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(items_max * col_blocks * kc, 1, 1);
    config.blockDim = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kc;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = pdl ? 2 : 1;
    err = phase == 0 ? cudaLaunchKernelEx(&config, moe_experts_kernel<0>, p) : cudaLaunchKernelEx(&config, moe_experts_kernel<1>, p);
    if (err != cudaSuccess) return fail(slot, "%s: expert launch failed: %s", what, cudaGetErrorString(err));
  }
  return 0;
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" {

int32_t b200q_moe_set_geometry(uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t top_k) {
  ErrorSlot &slot = moe_error();
  if (hidden == 0 || (hidden % 128u) != 0 || inter == 0 || (inter % 128u) != 0) {
    return fail(slot, "b200q_moe_set_geometry: hidden and inter must be positive multiples of 128");
  }
  if (experts == 0 || experts > 4096u || top_k == 0 || top_k > 32u || top_k > experts) {
    return fail(slot, "b200q_moe_set_geometry: experts must lie in 1..4096 and top_k in 1..min(32, experts)");
  }
  if (hidden / 128u > 8u * 40u || inter / 128u > 8u * 40u) return fail(slot, "b200q_moe_set_geometry: dimension too long");
  g_geo.hidden = hidden;
  g_geo.inter = inter;
  g_geo.experts = experts;
  g_geo.top_k = top_k;
  return 0;
}

int32_t ignis_moe_record_bytes(uint32_t projection, uint32_t k2, uint64_t *bytes) {
  ErrorSlot &slot = moe_error();
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

int32_t ignis_moe_prepare(void) {
  ErrorSlot &slot = moe_error();
  if (prepare_device(slot) != 0) return -1;
  cudaError_t err = cudaFuncSetAttribute(moe_experts_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  if (err == cudaSuccess) err = cudaFuncSetAttribute(moe_experts_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  if (err == cudaSuccess) err = cudaFuncSetAttribute(moe_router_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
  if (err != cudaSuccess) return fail(slot, "ignis_moe_prepare: %s", cudaGetErrorString(err));
  return 0;
}

uint64_t ignis_moe_workspace_bytes(uint32_t decode_tokens, uint32_t prefill_tokens) {
  const uint32_t tokens_max = decode_tokens > prefill_tokens ? decode_tokens : prefill_tokens;
  if (tokens_max == 0 || decode_tokens > IGNIS_MOE_DECODE_MAX_TOKENS) return 0;
  return layout_for(g_geo, tokens_max).total;
}

int32_t ignis_moe_workspace_init(const struct ignis_moe_workspace *workspace, int64_t *acc, void *stream) {
  ErrorSlot &slot = moe_error();
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

int32_t ignis_moe_plan_bytes(uint32_t decode_tokens, uint32_t prefill_tokens, struct ignis_moe_plan *plan) {
  ErrorSlot &slot = moe_error();
  if (plan == nullptr) return fail(slot, "ignis_moe_plan_bytes: plan is NULL");
  const uint64_t ws = ignis_moe_workspace_bytes(decode_tokens, prefill_tokens);
  if (ws == 0) return fail(slot, "ignis_moe_plan_bytes: no tokens, or more than %d decode tokens", IGNIS_MOE_DECODE_MAX_TOKENS);
  const uint64_t mx = decode_tokens > prefill_tokens ? decode_tokens : prefill_tokens;
  plan->workspace = ws;
  plan->acc = mx * g_geo.hidden * 8u;
  plan->router = mx * g_geo.top_k * 4u + mx * g_geo.top_k * 4u + mx * g_geo.experts * 4u;
  plan->shared = mx * g_geo.inter * 2u + mx * g_geo.hidden * 4u;
  plan->total = align256(plan->workspace) + align256(plan->acc) + align256(plan->router) + align256(plan->shared);
  return 0;
}

int32_t ignis_moe_router_logits(const void *x, uint32_t tokens, const void *w_router, float *logits, void *stream) {
  ErrorSlot &slot = moe_error();
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

int32_t ignis_moe_router(const void *x, uint32_t tokens, const void *w_router, int32_t *ids, float *weights, float *logits,
                         void *stream) {
  ErrorSlot &slot = moe_error();
  if (ids == nullptr || weights == nullptr) return fail(slot, "ignis_moe_router: NULL argument");
  if (ignis_moe_router_logits(x, tokens, w_router, logits, stream) != 0) return -1;
  const DeviceState *dev = prepared(slot, "ignis_moe_router");
  if (dev == nullptr) return -1;
  const cudaError_t err = launch(moe_router_select_kernel, dim3((tokens + 7u) / 8u), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                 dev->pdl != 0, static_cast<const float *>(logits), tokens, g_geo.experts, g_geo.top_k, ids, weights);
  if (err != cudaSuccess) return fail(slot, "ignis_moe_router: launch failed: %s", cudaGetErrorString(err));
  return 0;
}

int32_t ignis_moe_experts_decode(const void *x, uint32_t tokens, const int32_t *ids, const float *weights,
                                 const struct ignis_moe_slot *slots, const struct ignis_moe_workspace *workspace,
                                 int64_t *acc, void *stream) {
  const uint32_t limit = workspace != nullptr ? workspace->decode_tokens : 0u;
  return run_experts(x, tokens, ids, weights, slots, workspace, acc, stream, limit, "ignis_moe_experts_decode");
}

int32_t ignis_moe_experts_prefill(const void *x, uint32_t tokens, const int32_t *ids, const float *weights,
                                  const struct ignis_moe_slot *slots, const struct ignis_moe_workspace *workspace,
                                  int64_t *acc, void *stream) {
  const uint32_t limit = workspace != nullptr ? workspace->prefill_tokens : 0u;
  return run_experts(x, tokens, ids, weights, slots, workspace, acc, stream, limit, "ignis_moe_experts_prefill");
}

int32_t ignis_moe_decode_cluster_size(void) { return 0; }

int32_t ignis_moe_shared_expert(const void *gate, const void *up, const void *down, const void *x, uint32_t tokens, void *h,
                                float *shared, void *stream) {
  ErrorSlot &slot = moe_error();
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
  cudaError_t err = launch(moe_fp8_rows_kernel<0>, dim3((g_geo.inter + 7u) / 8u), dim3(256), 0, s, dev->pdl != 0,
                           static_cast<const uint8_t *>(gate), static_cast<const uint8_t *>(up), g_geo.inter, g_geo.hidden,
                           static_cast<const uint16_t *>(x), tokens, h);
  if (err == cudaSuccess) {
    err = launch(moe_fp8_rows_kernel<1>, dim3((g_geo.hidden + 7u) / 8u), dim3(256), 0, s, dev->pdl != 0,
                 static_cast<const uint8_t *>(down), static_cast<const uint8_t *>(down), g_geo.hidden, g_geo.inter,
                 static_cast<const uint16_t *>(h), tokens, static_cast<void *>(shared));
  }
  if (err != cudaSuccess) return fail(slot, "ignis_moe_shared_expert: launch failed: %s", cudaGetErrorString(err));
  return 0;
}

int32_t ignis_moe_combine(int64_t *acc, const float *shared, const void *x, const void *w_gate, uint32_t tokens, void *out,
                          void *stream) {
  ErrorSlot &slot = moe_error();
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

int32_t ignis_moe_stream_sync(void *stream) {
  const cudaError_t err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(moe_error(), "ignis_moe_stream_sync: %s", cudaGetErrorString(err));
  return 0;
}

int32_t ignis_moe_workspace_status(const struct ignis_moe_workspace *workspace, void *stream, uint32_t *status) {
  ErrorSlot &slot = moe_error();
  if (workspace == nullptr || workspace->base == nullptr || status == nullptr) return fail(slot, "ignis_moe_workspace_status: NULL argument");
  cudaError_t err = cudaMemcpyAsync(status, workspace->base, sizeof(uint32_t), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (err == cudaSuccess) err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(slot, "ignis_moe_workspace_status: %s", cudaGetErrorString(err));
  return 0;
}

const char *ignis_moe_last_error(void) { return moe_error().text; }

}  // extern "C"
