// The routed experts of wide calls on the tensor cores.
//
// Stands where the reference's prefill entry multiplies items of up to 64 rows with warp-level MMAs
// (kernel/src/moe_prefill.cu:252-262, kernels :405 and :421). Under skewed routing a few experts see
// hundreds of rows; here a work item is up to 256 sorted rows of one expert, and every item is
// multiplied with its expert's record by the kernel core of trellis_tc.cuh: the rows rotated once
// into plain fp16 rows with one scale per row, the record's trellis tiles decoded into swizzled
// shared memory, tcgen05.mma kind::f16 with the accumulator in tensor memory, and the output
// Hadamard in registers. Five launches behind the grouping:
//
//   moe_tc_rotate_kernel<0>   x o suh (the row's expert's gate|up record), Hadamard, fp16 rows
//   moe_tc_gemm_kernel<0>     rows x gate|up record -> gu fp32 [row][2 inter] (gate columns, then up)
//   moe_tc_rotate_kernel<1>   silu(g) u o suh (the down record), Hadamard, fp16 rows
//   moe_tc_gemm_kernel<1>     rows x down record, times the routing weight -> fp32 [token][rank][hidden]
//   moe_tc_fold_kernel        a token's products as 2^-32 fixed-point integers, summed, added to the
//                             token's int64 accumulator row (84 M atomic additions into the
//                             accumulator from the product's epilogue took two thirds of that launch)
//
// A row's arithmetic does not depend on the item it is in or on the rows beside it, so results are
// reproducible bit for bit whatever the grouping order.
#include "moe_internal.cuh"
#include "trellis_tc.cuh"

namespace b200q {
namespace {

using namespace trellis_tc;

constexpr uint32_t kRotateThreads = 64;

// One CTA of two warps per sorted row: the row's `in` values times the expert's suh, the 128-wide
// Hadamard per block (a warp per block), one power-of-two scale per row (largest magnitude in
// [2^13, 2^14)), fp16. PHASE 0 reads the token's activations, PHASE 1 silu(g) u of the row's gate|up
// products. The kernel is bound by instruction issue, and what every warp repeats for its row (the
// walk to the expert's record, the row maximum, the scale) weighs as much as the transforms: hence
// two warps a row (eight: 147 + 132 us for 40 960 rows of 2048 and 768 inputs; four: 106 + 91; two: a
// further 1.4 % on the step), and the scale from the maximum's exponent bits.
template <int PHASE>
__global__ void __launch_bounds__(kRotateThreads) moe_tc_rotate_kernel(const __grid_constant__ ExpertParams p, const uint32_t *offsets) {
  extern __shared__ __align__(16) float rot[];
  __shared__ float warp_max[kRotateThreads / 32];
  griddep_launch_dependents();
  griddep_wait();
  const uint32_t row = blockIdx.x;
  if (row >= offsets[p.experts]) return;   // fewer rows than the launch was sized for
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t a = p.sorted[row];
  const uint32_t expert = static_cast<uint32_t>(p.ids[a]);
  const ignis_moe_slot slot = p.slots[expert * 2u + PHASE];
  const uint32_t in = PHASE == 0 ? p.hidden : p.inter;
  uint16_t *dst = reinterpret_cast<uint16_t *>(PHASE == 0 ? p.frag_in : p.frag_h) + static_cast<size_t>(row) * in;
  float *inv = reinterpret_cast<float *>(PHASE == 0 ? p.scale_in : p.scale_h) + row;
  if (slot.record == nullptr || !(slot.k2 == 4 || slot.k2 == 5 || slot.k2 == 6 || slot.k2 == 8)) {
    // an absent record: the product kernel flags it and skips the item; leave finite rows behind
    for (uint32_t i = threadIdx.x * 4u; i < in; i += 4u * kRotateThreads) *reinterpret_cast<uint2 *>(dst + i) = make_uint2(0u, 0u);
    if (threadIdx.x == 0) *inv = 0.0f;
    return;
  }
  const uint32_t out_plane = PHASE == 0 ? 2u * p.inter : p.hidden;
  const uint64_t trellis_bytes = static_cast<uint64_t>(in) * out_plane * slot.k2 / 16u;
  const uint16_t *suh = reinterpret_cast<const uint16_t *>(static_cast<const uint8_t *>(slot.record) + trellis_bytes);
  const uint32_t token = a / p.top_k;
  const uint32_t nblk = in / 128u;
  float m = 0.0f;
  for (uint32_t bl = static_cast<uint32_t>(warp); bl < nblk; bl += kRotateThreads / 32u) {
    const size_t k0 = static_cast<size_t>(bl) * 128u + 4u * lane;
    const uint2 sb = *reinterpret_cast<const uint2 *>(suh + k0);
    const __half2 s01 = *reinterpret_cast<const __half2 *>(&sb.x), s23 = *reinterpret_cast<const __half2 *>(&sb.y);
    const float sv[4] = {__low2float(s01), __high2float(s01), __low2float(s23), __high2float(s23)};
    float v[4];
    if (PHASE == 0) {
      const uint2 xb = ldg64_coherent(p.x + static_cast<size_t>(token) * p.hidden + k0);
      v[0] = bf16_bits_to_f32(xb.x & 0xFFFFu) * sv[0];
      v[1] = __uint_as_float(xb.x & 0xFFFF0000u) * sv[1];
      v[2] = bf16_bits_to_f32(xb.y & 0xFFFFu) * sv[2];
      v[3] = __uint_as_float(xb.y & 0xFFFF0000u) * sv[3];
    } else {
      const float *g = p.gu + static_cast<size_t>(row) * 2u * p.inter + k0;
      const uint4 gb = ldg128_coherent(g), ub = ldg128_coherent(g + p.inter);
      const float gv[4] = {__uint_as_float(gb.x), __uint_as_float(gb.y), __uint_as_float(gb.z), __uint_as_float(gb.w)};
      const float uv[4] = {__uint_as_float(ub.x), __uint_as_float(ub.y), __uint_as_float(ub.z), __uint_as_float(ub.w)};
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = gv[i] / (1.0f + __expf(-gv[i])) * uv[i] * sv[i];
    }
    hadamard128(v, lane);
    *reinterpret_cast<float4 *>(rot + k0) = make_float4(v[0], v[1], v[2], v[3]);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  if (lane == 0) warp_max[warp] = m;
  __syncthreads();
  m = warp_max[0];
#pragma unroll
  for (uint32_t i = 1; i < kRotateThreads / 32u; ++i) m = fmaxf(m, warp_max[i]);
  // m in [2^(e-1), 2^e) with e = (exponent field) - 126: the scale 2^(14 - e), held to what a float carries
  int shift = 0;
  if (m > 0.0f && m <= 3.0e38f) shift = max(-126, min(126, 140 - static_cast<int>(__float_as_uint(m) >> 23)));
  const float scale = __uint_as_float(static_cast<uint32_t>(shift + 127) << 23);
  if (threadIdx.x == 0) *inv = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
  for (uint32_t i = threadIdx.x * 4u; i < in; i += 4u * kRotateThreads) {
    const float4 v = *reinterpret_cast<const float4 *>(rot + i);
    const __half2 h01 = __floats2half2_rn(v.x * scale, v.y * scale), h23 = __floats2half2_rn(v.z * scale, v.w * scale);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t *>(&h01);
    packed.y = *reinterpret_cast<const uint32_t *>(&h23);
    *reinterpret_cast<uint2 *>(dst + i) = packed;
  }
}

// PHASE 0: gate | up products of an item into gu. PHASE 1: down, weighted, into the rows the fold
// kernel adds up. One CTA per (item, 16 DW output columns); no CTA waits for another.
template <int PHASE, int DW>
__global__ void __launch_bounds__(Shape<DW>::kThreads, DW == 16 ? 1 : 2) moe_tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                 const __grid_constant__ ExpertParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t in = PHASE == 0 ? p.hidden : p.inter;
  const uint32_t out_plane = PHASE == 0 ? 2u * p.inter : p.hidden;
  constexpr uint32_t kCols = Shape<DW>::kCols, kBlocks = Shape<DW>::kBlocks;
  const uint32_t col_tiles = (out_plane + kCols - 1u) / kCols;
  const uint32_t item_index = blockIdx.x / col_tiles, col_tile = blockIdx.x % col_tiles;
  griddep_launch_dependents();
  griddep_wait();   // the item list and the rotated rows come from the kernels before
  if (item_index >= p.n_items[0]) return;
  const Item item = p.items[item_index];
  const ignis_moe_slot slot = p.slots[item.expert * 2u + PHASE];
  if (slot.record == nullptr || !(slot.k2 == 4 || slot.k2 == 5 || slot.k2 == 6 || slot.k2 == 8)) {
    if (threadIdx.x == 0 && col_tile == 0) atomicOr(p.status, kStatusAbsentRecord);
    return;
  }
  const Core c = core_setup<DW>(smem_raw);
  Job job;
  job.trellis = static_cast<const uint32_t *>(slot.record);
  job.k2 = slot.k2;
  job.tile_stride = out_plane / 16u;
  job.in = in;
  job.blk0 = kBlocks * col_tile;
  job.blk1 = kBlocks * col_tile + 1u;
  job.nblk = kBlocks == 2u && job.blk1 < out_plane / 128u ? 2u : 1u;
  job.row0 = item.first;
  job.rows = item.count;
  const uint64_t trellis_bytes = static_cast<uint64_t>(in) * out_plane * slot.k2 / 16u;
  const uint16_t *svh = reinterpret_cast<const uint16_t *>(static_cast<const uint8_t *>(slot.record) + trellis_bytes) + in;
  const float *inv_rows = reinterpret_cast<const float *>(PHASE == 0 ? p.scale_in : p.scale_h);
  const bool decoded = core_roles<DW>(c, job, &map_a, p.status + 1);   // word 1 of the status line: waits of this kernel that ran out
  if (c.warp < DW) {
    // One row tile: (block, half of its columns) per warp group, all groups at work. Two row
    // tiles: (row tile, block) per group. What the epilogue needs from global memory is asked for
    // here, before the wait for the accumulator: the loads travel while the last MMAs retire.
    const uint32_t tiles = job.rows > 128u ? 2u : 1u, items = tiles * job.nblk;
    const uint32_t group = static_cast<uint32_t>(c.warp) >> 2, quad = static_cast<uint32_t>(c.warp) & 3u;
    const uint32_t lane = static_cast<uint32_t>(c.lane);
    const bool split = tiles == 1u;
    const uint32_t tt = split ? 0u : group / job.nblk, cb = split ? group % kBlocks : group % job.nblk;
    const uint32_t half = group / kBlocks;   // split jobs: which 64 columns of the block
    const bool live = split ? cb < job.nblk : group < items;
    const uint32_t first = tt * 128u + quad * 32u;                         // the warp's first row of the item
    const uint32_t rows = !live || item.count <= first ? 0u : (item.count - first < 32u ? item.count - first : 32u);
    const bool valid = lane < rows;
    const uint32_t row = item.first + first + (valid ? lane : 0u);
    const uint32_t col0 = (cb == 0u ? job.blk0 : job.blk1) * 128u;
    const float inv = valid ? inv_rows[row] : 0.0f;
    // the lane's own row (PHASE 1): which assignment (token, rank) it is and its routing weight
    const uint32_t my_a = PHASE == 1 && valid ? p.sorted[row] : 0u;
    const float my_weight = PHASE == 1 && valid ? p.weights[my_a] : 0.0f;
    float sv[2][2];   // svh of the four columns a lane writes: [pass][lo, hi] = columns 64 pass + lane, + 32
#pragma unroll
    for (int ps = 0; ps < 2; ++ps) {
      sv[ps][0] = live ? __half2float(__ushort_as_half(__ldg(svh + col0 + 64u * ps + lane))) : 0.0f;
      sv[ps][1] = live ? __half2float(__ushort_as_half(__ldg(svh + col0 + 64u * ps + 32u + lane))) : 0.0f;
    }
    if (core_accumulator<DW>(c, decoded, p.status + 1) && (split || live)) {
      float *areas = reinterpret_cast<float *>(smem_raw + (c.base - smem_u32(smem_raw)));
      float *mine = areas + group * 8192u;
      const float *other = areas + (group ^ kBlocks) * 8192u;
      const uint32_t taddr = c.tmem + ((quad * 32u) << 16) + tt * kCols + cb * 128u;
      if (PHASE == 0) {
        float *out = p.gu + static_cast<size_t>(item.first + first) * 2u * p.inter + col0 + lane;
        auto emit = [&](uint32_t ps, uint32_t r, float lo, float hi) {
          float *dst = out + static_cast<size_t>(r) * 2u * p.inter + 64u * ps;
          dst[0] = lo * sv[ps][0];
          dst[32] = hi * sv[ps][1];
        };
        if (split) half_epilogue<DW>(taddr, half, live, inv, valid, mine, other, quad, lane, rows, emit);
        else block_epilogue(taddr, inv, valid, mine, quad, lane, rows, emit);
      } else {
        auto emit = [&](uint32_t ps, uint32_t r, float lo, float hi) {   // the row's assignment and weight, handed round by shuffle
          const uint32_t a = __shfl_sync(0xFFFFFFFFu, my_a, static_cast<int>(r));
          const float wr = __shfl_sync(0xFFFFFFFFu, my_weight, static_cast<int>(r));
          float *dst = p.down_rows + static_cast<size_t>(a) * p.hidden + col0 + 64u * ps + lane;
          dst[0] = wr * (lo * sv[ps][0]);
          dst[32] = wr * (hi * sv[ps][1]);
        };
        if (split) half_epilogue<DW>(taddr, half, live, inv, valid, mine, other, quad, lane, rows, emit);
        else block_epilogue(taddr, inv, valid, mine, quad, lane, rows, emit);
      }
    }
  }
  core_finish<DW>(c);
}

// One CTA per token: the token's weighted down products (one row per choice that had an expert with a
// record) become 2^-32 fixed-point integers and are added to the token's accumulator row. Integer
// sums do not depend on their order: the bits are those of adding every product on its own.
__global__ void __launch_bounds__(256) moe_tc_fold_kernel(const __grid_constant__ ExpertParams p, uint32_t tokens) {
  griddep_launch_dependents();
  griddep_wait();
  const uint32_t token = blockIdx.x;
  if (token >= tokens) return;
  __shared__ uint32_t present[64];
  const uint32_t top_k = p.top_k < 64u ? p.top_k : 64u;
  if (threadIdx.x < top_k) {
    const int32_t e = p.ids[static_cast<size_t>(token) * p.top_k + threadIdx.x];
    bool ok = e >= 0 && static_cast<uint32_t>(e) < p.experts;
    if (ok) {
      const ignis_moe_slot slot = p.slots[static_cast<uint32_t>(e) * 2u + 1u];
      ok = slot.record != nullptr && (slot.k2 == 4 || slot.k2 == 5 || slot.k2 == 6 || slot.k2 == 8);
    }
    present[threadIdx.x] = ok ? 1u : 0u;
  }
  __syncthreads();
  bool range = false;
  // four columns per thread and trip (hidden is a multiple of 128), the choices' loads issued together
  const float4 *rows4 = reinterpret_cast<const float4 *>(p.down_rows + static_cast<size_t>(token) * p.top_k * p.hidden);
  const uint32_t quads = p.hidden / 4u;
  for (uint32_t c4 = threadIdx.x; c4 < quads; c4 += 256u) {
    long long sum[4] = {0, 0, 0, 0};
    for (uint32_t k0 = 0; k0 < top_k; k0 += 8u) {
      float4 v[8];
#pragma unroll
      for (uint32_t j = 0; j < 8u; ++j) {
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k0 + j < top_k && present[k0 + j] != 0u) v[j] = __ldcs(rows4 + static_cast<size_t>(k0 + j) * quads + c4);
      }
#pragma unroll
      for (uint32_t j = 0; j < 8u; ++j) {
        const float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (!(fabsf(e[i]) < 2147483648.0f)) {   // also catches NaN
            range = true;
          } else {
            // times 2^32 is exact in a float (the magnitude is below 2^31): the integer a double product would round to
            sum[i] += __float2ll_rn(e[i] * 4294967296.0f);
          }
        }
      }
    }
    long long *dst = p.acc + static_cast<size_t>(token) * p.hidden + 4u * c4;   // the caller's buffer: 8-byte alignment is all it promises
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] += sum[i];
  }
  if (range) atomicOr(p.status, kStatusRange);
}

constexpr size_t kRotateSmemMax = 200 * 1024;


// Which shape the expert products take: 8 decoder warps and two CTAs per SM unless B200Q_MOE_TC_WIDE
// is set to 1 (read when the kernels are prepared).
int g_moe_dw = 8;

template <int DW>
cudaError_t set_gemm_attrs() {
  cudaError_t err = cudaFuncSetAttribute(moe_tc_gemm_kernel<0, DW>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Shape<DW>::kSmemBytes));
  if (err == cudaSuccess) err = cudaFuncSetAttribute(moe_tc_gemm_kernel<1, DW>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Shape<DW>::kSmemBytes));
  return err;
}

template <int DW>
cudaError_t launch_gemm(int phase, uint32_t items_max, uint32_t out_plane, cudaStream_t stream, bool pdl, const CUtensorMap &map_a, const ExpertParams &p) {
  const uint32_t col_tiles = (out_plane + Shape<DW>::kCols - 1u) / Shape<DW>::kCols;
  const dim3 grid(items_max * col_tiles);
  return phase == 0 ? launch(moe_tc_gemm_kernel<0, DW>, grid, dim3(Shape<DW>::kThreads), Shape<DW>::kSmemBytes, stream, pdl, map_a, p)
                    : launch(moe_tc_gemm_kernel<1, DW>, grid, dim3(Shape<DW>::kThreads), Shape<DW>::kSmemBytes, stream, pdl, map_a, p);
}

}  // namespace

int32_t moe_tc_prepare(ErrorSlot &slot) {
  const char *wide = getenv("B200Q_MOE_TC_WIDE");
  g_moe_dw = wide != nullptr && wide[0] == '1' ? 16 : 8;
  cudaError_t err = set_gemm_attrs<16>();
  if (err == cudaSuccess) err = set_gemm_attrs<8>();
  if (err == cudaSuccess) err = cudaFuncSetAttribute(moe_tc_rotate_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kRotateSmemMax));
  if (err == cudaSuccess) err = cudaFuncSetAttribute(moe_tc_rotate_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kRotateSmemMax));
  if (err != cudaSuccess) return fail(slot, "MoE tensor-core kernel attributes: %s", cudaGetErrorString(err));
  if (encode_tiled_fn() == nullptr) return fail(slot, "cuTensorMapEncodeTiled is not available from this driver");
  return 0;
}

int32_t moe_tc_experts(ErrorSlot &slot, const DeviceState &dev, const ExpertParams &p, uint32_t rows, uint32_t items_max,
                       const uint32_t *offsets, cudaStream_t stream, const char *what) {
  const bool pdl = dev.pdl != 0;
  const uint32_t tokens = rows / p.top_k;
  if (p.top_k > 64u) return fail(slot, "%s: more than 64 choices per token on the tensor-core route", what);
  for (int phase = 0; phase < 2; ++phase) {
    const uint32_t in = phase == 0 ? p.hidden : p.inter;
    const uint32_t out_plane = phase == 0 ? 2u * p.inter : p.hidden;
    if (static_cast<size_t>(in) * 4u > kRotateSmemMax) return fail(slot, "%s: a dimension is too long for the tensor-core route", what);
    cudaError_t err = phase == 0 ? launch(moe_tc_rotate_kernel<0>, dim3(rows), dim3(kRotateThreads), static_cast<size_t>(in) * 4u, stream, pdl, p, offsets)
                                 : launch(moe_tc_rotate_kernel<1>, dim3(rows), dim3(kRotateThreads), static_cast<size_t>(in) * 4u, stream, pdl, p, offsets);
    if (err != cudaSuccess) return fail(slot, "%s: rotation launch failed: %s", what, cudaGetErrorString(err));
    CUtensorMap map_a;
    if (!make_rows_map(&map_a, phase == 0 ? static_cast<const void *>(p.frag_in) : static_cast<const void *>(p.frag_h), rows, in)) {
      return fail(slot, "%s: tensor map encoding failed", what);
    }
    err = g_moe_dw == 16 ? launch_gemm<16>(phase, items_max, out_plane, stream, pdl, map_a, p) : launch_gemm<8>(phase, items_max, out_plane, stream, pdl, map_a, p);
    if (err != cudaSuccess) return fail(slot, "%s: expert launch failed: %s", what, cudaGetErrorString(err));
  }
  const cudaError_t err = launch(moe_tc_fold_kernel, dim3(tokens), dim3(256), 0, stream, pdl, p, tokens);
  if (err != cudaSuccess) return fail(slot, "%s: fold launch failed: %s", what, cudaGetErrorString(err));
  return 0;
}

}  // namespace b200q
