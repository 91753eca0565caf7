// The routed experts of wide calls on the tensor cores.
//
// Stands where the reference's prefill entry multiplies items of up to 64 rows with warp-level MMAs
// (kernel/src/moe_prefill.cu:252-262, kernels :405 and :421). Under skewed routing a few experts see
// hundreds of rows; here a work item is up to 256 sorted rows of one expert, and every item is
// multiplied with its expert's record by the kernel core of trellis_tc.cuh: the rows rotated once
// into plain fp16 rows with one scale per row, the record's trellis tiles decoded into swizzled
// shared memory, tcgen05.mma kind::f16 with the accumulator in tensor memory, and the output
// Hadamard in registers. Four launches behind the grouping:
//
//   moe_tc_rotate_kernel<0>   x o suh (the row's expert's gate|up record), Hadamard, fp16 rows
//   moe_tc_gemm_kernel<0>     rows x gate|up record -> gu fp32 [row][2 inter] (gate columns, then up)
//   moe_tc_rotate_kernel<1>   silu(g) u o suh (the down record), Hadamard, fp16 rows
//   moe_tc_gemm_kernel<1>     rows x down record, times the routing weight, added to the int64
//                             fixed-point accumulator of the row's token (atomic, order-free)
//
// A row's arithmetic does not depend on the item it is in or on the rows beside it, so results are
// reproducible bit for bit whatever the grouping order.
#include "moe_internal.cuh"
#include "trellis_tc.cuh"

namespace b200q {
namespace {

using namespace trellis_tc;

// One CTA per sorted row: the row's `in` values times the expert's suh, the 128-wide Hadamard per
// block (a warp per block), one power-of-two scale per row (largest magnitude in [2^13, 2^14)),
// fp16. PHASE 0 reads the token's activations, PHASE 1 silu(g) u of the row's gate|up products.
template <int PHASE>
__global__ void __launch_bounds__(256) moe_tc_rotate_kernel(const __grid_constant__ ExpertParams p, const uint32_t *offsets) {
  extern __shared__ __align__(16) float rot[];
  __shared__ float warp_max[8];
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
    for (uint32_t i = threadIdx.x * 4u; i < in; i += 1024u) *reinterpret_cast<uint2 *>(dst + i) = make_uint2(0u, 0u);
    if (threadIdx.x == 0) *inv = 0.0f;
    return;
  }
  const uint32_t out_plane = PHASE == 0 ? 2u * p.inter : p.hidden;
  const uint64_t trellis_bytes = static_cast<uint64_t>(in) * out_plane * slot.k2 / 16u;
  const uint16_t *suh = reinterpret_cast<const uint16_t *>(static_cast<const uint8_t *>(slot.record) + trellis_bytes);
  const uint32_t token = a / p.top_k;
  const uint32_t nblk = in / 128u;
  float m = 0.0f;
  for (uint32_t bl = static_cast<uint32_t>(warp); bl < nblk; bl += 8u) {
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
  for (int i = 1; i < 8; ++i) m = fmaxf(m, warp_max[i]);
  int shift = 0;
  if (m > 0.0f && m <= 3.0e38f) {
    int e;
    (void)frexpf(m, &e);
    shift = max(-126, min(126, 14 - e));
  }
  const float scale = ldexpf(1.0f, shift);
  if (threadIdx.x == 0) *inv = ldexpf(1.0f, -shift);
  for (uint32_t i = threadIdx.x * 4u; i < in; i += 1024u) {
    const float4 v = *reinterpret_cast<const float4 *>(rot + i);
    const __half2 h01 = __floats2half2_rn(v.x * scale, v.y * scale), h23 = __floats2half2_rn(v.z * scale, v.w * scale);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t *>(&h01);
    packed.y = *reinterpret_cast<const uint32_t *>(&h23);
    *reinterpret_cast<uint2 *>(dst + i) = packed;
  }
}

// PHASE 0: gate | up products of an item into gu. PHASE 1: down, weighted, into acc.
// One CTA per (item, 256 output columns); no CTA waits for another.
template <int PHASE>
__global__ void __launch_bounds__(kThreads, 1) moe_tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                 const __grid_constant__ ExpertParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t in = PHASE == 0 ? p.hidden : p.inter;
  const uint32_t out_plane = PHASE == 0 ? 2u * p.inter : p.hidden;
  const uint32_t col_tiles = (out_plane + 255u) / 256u;
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
  const Core c = core_setup(smem_raw);
  Job job;
  job.trellis = static_cast<const uint32_t *>(slot.record);
  job.k2 = slot.k2;
  job.tile_stride = out_plane / 16u;
  job.in = in;
  job.blk0 = 2u * col_tile;
  job.blk1 = 2u * col_tile + 1u;
  job.nblk = job.blk1 < out_plane / 128u ? 2u : 1u;
  job.row0 = item.first;
  job.rows = item.count;
  const uint64_t trellis_bytes = static_cast<uint64_t>(in) * out_plane * slot.k2 / 16u;
  const uint16_t *svh = reinterpret_cast<const uint16_t *>(static_cast<const uint8_t *>(slot.record) + trellis_bytes) + in;
  const float *inv_rows = reinterpret_cast<const float *>(PHASE == 0 ? p.scale_in : p.scale_h);
  const bool have = core_run(c, job, &map_a, p.status + 1);   // word 1 of the status line: waits of this kernel that ran out
  if (have) {
    const uint32_t tiles = job.rows > 128u ? 2u : 1u, items = tiles * job.nblk;
    const uint32_t group = static_cast<uint32_t>(c.warp) >> 2, quad = static_cast<uint32_t>(c.warp) & 3u;
    float *stash = reinterpret_cast<float *>(smem_raw + (c.base - smem_u32(smem_raw))) + group * 8192u + quad * 32u + static_cast<uint32_t>(c.lane);
    for (uint32_t it = group; it < items; it += kDecoderWarps / 4) {
      const uint32_t tt = it / job.nblk, cb = it % job.nblk;
      const uint32_t local = tt * 128u + quad * 32u + static_cast<uint32_t>(c.lane);
      const bool valid = local < item.count;
      const uint32_t row = item.first + (valid ? local : 0u);
      const uint32_t col0 = (cb == 0u ? job.blk0 : job.blk1) * 128u;
      const uint2 *sv = reinterpret_cast<const uint2 *>(svh + col0);
      const uint32_t taddr = c.tmem + ((quad * 32u) << 16) + tt * 256u + cb * 128u;
      if (PHASE == 0) {
        float4 *dst = reinterpret_cast<float4 *>(p.gu + static_cast<size_t>(row) * 2u * p.inter + col0);
        block_epilogue(taddr, valid ? inv_rows[row] : 0.0f, valid, stash, [&](int q, const float (&r)[4]) {
          const uint2 s = sv[q];
          const __half2 s01 = *reinterpret_cast<const __half2 *>(&s.x), s23 = *reinterpret_cast<const __half2 *>(&s.y);
          dst[q] = make_float4(r[0] * __low2float(s01), r[1] * __high2float(s01), r[2] * __low2float(s23), r[3] * __high2float(s23));
        });
      } else {
        const uint32_t a = p.sorted[row];
        const uint32_t token = a / p.top_k;
        const float wr = p.weights[a];
        long long *dst = p.acc + static_cast<size_t>(token) * p.hidden + col0;
        bool range = false;
        block_epilogue(taddr, valid ? inv_rows[row] : 0.0f, valid, stash, [&](int q, const float (&r)[4]) {
          const uint2 s = sv[q];
          const __half2 s01 = *reinterpret_cast<const __half2 *>(&s.x), s23 = *reinterpret_cast<const __half2 *>(&s.y);
          const float y[4] = {r[0] * __low2float(s01), r[1] * __high2float(s01), r[2] * __low2float(s23), r[3] * __high2float(s23)};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float cval = wr * y[e];
            if (!(fabsf(cval) < 2147483648.0f)) {   // also catches NaN
              range = true;
            } else {
              atomicAdd(reinterpret_cast<unsigned long long *>(dst + 4 * q + e),
                        static_cast<unsigned long long>(__double2ll_rn(static_cast<double>(cval) * 4294967296.0)));
            }
          }
        });
        if (range) atomicOr(p.status, kStatusRange);
      }
      __syncwarp();   // the accumulator loads of the next item are warp-wide
    }
  }
  core_finish(c);
}

constexpr size_t kRotateSmemMax = 200 * 1024;

}  // namespace

int32_t moe_tc_prepare(ErrorSlot &slot) {
  cudaError_t err = cudaFuncSetAttribute(moe_tc_gemm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes));
  if (err == cudaSuccess) err = cudaFuncSetAttribute(moe_tc_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes));
  if (err == cudaSuccess) err = cudaFuncSetAttribute(moe_tc_rotate_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kRotateSmemMax));
  if (err == cudaSuccess) err = cudaFuncSetAttribute(moe_tc_rotate_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kRotateSmemMax));
  if (err != cudaSuccess) return fail(slot, "MoE tensor-core kernel attributes: %s", cudaGetErrorString(err));
  if (encode_tiled_fn() == nullptr) return fail(slot, "cuTensorMapEncodeTiled is not available from this driver");
  return 0;
}

int32_t moe_tc_experts(ErrorSlot &slot, const DeviceState &dev, const ExpertParams &p, uint32_t rows, uint32_t items_max,
                       const uint32_t *offsets, cudaStream_t stream, const char *what) {
  const bool pdl = dev.pdl != 0;
  for (int phase = 0; phase < 2; ++phase) {
    const uint32_t in = phase == 0 ? p.hidden : p.inter;
    const uint32_t out_plane = phase == 0 ? 2u * p.inter : p.hidden;
    if (static_cast<size_t>(in) * 4u > kRotateSmemMax) return fail(slot, "%s: a dimension is too long for the tensor-core route", what);
    cudaError_t err = phase == 0 ? launch(moe_tc_rotate_kernel<0>, dim3(rows), dim3(256), static_cast<size_t>(in) * 4u, stream, pdl, p, offsets)
                                 : launch(moe_tc_rotate_kernel<1>, dim3(rows), dim3(256), static_cast<size_t>(in) * 4u, stream, pdl, p, offsets);
    if (err != cudaSuccess) return fail(slot, "%s: rotation launch failed: %s", what, cudaGetErrorString(err));
    CUtensorMap map_a;
    if (!make_rows_map(&map_a, phase == 0 ? static_cast<const void *>(p.frag_in) : static_cast<const void *>(p.frag_h), rows, in)) {
      return fail(slot, "%s: tensor map encoding failed", what);
    }
    const uint32_t col_tiles = (out_plane + 255u) / 256u;
    const dim3 grid(items_max * col_tiles);
    err = phase == 0 ? launch(moe_tc_gemm_kernel<0>, grid, dim3(kThreads), kSmemBytes, stream, pdl, map_a, p)
                     : launch(moe_tc_gemm_kernel<1>, grid, dim3(kThreads), kSmemBytes, stream, pdl, map_a, p);
    if (err != cudaSuccess) return fail(slot, "%s: expert launch failed: %s", what, cudaGetErrorString(err));
  }
  return 0;
}

}  // namespace b200q
