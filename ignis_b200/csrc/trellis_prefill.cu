// Dense trellis linear beyond 64 tokens: the prefill route on the tensor cores.
//
// Stands where the reference switches from its decode kernel to its prefill kernel
// (kernel/src/trellis_linear.cu: rotate_kernel + prefill_kernel, trellis_linear_prefill.cu:162-279;
// the route needs the workspace, as theirs does). Two launches: `trellis_rotate_rows_kernel` writes
// the rotated activations as fp16 rows with one scale per token into the workspace, and
// `trellis_tc_dense_kernel` multiplies them with the trellis plane on tcgen05 (trellis_tc.cuh).
// SwiGLU runs the gate product first (BF16 into h, as the reference's prefill route stores the gate
// between its passes: ignis_trellis_linear.h:43-44) and the up product with an epilogue that
// multiplies by silu of what it finds there.
#include "../../include/ignis_trellis_linear.h"

#include "trellis_internal.cuh"
#include "trellis_tc.cuh"

namespace b200q {
namespace {

using namespace trellis_tc;

__device__ uint32_t g_trellis_tc_status = 0;

// ---- rotation: one CTA per token ------------------------------------------------------------------
// x o suh, the 128-wide Hadamard per block (a warp per block, fp32), one power-of-two scale for the
// whole token (largest magnitude in [2^13, 2^14)), fp16. The token's rotated values wait in shared
// memory between the two passes (4 bytes per input).
__global__ void __launch_bounds__(256) trellis_rotate_rows_kernel(const uint16_t *x, const uint16_t *suh, uint32_t in,
                                                                  uint16_t *rows_f16, float *inv) {
  extern __shared__ __align__(16) float rot[];
  __shared__ float warp_max[8];
  griddep_launch_dependents();
  griddep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t token = blockIdx.x;
  const uint32_t nblk = in / 128u;
  float m = 0.0f;
  for (uint32_t bl = static_cast<uint32_t>(warp); bl < nblk; bl += 8u) {
    const size_t k0 = static_cast<size_t>(bl) * 128u + 4u * lane;
    const uint2 xb = ldg64_coherent(x + static_cast<size_t>(token) * in + k0);
    const uint2 sb = *reinterpret_cast<const uint2 *>(suh + k0);
    const __half2 s01 = *reinterpret_cast<const __half2 *>(&sb.x), s23 = *reinterpret_cast<const __half2 *>(&sb.y);
    float v[4];
    v[0] = bf16_bits_to_f32(xb.x & 0xFFFFu) * __low2float(s01);
    v[1] = __uint_as_float(xb.x & 0xFFFF0000u) * __high2float(s01);
    v[2] = bf16_bits_to_f32(xb.y & 0xFFFFu) * __low2float(s23);
    v[3] = __uint_as_float(xb.y & 0xFFFF0000u) * __high2float(s23);
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
  // m in [2^(e-1), 2^e) with e = (exponent field) - 126: the scale 2^(14 - e), held to what a float carries
  int shift = 0;
  if (m > 0.0f && m <= 3.0e38f) shift = max(-126, min(126, 140 - static_cast<int>(__float_as_uint(m) >> 23)));
  const float scale = __uint_as_float(static_cast<uint32_t>(shift + 127) << 23);
  if (threadIdx.x == 0) inv[token] = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
  uint16_t *dst = rows_f16 + static_cast<size_t>(token) * in;
  for (uint32_t i = threadIdx.x * 4u; i < in; i += 1024u) {
    const float4 v = *reinterpret_cast<const float4 *>(rot + i);
    const __half2 h01 = __floats2half2_rn(v.x * scale, v.y * scale), h23 = __floats2half2_rn(v.z * scale, v.w * scale);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t *>(&h01);
    packed.y = *reinterpret_cast<const uint32_t *>(&h23);
    *reinterpret_cast<uint2 *>(dst + i) = packed;
  }
}

// ---- the product -----------------------------------------------------------------------------------
constexpr uint32_t kEpiStore = 0, kEpiAdd = 1, kEpiSiluMul = 2;   // kEpiSiluMul: y = BF16(silu(float(y)) * v)

struct DenseParams {
  const uint32_t *trellis;
  const uint16_t *svh;
  const float *inv;      // the tokens' inverse scales
  uint16_t *y;           // BF16 [tokens][ldy]
  uint32_t k2, tile_stride, in, out, tokens, ldy, epilogue;
};

// DW: the core's shape - 16 (256 columns a CTA, one CTA per SM) or 8 (128 columns, two per SM).
template <int DW>
__global__ void __launch_bounds__(Shape<DW>::kThreads, DW == 16 ? 1 : 2) trellis_tc_dense_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                                              const __grid_constant__ DenseParams p) {
  constexpr int kDenseDw = DW;
  constexpr uint32_t kCols = Shape<DW>::kCols, kBlocks = Shape<DW>::kBlocks;
  extern __shared__ uint8_t smem_raw[];
  const Core c = core_setup<kDenseDw>(smem_raw);
  // Token tiles run fastest over the grid, so the CTAs at work at one time decode the same columns
  // of the plane (read from HBM once, then from the L2).
  const uint32_t row_tiles = (p.tokens + 255u) / 256u;
  const uint32_t col_tile = blockIdx.x / row_tiles, row_tile = blockIdx.x % row_tiles;
  Job job;
  job.trellis = p.trellis;
  job.k2 = p.k2;
  job.tile_stride = p.tile_stride;
  job.in = p.in;
  job.blk0 = kBlocks * col_tile;
  job.blk1 = kBlocks * col_tile + 1u;
  job.nblk = kBlocks == 2u && job.blk1 < p.out / 128u ? 2u : 1u;
  job.row0 = row_tile * 256u;
  job.rows = p.tokens - job.row0 < 256u ? p.tokens - job.row0 : 256u;
  const bool decoded = core_roles<kDenseDw>(c, job, &map_a, &g_trellis_tc_status);
  if (c.warp < kDenseDw) {
    // Two row tiles: the (row tile, block) items go to the groups of four warps. One: a group takes
    // half a block's columns, so that all groups are at work. A warp's lanes are the rows
    // 32 (warp % 4) .. + 31 of the row tile. What the epilogue needs from global memory is asked
    // for before the wait for the accumulator, while the last MMAs retire.
    const uint32_t tiles = job.rows > 128u ? 2u : 1u, items = tiles * job.nblk;
    const uint32_t group = static_cast<uint32_t>(c.warp) >> 2, quad = static_cast<uint32_t>(c.warp) & 3u;
    const uint32_t lane = static_cast<uint32_t>(c.lane);
    const bool split = tiles == 1u;
    const uint32_t tt = split ? 0u : group / job.nblk, cb = split ? group % kBlocks : group % job.nblk;
    const uint32_t half = group / kBlocks;   // split jobs: which 64 columns of the block
    const bool live = split ? cb < job.nblk : group < items;
    const uint32_t first = tt * 128u + quad * 32u;   // the warp's first row of the job
    const uint32_t rows = !live || job.rows <= first ? 0u : (job.rows - first < 32u ? job.rows - first : 32u);
    const bool valid = lane < rows;
    const uint32_t token0 = job.row0 + first;
    const uint32_t col0 = (cb == 0u ? job.blk0 : job.blk1) * 128u;
    const float inv = valid ? p.inv[token0 + lane] : 0.0f;
    float sv[2][2];   // svh of the four columns a lane writes: [pass][lo, hi] = columns 64 pass + lane, + 32
#pragma unroll
    for (int ps = 0; ps < 2; ++ps) {
      sv[ps][0] = live ? __half2float(__ushort_as_half(__ldg(p.svh + col0 + 64u * ps + lane))) : 0.0f;
      sv[ps][1] = live ? __half2float(__ushort_as_half(__ldg(p.svh + col0 + 64u * ps + 32u + lane))) : 0.0f;
    }
    if (core_accumulator<kDenseDw>(c, decoded, &g_trellis_tc_status) && (split || live)) {
      float *areas = reinterpret_cast<float *>(smem_raw + (c.base - smem_u32(smem_raw)));
      uint16_t *out = p.y + static_cast<size_t>(token0) * p.ldy + col0 + lane;
      auto emit = [&](uint32_t ps, uint32_t r, float lo, float hi) {
        uint16_t *dst = out + static_cast<size_t>(r) * p.ldy + 64u * ps;
        float v[2] = {lo * sv[ps][0], hi * sv[ps][1]};
        if (p.epilogue != kEpiStore) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float o = bf16_bits_to_f32(dst[32 * e]);
            v[e] = p.epilogue == kEpiAdd ? v[e] + o : o / (1.0f + __expf(-o)) * v[e];
          }
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) dst[32 * e] = __bfloat16_as_ushort(__float2bfloat16_rn(v[e]));
      };
      const uint32_t taddr = c.tmem + ((quad * 32u) << 16) + tt * kCols + cb * 128u;
      float *mine = areas + group * 8192u;
      if (split) half_epilogue<kDenseDw>(taddr, half, live, inv, valid, mine, areas + (group ^ kBlocks) * 8192u, quad, lane, rows, emit);
      else block_epilogue(taddr, inv, valid, mine, quad, lane, rows, emit);
    }
  }
  core_finish<kDenseDw>(c);
}

uint64_t align256(uint64_t v) { return (v + 255u) & ~static_cast<uint64_t>(255u); }

constexpr size_t kRotateMaxSmem = 200 * 1024;   // 4 bytes per input: in <= 51200

bool aligned_to(const void *p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace

uint64_t trellis_tc_workspace_bytes(uint32_t in, uint32_t weights, uint32_t tokens) {
  // a status line, then per weight the rotated rows (fp16) and the tokens' inverse scales
  return 256u + static_cast<uint64_t>(weights) * (align256(static_cast<uint64_t>(tokens) * in * 2u) + align256(static_cast<uint64_t>(tokens) * 4u));
}

// Which shape a dense product takes: the narrow one (8 decoder warps, two CTAs per SM), which
// measured faster at 256, 1024 and 4096 tokens (a decoded tile serves 256 tokens in both, and the
// narrow CTAs overlap each other's fill, drain and epilogue); B200Q_TRELLIS_TC_SHAPE = 16 selects
// the wide one (read when the kernels are prepared).
int g_dense_dw = 8;

int32_t trellis_tc_prepare(ErrorSlot &slot) {
  const char *shape = getenv("B200Q_TRELLIS_TC_SHAPE");
  g_dense_dw = shape != nullptr && atoi(shape) == 16 ? 16 : 8;
  cudaError_t err = cudaFuncSetAttribute(trellis_tc_dense_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Shape<16>::kSmemBytes));
  if (err == cudaSuccess) err = cudaFuncSetAttribute(trellis_tc_dense_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Shape<8>::kSmemBytes));
  if (err == cudaSuccess) {
    err = cudaFuncSetAttribute(trellis_rotate_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kRotateMaxSmem));
  }
  if (err != cudaSuccess) return fail(slot, "trellis prefill kernel attributes: %s", cudaGetErrorString(err));
  if (encode_tiled_fn() == nullptr) return fail(slot, "cuTensorMapEncodeTiled is not available from this driver");
  return 0;
}

bool trellis_tc_takes(const DeviceState &dev, uint32_t in, uint32_t tokens, uint32_t weights, const ignis_trellis_workspace *workspace) {
  if (dev.trellis_tc == 0 || tokens <= IGNIS_TRELLIS_DECODE_MAX_TOKENS) return false;
  if (static_cast<size_t>(in) * 4u > kRotateMaxSmem) return false;
  if (workspace == nullptr || workspace->base == nullptr || !aligned_to(workspace->base, 256)) return false;
  return workspace->bytes >= trellis_tc_workspace_bytes(in, weights, tokens);
}

namespace {
int32_t one_product(ErrorSlot &slot, const DeviceState &dev, const ignis_trellis_weight *w, const uint16_t *x, uint32_t tokens, uint16_t *y,
                    uint32_t ldy, uint32_t epilogue, uint8_t *region, cudaStream_t stream, const char *what) {
  uint16_t *rows = reinterpret_cast<uint16_t *>(region);
  float *inv = reinterpret_cast<float *>(region + align256(static_cast<uint64_t>(tokens) * w->in * 2u));
  cudaError_t err = launch(trellis_rotate_rows_kernel, dim3(tokens), dim3(256), static_cast<size_t>(w->in) * 4u, stream, dev.pdl != 0, x,
                           static_cast<const uint16_t *>(w->suh), w->in, rows, inv);
  if (err != cudaSuccess) return fail(slot, "%s: rotation launch failed: %s", what, cudaGetErrorString(err));
  CUtensorMap map_a;
  if (!make_rows_map(&map_a, rows, tokens, w->in)) return fail(slot, "%s: tensor map encoding failed", what);
  DenseParams p = {};
  p.trellis = static_cast<const uint32_t *>(w->trellis);
  p.svh = static_cast<const uint16_t *>(w->svh);
  p.inv = inv;
  p.y = y;
  p.k2 = w->k2;
  p.tile_stride = w->tile_stride ? w->tile_stride : w->out / 16u;
  p.in = w->in;
  p.out = w->out;
  p.tokens = tokens;
  p.ldy = ldy;
  p.epilogue = epilogue;
  const uint32_t row_tiles = (tokens + 255u) / 256u;
  const uint32_t wide_ctas = (w->out + 255u) / 256u * row_tiles;
  err = g_dense_dw == 16 ? launch(trellis_tc_dense_kernel<16>, dim3(wide_ctas), dim3(Shape<16>::kThreads), Shape<16>::kSmemBytes, stream, dev.pdl != 0, map_a, p)
                 : launch(trellis_tc_dense_kernel<8>, dim3((w->out + 127u) / 128u * row_tiles), dim3(Shape<8>::kThreads), Shape<8>::kSmemBytes, stream,
                          dev.pdl != 0, map_a, p);
  if (err != cudaSuccess) return fail(slot, "%s: launch failed: %s", what, cudaGetErrorString(err));
  return 0;
}
}  // namespace

int32_t trellis_tc_linear(ErrorSlot &slot, const DeviceState &dev, const ignis_trellis_weight *w, const ignis_trellis_weight *up,
                          const void *x, uint32_t tokens, void *y, uint32_t ldy, uint32_t epilogue,
                          const ignis_trellis_workspace *workspace, cudaStream_t stream, const char *what) {
  uint8_t *base = static_cast<uint8_t *>(workspace->base) + 256;
  const uint16_t *xs = static_cast<const uint16_t *>(x);
  uint16_t *ys = static_cast<uint16_t *>(y);
  if (up == nullptr) return one_product(slot, dev, w, xs, tokens, ys, ldy, epilogue == 1u ? kEpiAdd : kEpiStore, base, stream, what);
  // SwiGLU: the gate product into h, then the up product times silu of what it finds there
  if (one_product(slot, dev, w, xs, tokens, ys, ldy, kEpiStore, base, stream, what) != 0) return -1;
  uint8_t *second = base + align256(static_cast<uint64_t>(tokens) * w->in * 2u) + align256(static_cast<uint64_t>(tokens) * 4u);
  return one_product(slot, dev, up, xs, tokens, ys, ldy, kEpiSiluMul, second, stream, what);
}

int32_t trellis_tc_status(ErrorSlot &slot, cudaStream_t stream, uint32_t *status) {
  cudaError_t err = cudaMemcpyFromSymbolAsync(status, g_trellis_tc_status, sizeof(uint32_t), 0, cudaMemcpyDeviceToHost, stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
  if (err != cudaSuccess) return fail(slot, "b200q_trellis_device_status: %s", cudaGetErrorString(err));
  return 0;
}

}  // namespace b200q
