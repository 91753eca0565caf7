// The trellis products on the 5th-generation tensor cores: the part shared by the dense prefill
// route (trellis_prefill.cu) and the MoE expert GEMMs (moe_tc.cu).
//
// Stands where the reference runs its prefill kernels on warp-level MMAs - trellis tiles decoded
// from shared memory into mma.sync fragments, fp16 accumulation folded every 32 inputs
// (kernel/src/trellis_linear_prefill.cu:162-279, kernel/src/moe_prefill.cu:252-421). The design
// here is not theirs:
//
//  * The activations are rotated once by a kernel of their own (x o suh, the 128-wide Hadamard in
//    fp32) and stored as plain fp16 rows [row][in] with ONE power-of-two scale per row (largest
//    magnitude in [2^13, 2^14)), so the whole sum over `in` accumulates in tensor memory and the
//    inverse scale is applied once, in the epilogue. fp16 keeps 11 significant bits of every value
//    down to 2^-28 of the row's largest; what lies below contributes less than that to any sum.
//  * A CTA owns up to 256 rows (two MMA tiles of M = 128: the rows are the accumulator's lanes) and
//    256 output columns (two 128-column Hadamard blocks: the MMA's N), and walks `in` in stages of
//    64. Sixteen decoder warps (four per scheduler: the decode is a chain of dependent integer
//    operations, and two warps per scheduler left it idle most cycles) turn the stage's 64
//    trellis tiles into fp16 in registers (the decode of
//    trellis_device.cuh: funnel shifts, IMAD, DP4A, half an HFMA2 per weight) and store them into
//    the stage's B tile in the K-major 128-byte-swizzle layout the tensor core reads: a lane's
//    eight values are four 4-byte stores that hit 32 different banks across the warp. A producer
//    thread brings the rows' fp16 activations by TMA (the same swizzle); one thread issues
//    tcgen05.mma kind::f16 (M 128, N 256, K 16; fp16 x fp16, fp32 accumulation in tensor memory).
//    Every decoded tile serves both row tiles: 512 accumulator columns, all of tensor memory.
//  * The epilogue: a thread owns one row of one 128-column block (of half a block when the job has
//    one row tile, so that all sixteen warps take part). It reads 64 accumulator columns, applies
//    the row's inverse scale and six Hadamard stages in registers and parks the 64 values in the
//    (by then idle) stage ring, where the seventh stage combines the two halves; the results are
//    parked once more and written out row-wise - a warp per row, a lane per column - with svh and
//    the caller's epilogue, so that a warp's stores (or atomics) are contiguous.
//  * Every mbarrier wait is bounded; a wait that runs out sets a bit of a status word and the CTA
//    falls through to the common exit and frees its tensor memory.
#ifndef B200Q_TRELLIS_TC_CUH
#define B200Q_TRELLIS_TC_CUH

#include "nvfp4_tc.cuh"
#include "trellis_device.cuh"

namespace b200q {
namespace trellis_tc {

using namespace trellis_dev;

constexpr uint32_t kABytes = 128 * 128;     // one row tile of a stage: 128 rows x 64 fp16

// Two shapes of the CTA. DW = 16 decoder warps: 256 output columns (two Hadamard blocks), three
// stages, all 512 tensor-memory columns, one CTA per SM - every decoded tile serves up to 256 rows
// once. DW = 8: 128 output columns (one block), two stages, 256 tensor-memory columns, so that TWO
// CTAs share an SM (the same sixteen decoder warps in all) and one's setup, pipeline fill, drain and
// epilogue run under the other's decoding: for jobs too short to amortise those (the MoE items).
template <int DW>
struct Shape {
  static constexpr int kDecoderWarps = DW;
  static constexpr int kThreads = (DW + 2) * 32;   // the decoder / epilogue warps, the producer warp, the MMA warp
  static constexpr uint32_t kBlocks = DW / 8;       // 128-column blocks per CTA
  static constexpr uint32_t kCols = DW * 16;        // output columns per CTA = accumulator columns per row tile
  static constexpr uint32_t kStages = DW == 16 ? 3 : 2;
  static constexpr uint32_t kBBytes = kCols * 128;  // one stage of decoded weights: kCols columns x 64 fp16
  static constexpr uint32_t kStageBytes = 2 * kABytes + kBBytes;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + 256 + 1024;   // + barriers and the tensor-memory slot + alignment slack
  static constexpr uint32_t kTmemCols = 2 * kCols;
};
constexpr uint32_t kStatusProducer = 1u, kStatusMma = 2u, kStatusEpilogue = 4u, kStatusDecoder = 8u;

// What one CTA multiplies: rows [row0, row0 + rows) of the rotated activations (rows <= 256) with
// two 128-column blocks of one trellis plane.
struct Job {
  const uint32_t *trellis;  // the plane: tile (tk, tn) at word (tk * tile_stride + tn) * 4 k2
  uint32_t k2;
  uint32_t tile_stride;     // tiles per stored row of the plane
  uint32_t in;              // a multiple of 128
  uint32_t blk0, blk1;      // the 128-column blocks behind accumulator columns 0..127 and 128..255
  uint32_t nblk;            // 1: blk1 does not exist (the MMA's N is 128)
  uint32_t row0, rows;      // row0 is also the TMA row coordinate
};

// The raw words of the 4 tiles a decoder warp owns in one stage (1 tile column x 4 tile rows), one
// word per lane and tile (two for the widths whose tiles have more than 32 words): lane l holds
// word l of the tile, and the three words a lane's window needs come from its neighbours by shuffle.
// A 16 x 16 tile is 4 k2 words, so one coalesced load of up to 128 bytes fetches a whole tile.
template <int K2>
struct StageWords {
  static constexpr int kPerTile = (4 * K2 + 31) / 32;
  uint32_t w[4][kPerTile];
};

constexpr int kWordRing = 4;   // stages of raw words a decoder warp keeps in flight in registers

// Six stages of the in-register Sylvester Hadamard (natural order) on 64 values: one half of a
// 128-wide transform, whose seventh stage pairs value i of one half with value i of the other.
__device__ __forceinline__ void hadamard64_regs(float (&v)[64]) {
#pragma unroll
  for (int h = 1; h < 64; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      if ((i & h) == 0) {
        const float a = v[i], b = v[i + h];
        v[i] = a + b;
        v[i + h] = a - b;
      }
    }
  }
}

template <int K2>
__device__ __forceinline__ void load_stage_words(StageWords<K2> &sw, const uint32_t *col0, int lane, uint64_t row_words, uint32_t ks) {
  // tile rows 4 ks .. 4 ks + 3 of the warp's tile column
  const uint32_t *base = col0 + static_cast<uint64_t>(ks) * 4u * row_words + lane;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const uint32_t *t = base + static_cast<uint64_t>(r) * row_words;
#pragma unroll
    for (int h = 0; h < StageWords<K2>::kPerTile; ++h) {
      sw.w[r][h] = (32 * h + lane < 4 * K2) ? __ldg(t + 32 * h) : 0u;
    }
  }
}

// Word `index` of a tile whose words lie one per lane (and, beyond 32, in the second register).
template <int K2>
__device__ __forceinline__ uint32_t tile_word(const uint32_t (&w)[(4 * K2 + 31) / 32], uint32_t index) {
  if ((4 * K2 + 31) / 32 == 1) return __shfl_sync(0xFFFFFFFFu, w[0], static_cast<int>(index));
  const uint32_t lo = __shfl_sync(0xFFFFFFFFu, w[0], static_cast<int>(index & 31u));
  const uint32_t hi = __shfl_sync(0xFFFFFFFFu, w[(4 * K2 + 31) / 32 - 1], static_cast<int>(index & 31u));
  return index < 32u ? lo : hi;
}

// The decoder warps' loop over the job's K stages. `stages_base` is the shared-memory address of
// stage 0; `bars`: full[kStages], empty[kStages].
template <int K2, int DW>
__device__ __forceinline__ bool decode_stages(const Job &job, uint32_t stages_base, uint32_t bars, int warp, int lane, uint32_t *status) {
  constexpr uint32_t kStages = Shape<DW>::kStages, kStageBytes = Shape<DW>::kStageBytes;
  const LaneWindow win = lane_window(K2, lane);
  const uint32_t k_stages = job.in / 64u;
  const uint32_t cb = static_cast<uint32_t>(warp) >> 3;                    // which of the job's two column blocks
  const uint32_t blk = cb == 0u ? job.blk0 : job.blk1;
  const uint32_t tn = blk * 8u + (static_cast<uint32_t>(warp) & 7u);        // the warp's tile column in the plane
  const uint64_t row_words = static_cast<uint64_t>(job.tile_stride) * 4u * K2;
  const uint32_t *col0 = job.trellis + static_cast<uint64_t>(tn) * 4u * K2;
  const bool live = cb < job.nblk;
  const uint32_t c0 = static_cast<uint32_t>(lane) >> 2, t = static_cast<uint32_t>(lane) & 3u;
  // row n = 16 warp + c0 (+ 8) of the B tile: 8-row group 2 warp (+ 1)
  const uint32_t lane_off = kABytes * 2u + (2u * static_cast<uint32_t>(warp)) * 1024u + c0 * 128u + 4u * t;
  // The words of the next kWordRing stages are in flight in registers: a load issued when its
  // stage's slot of the ring was last decoded has several stage times to arrive (one stage ahead is
  // not enough: a stage is shorter than the latency of HBM).
  StageWords<K2> ring[kWordRing];
#pragma unroll
  for (int d = 0; d < kWordRing; ++d) {   // the weights never depend on the previous kernel
    if (live && static_cast<uint32_t>(d) < k_stages) load_stage_words<K2>(ring[d], col0, lane, row_words, static_cast<uint32_t>(d));
  }
  griddep_launch_dependents();
  griddep_wait();   // from here on the warp may also touch what an earlier kernel wrote
  for (uint32_t it0 = 0; it0 < k_stages; it0 += kWordRing) {
#pragma unroll
    for (int d = 0; d < kWordRing; ++d) {
      const uint32_t it = it0 + static_cast<uint32_t>(d);
      if (it >= k_stages) break;
      const uint32_t slot = it % kStages;
      if (!mbar_wait(bars + 8u * (kStages + slot), ((it / kStages) & 1u) ^ 1u)) {
        if (lane == 0) atomicOr(status, kStatusDecoder);
        return false;
      }
      if (live) {
        const uint32_t tile = stages_base + slot * kStageBytes + lane_off;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const uint32_t w0 = tile_word<K2>(ring[d].w[r], win.w0), w1 = tile_word<K2>(ring[d].w[r], win.w1),
                         w2 = tile_word<K2>(ring[d].w[r], win.w2);
          uint32_t frag[4];
          decode8<K2>(w0, w1, w2, win.off, frag);
          const uint32_t lo = ((2u * r) ^ c0) << 4, hi = ((2u * r + 1u) ^ c0) << 4;
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile + lo), "r"(frag[0]) : "memory");
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile + hi), "r"(frag[1]) : "memory");
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile + 1024u + lo), "r"(frag[2]) : "memory");
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile + 1024u + hi), "r"(frag[3]) : "memory");
        }
        // the tile is read by the tensor core (async proxy): order these writes before it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      mbar_arrive(bars + 8u * slot);
      if (live && it + kWordRing < k_stages) load_stage_words<K2>(ring[d], col0, lane, row_words, it + kWordRing);
    }
  }
  return true;
}

template <int DW>
__device__ __forceinline__ bool decode_stages_any(const Job &job, uint32_t stages_base, uint32_t bars, int warp, int lane, uint32_t *status) {
  switch (job.k2) {
    case 4: return decode_stages<4, DW>(job, stages_base, bars, warp, lane, status);
    case 5: return decode_stages<5, DW>(job, stages_base, bars, warp, lane, status);
    case 6: return decode_stages<6, DW>(job, stages_base, bars, warp, lane, status);
    case 8: return decode_stages<8, DW>(job, stages_base, bars, warp, lane, status);
    case 10: return decode_stages<10, DW>(job, stages_base, bars, warp, lane, status);
    default: return decode_stages<12, DW>(job, stages_base, bars, warp, lane, status);
  }
}

// Shared-memory carve-up and the three roles up to the finished accumulator. On return with true,
// the calling decoder warp may read the accumulators: tensor-memory columns [256 tt, 256 tt + 256)
// hold row tile tt, lanes = rows, the job's block 0 in the first 128 columns of a tile. The caller
// ends with core_finish().
struct Core {
  uint32_t base, bars, bar_acc, tmem;
  uint32_t *tmem_slot;
  int warp, lane;
};

template <int DW>
__device__ __forceinline__ Core core_setup(uint8_t *smem_raw) {
  constexpr uint32_t kStages = Shape<DW>::kStages, kStageBytes = Shape<DW>::kStageBytes, kTmemCols = Shape<DW>::kTmemCols;
  constexpr int kDecoderWarps = DW;
  Core c;
  const uint32_t raw = smem_u32(smem_raw);
  c.base = (raw + 1023u) & ~1023u;   // the 128-byte swizzle wants 1024-byte aligned tiles
  c.bars = c.base + kStages * kStageBytes;       // full[kStages], empty[kStages], accumulator full
  c.bar_acc = c.bars + 8u * 2u * kStages;
  c.tmem_slot = reinterpret_cast<uint32_t *>(smem_raw + (c.base - raw) + kStages * kStageBytes + 128);
  c.warp = threadIdx.x >> 5;
  c.lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < kStages; ++s) {
      mbar_init(c.bars + 8u * s, kDecoderWarps * 32 + 1);   // every decoder thread and the producer's expect_tx arrival
      mbar_init(c.bars + 8u * (kStages + s), 1);            // the MMA thread's commit
    }
    mbar_init(c.bar_acc, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (c.warp == kDecoderWarps + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(c.tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  c.tmem = *c.tmem_slot;
  return c;
}

// The decoder warps' second step: waits for the accumulator. Returns true in the decoder warps when
// all of them have the complete accumulator (the epilogue may read tensor memory and use barrier 1).
// Every decoder warp calls it, with what core_roles returned to it.
template <int DW>
__device__ __forceinline__ bool core_accumulator(const Core &c, bool decoded, uint32_t *status) {
  constexpr int kDecoderWarps = DW;
  bool have = false;
  if (decoded) {
    have = mbar_wait(c.bar_acc, 0u);
    if (!have && c.lane == 0) atomicOr(status, kStatusEpilogue);
  }
  // The epilogue's warps meet at barriers of their own: either every decoder warp has its
  // accumulator or none goes on (a warp whose wait ran out must not leave the others waiting).
  uint32_t all;
  asm volatile("{ .reg .pred p, q; setp.ne.u32 p, %1, 0; bar.red.and.pred q, 1, %2, p; selp.u32 %0, 1, 0, q; }"
               : "=r"(all) : "r"(static_cast<uint32_t>(have)), "n"(kDecoderWarps * 32) : "memory");
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  return all != 0u;
}

// Runs the CTA's roles: the producer and the MMA thread to their end, the decoder warps through
// their K stages. Returns true in a decoder warp that decoded all of them; such a warp has time for
// loads of its own (what its epilogue will need) before it calls core_accumulator, while the last
// MMAs retire.
template <int DW>
__device__ __forceinline__ bool core_roles(const Core &c, const Job &job, const CUtensorMap *map_a, uint32_t *status) {
  constexpr uint32_t kStages = Shape<DW>::kStages, kStageBytes = Shape<DW>::kStageBytes;
  constexpr int kDecoderWarps = DW;
  const uint32_t k_stages = job.in / 64u;
  const uint32_t row_tiles = job.rows > 128u ? 2u : 1u;
  if (c.warp < kDecoderWarps) return decode_stages_any<DW>(job, c.base, c.bars, c.warp, c.lane, status);
  if (c.warp == kDecoderWarps) {
    // ---- producer of the activation tiles ----
    griddep_launch_dependents();
    griddep_wait();   // the rotated activations come from the kernel before
    if (c.lane == 0) {
      for (uint32_t it = 0; it < k_stages; ++it) {
        const uint32_t slot = it % kStages;
        if (!mbar_wait(c.bars + 8u * (kStages + slot), ((it / kStages) & 1u) ^ 1u)) {
          atomicOr(status, kStatusProducer);
          break;
        }
        const uint32_t full = c.bars + 8u * slot;
        mbar_expect_tx(full, row_tiles * kABytes);
        const uint32_t stage = c.base + slot * kStageBytes;
        tma_load_2d(stage, map_a, full, static_cast<int32_t>(it * 64u), static_cast<int32_t>(job.row0));
        if (row_tiles == 2u) tma_load_2d(stage + kABytes, map_a, full, static_cast<int32_t>(it * 64u), static_cast<int32_t>(job.row0 + 128u));
      }
    }
    return false;
  }
  // ---- MMA issuer ----
  griddep_launch_dependents();
  griddep_wait();
  if (c.lane == 0) {
    // instruction descriptor: FP32 accumulator (bit 4), A and B FP16 (format 0), both K-major,
    // N >> 3 at bit 17, M >> 4 at bit 24
    const uint32_t mma_n = job.nblk * 128u;
    const uint32_t idesc = (1u << 4) | ((mma_n >> 3) << 17) | ((128u >> 4) << 24);
    bool ok = true;
    for (uint32_t it = 0; it < k_stages; ++it) {
      const uint32_t slot = it % kStages;
      if (!mbar_wait(c.bars + 8u * slot, (it / kStages) & 1u)) {
        atomicOr(status, kStatusMma);
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t stage = c.base + slot * kStageBytes;
      const uint64_t a0 = smem_desc_sw128(stage), a1 = smem_desc_sw128(stage + kABytes), b = smem_desc_sw128(stage + 2u * kABytes);
#pragma unroll
      for (uint32_t kb = 0; kb < 4; ++kb) {   // 16 values along K are 32 bytes: two 16-byte units further
        mma_f16(c.tmem, a0 + 2u * kb, b + 2u * kb, idesc, (it | kb) != 0u ? 1u : 0u);
        if (row_tiles == 2u) mma_f16(c.tmem + Shape<DW>::kCols, a1 + 2u * kb, b + 2u * kb, idesc, (it | kb) != 0u ? 1u : 0u);
      }
      mma_commit(c.bars + 8u * (kStages + slot));
    }
    if (ok) mma_commit(c.bar_acc);
  }
  return false;
}

// Both steps back to back.
template <int DW>
__device__ __forceinline__ bool core_run(const Core &c, const Job &job, const CUtensorMap *map_a, uint32_t *status) {
  const bool decoded = core_roles<DW>(c, job, map_a, status);
  return c.warp < DW ? core_accumulator<DW>(c, decoded, status) : false;
}

// ---- epilogue ------------------------------------------------------------------------------------
// A warp group (warp / 4: four warps, 128 threads = the 128 rows of a row tile, a warp's lanes the
// rows 32 (warp % 4) .. + 31) owns 32 KB of the idle stage ring as [value 64][row 128] floats. The
// row's low five bits are XORed with the value index, so a warp's accesses are free of bank
// conflicts both when its lanes are 32 rows of one value (a thread parking its row) and when they
// are 32 values of one row (the warp writing a row out).
__device__ __forceinline__ uint32_t stash_at(uint32_t i, uint32_t t) { return i * 128u + (t & 96u) + ((t ^ i) & 31u); }

// Hands the calling warp's first `rows` rows of 64 parked values to `emit(r, lo, hi)`: lane l gets
// values l and l + 32 of row r, so what the caller stores per row is contiguous across the warp.
// (A thread storing its own row touches 32 different lines per instruction, and the memory pipe
// takes them one per cycle: the row-wise form is what makes the epilogue short.)
template <class RowEmit>
__device__ __forceinline__ void emit_rows(const float *area, uint32_t quad, uint32_t lane, uint32_t rows, RowEmit emit) {
  for (uint32_t r = 0; r < rows; ++r) {
    const uint32_t t = quad * 32u + r;
    emit(r, area[stash_at(lane, t)], area[stash_at(lane + 32u, t)]);
  }
}

__device__ __forceinline__ void load_half_row(uint32_t taddr, float inv, float (&v)[64]) {
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    uint32_t r[32];
    tmem_ld32(taddr + 32u * q, r);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[32 * q + i] = __uint_as_float(r[i]) * inv;
  }
}

// The epilogue of one (row tile, block) item for the calling warp: a thread owns one row (lane =
// row 32 quad + lane of the row tile; `rows` of the warp's 32 exist, `valid` = lane < rows) and
// `taddr` is the tensor-memory address of the block's first column in those lanes. The thread
// applies `inv` and six Hadamard stages to each half of its 128 columns in registers, the seventh
// stage combines the halves through `area`, and `emit(pass, r, lo, hi)` receives, a row at a
// time, columns 64 pass + lane (lo) and 64 pass + 32 + lane (hi), 1 / sqrt(128) included.
template <class RowEmit>
__device__ __forceinline__ void block_epilogue(uint32_t taddr, float inv, bool valid, float *area, uint32_t quad, uint32_t lane,
                                               uint32_t rows, RowEmit emit) {
  const uint32_t t = quad * 32u + lane;
  float v[64];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    load_half_row(taddr + 64u * half, inv, v);
    if (valid) {
      hadamard64_regs(v);
      if (half == 0) {
#pragma unroll
        for (int i = 0; i < 64; ++i) area[stash_at(i, t)] = v[i];
      }
    }
  }
  const float c = 0.08838834764831845f;   // 1 / sqrt(128)
  if (valid) {   // the seventh stage: columns i (sum, parked) and 64 + i (difference, kept)
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      const float a = area[stash_at(i, t)], b = v[i];
      area[stash_at(i, t)] = (a + b) * c;
      v[i] = (a - b) * c;
    }
  }
  __syncwarp();
  emit_rows(area, quad, lane, rows, [&](uint32_t r, float lo, float hi) { emit(0u, r, lo, hi); });
  __syncwarp();
  if (valid) {
#pragma unroll
    for (int i = 0; i < 64; ++i) area[stash_at(i, t)] = v[i];
  }
  __syncwarp();
  emit_rows(area, quad, lane, rows, [&](uint32_t r, float lo, float hi) { emit(1u, r, lo, hi); });
}

// The same for a job of one row tile, where only two of the four warp groups would have a block:
// groups g and g ^ 2 share block g & 1, a thread owning 64 columns of its row (half = g >> 1). Each
// transforms its half and parks it in its group's area (`mine`); all decoder warps meet at barrier 1;
// the seventh stage gives the first half's owner columns 0..63 (sums) and the other's columns
// 64..127 (differences), parked again after a second meeting and written out row-wise:
// `emit(half, r, lo, hi)` as above. Every decoder warp calls this exactly once (`live`: the group's
// block exists - warp-uniform).
template <int DW, class RowEmit>
__device__ __forceinline__ void half_epilogue(uint32_t taddr_block, uint32_t half, bool live, float inv, bool valid, float *mine,
                                              const float *other, uint32_t quad, uint32_t lane, uint32_t rows, RowEmit emit) {
  const uint32_t t = quad * 32u + lane;
  float v[64];
  if (live) {
    load_half_row(taddr_block + 64u * half, inv, v);
    if (valid) {
      hadamard64_regs(v);
#pragma unroll
      for (int i = 0; i < 64; ++i) mine[stash_at(i, t)] = v[i];
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(DW * 32) : "memory");
  const float c = 0.08838834764831845f;   // 1 / sqrt(128)
  if (live && valid) {
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      const float o = other[stash_at(i, t)];
      v[i] = half == 0u ? (v[i] + o) * c : (o - v[i]) * c;
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(DW * 32) : "memory");
  if (!live) return;
  if (valid) {
#pragma unroll
    for (int i = 0; i < 64; ++i) mine[stash_at(i, t)] = v[i];
  }
  __syncwarp();
  emit_rows(mine, quad, lane, rows, [&](uint32_t r, float lo, float hi) { emit(half, r, lo, hi); });
}

template <int DW>
__device__ __forceinline__ void core_finish(const Core &c) {
  constexpr int kDecoderWarps = DW;
  constexpr uint32_t kTmemCols = Shape<DW>::kTmemCols;
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (c.warp == kDecoderWarps + 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(c.tmem), "r"(kTmemCols) : "memory");
  }
}

// The rotated activations [rows][in] fp16 as a 2-D tensor with boxes of 128 rows x 64 values, 128-byte swizzle.
inline bool make_rows_map(CUtensorMap *map, const void *rows_f16, uint64_t rows, uint64_t in) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {in, rows};
  const cuuint64_t strides[1] = {in * 2u};
  const cuuint32_t box[2] = {64u, 128u};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(rows_f16), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace trellis_tc
}  // namespace b200q

#endif
