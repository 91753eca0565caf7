// Thin C entry points over the reference's OWN host-side oracle code, compiled from the
// reference's headers where they lie in its checkout (nothing of it is copied here):
//   kernel/vendor/tests/ops/quantized_weight.h   NVFP4 patterned weights and logical_weight_fp64
//   kernel/tests/moe_fixture.h                   trellis host decoder, counter hash, checksum,
//                                                Hadamard and fp64 projection
// TEST INFRASTRUCTURE ONLY: built by oracle/build.py into oracle/_ref/, loaded by the tests to
// validate oracle/b200q_oracle.c and by the benchmark's CPU-baseline leg. The library never
// loads it.
#include "ops/quantized_weight.h"

#include "moe_fixture.h"

#include <cstdint>
#include <cstring>
#include <vector>

namespace qw = ninfer::test::quantized_weight;

extern "C" {

// Patterned NVFP4 weight of the reference's linear tests; planes copied out.
int32_t ref_nvfp4_patterned(int32_t n, int32_t k, uint32_t seed, float d_w, float d_in, uint8_t *codes,
                            uint8_t *scales) {
  try {
    qw::PatternedWeightOptions options;
    options.weight_scale_divisor = d_w;
    options.input_scale_divisor = d_in;
    const qw::PackedWeight packed = qw::make_patterned_weight(ninfer::QType::NVFP4, n, k, seed, options);
    std::memcpy(codes, packed.payload.data(), packed.code_plane_bytes);
    std::memcpy(scales, packed.payload.data() + packed.scale_plane_offset, packed.scale_plane_bytes);
    return 0;
  } catch (...) {
    return -1;
  }
}

// logical_weight_fp64 over rows [row0, row1) of caller-supplied planes, as float.
int32_t ref_nvfp4_dequant(const uint8_t *codes, const uint8_t *scales, int32_t n, int32_t k, float d_w,
                          int32_t row0, int32_t row1, float *out) {
  try {
    qw::PatternedWeightOptions options;
    options.weight_scale_divisor = d_w;
    options.input_scale_divisor = 1.0F;
    qw::PackedWeight packed = qw::make_patterned_weight(ninfer::QType::NVFP4, n, k, 0, options);
    std::memcpy(packed.payload.data(), codes, packed.code_plane_bytes);
    std::memcpy(packed.payload.data() + packed.scale_plane_offset, scales, packed.scale_plane_bytes);
    for (int32_t r = row0; r < row1; ++r) {
      for (int32_t c = 0; c < k; ++c) {
        out[static_cast<std::size_t>(r - row0) * k + c] = static_cast<float>(qw::logical_weight_fp64(packed, r, c));
      }
    }
    return 0;
  } catch (...) {
    return -1;
  }
}

void ref_trellis_decode(const uint16_t *words, uint32_t k2, int32_t in, int32_t out, uint16_t *inner) {
  const std::vector<uint16_t> w = moe_test::host_trellis_decode(words, k2, in, out);
  std::memcpy(inner, w.data(), w.size() * sizeof(uint16_t));
}

void ref_hash_trellis_words(uint32_t stream, int32_t in, int32_t out, uint32_t k2, uint16_t *words) {
  const std::vector<uint16_t> w = moe_test::hash_trellis_words(stream, in, out, k2);
  std::memcpy(words, w.data(), w.size() * sizeof(uint16_t));
}

uint64_t ref_checksum_u16(const uint16_t *v, uint64_t n) {
  return moe_test::checksum_u16(std::vector<uint16_t>(v, v + n));
}

float ref_hash_uniform(uint32_t stream, uint64_t i, float amplitude) {
  return moe_test::hash_uniform(stream, i, amplitude);
}

void ref_trellis_project(const uint16_t *inner, const uint16_t *suh, const uint16_t *svh, int32_t in,
                         int32_t out, const double *x, double *y) {
  const std::vector<uint16_t> w(inner, inner + static_cast<std::size_t>(in) * out);
  const std::vector<double> r = moe_test::project_f64(w, suh, svh, in, out, x);
  std::memcpy(y, r.data(), r.size() * sizeof(double));
}

}  // extern "C"
