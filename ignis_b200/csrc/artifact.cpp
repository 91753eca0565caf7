// Reader of the `.ninfer` v2 container behind the C ABI of include/b200q_artifact.h. Host code only.
//
// Follows crates/artifact/src/lib.rs of the reference check for check and message for message:
// framing (:145-161, :1075-1115), the closed JSON directory (:743-856), payload geometry of every
// registered layout (:421-660), ordering / alignment / bounds / duplicates (:1130-1160) and the
// structural content hash (:1204-1240). The JSON parser and SHA-256 below are this file's own (the
// reference takes them from serde_json and sha2).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../../include/b200q_artifact.h"

namespace {

thread_local char g_error[512] = "";

int32_t fail(const char *fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return -1;
}

constexpr uint64_t kPrefixBytes = 16, kPayloadAlignment = 4096, kDirectIoAlignment = 4096, kTensorAlignment = 256,
                   kKAlignment = 128;
const uint8_t kMagic[8] = {'N', 'I', 'N', 'F', 'E', 'R', 0, 2};
const uint8_t kV1Magic[8] = {'N', 'I', 'N', 'F', 'E', 'R', 0, 1};

// ---- checked arithmetic ------------------------------------------------------------------------

bool checked_add(uint64_t a, uint64_t b, const char *label, uint64_t *out) {
  if (a > UINT64_MAX - b) {
    fail("%s overflows", label);
    return false;
  }
  *out = a + b;
  return true;
}

bool checked_mul(uint64_t a, uint64_t b, const char *label, uint64_t *out) {
  if (a != 0 && b > UINT64_MAX / a) {
    fail("%s overflows", label);
    return false;
  }
  *out = a * b;
  return true;
}

bool align_up(uint64_t value, uint64_t alignment, const char *label, uint64_t *out) {
  const uint64_t rem = value % alignment;
  if (rem == 0) {
    *out = value;
    return true;
  }
  return checked_add(value, alignment - rem, label, out);
}

// ---- registries --------------------------------------------------------------------------------

const char *const kFormatNames[] = {nullptr,
                                    "BF16",
                                    "FP32",
                                    "I32",
                                    "Q4G64_F16S",
                                    "Q5G64_F16S",
                                    "Q6G64_F16S",
                                    "W8G32_F16S",
                                    "NVFP4",
                                    "FP8_E4M3FN_ROW_BF16S",
                                    "I64",
                                    "Q4G32_F16S",
                                    "TRELLIS_MUL1_K2",
                                    "TRELLIS_MUL1_K2P5",
                                    "TRELLIS_MUL1_K3",
                                    "TRELLIS_MUL1_K4",
                                    "TRELLIS_MUL1_K5",
                                    "TRELLIS_MUL1_K6"};
constexpr uint32_t kFormatCount = sizeof(kFormatNames) / sizeof(kFormatNames[0]);

const char *const kLayoutNames[] = {nullptr,
                                    "contiguous-le-v1",
                                    "row-split-k128-v1",
                                    "blockscale-k16-m128x4-v1",
                                    "row-scale-v1",
                                    "trellis-tile16-v1",
                                    "row-interleaved-v1",
                                    "raw-bytes-v1"};
constexpr uint32_t kLayoutCount = sizeof(kLayoutNames) / sizeof(kLayoutNames[0]);

uint32_t trellis_k2(uint32_t format) {
  switch (format) {
    case B200Q_FORMAT_TRELLIS_MUL1_K2: return 4;
    case B200Q_FORMAT_TRELLIS_MUL1_K2P5: return 5;
    case B200Q_FORMAT_TRELLIS_MUL1_K3: return 6;
    case B200Q_FORMAT_TRELLIS_MUL1_K4: return 8;
    case B200Q_FORMAT_TRELLIS_MUL1_K5: return 10;
    case B200Q_FORMAT_TRELLIS_MUL1_K6: return 12;
    default: return 0;
  }
}

uint64_t layout_alignment(uint32_t layout) {
  switch (layout) {
    case B200Q_LAYOUT_TRELLIS_TILE16_V1:
    case B200Q_LAYOUT_ROW_INTERLEAVED_V1: return kDirectIoAlignment;
    case B200Q_LAYOUT_RAW_BYTES_V1: return 1;
    default: return kTensorAlignment;
  }
}

// ---- payload geometry --------------------------------------------------------------------------

bool require_rank2(const char *label, const uint64_t *shape, uint32_t rank) {
  if (rank != 2 || shape[0] == 0 || shape[1] == 0) {
    fail("%s requires a positive rank-two shape", label);
    return false;
  }
  return true;
}

bool blockscale_geometry(uint32_t format, const uint64_t *shape, uint32_t rank, b200q_blockscale_geometry *g) {
  if (format != B200Q_FORMAT_NVFP4) return fail("blockscale-k16-m128x4-v1 requires NVFP4"), false;
  if (!require_rank2("blockscale-k16-m128x4-v1", shape, rank)) return false;
  const uint64_t rows = shape[0], columns = shape[1];
  if (rows % 128 != 0 || columns % 64 != 0)
    return fail("blockscale-k16-m128x4-v1 requires N divisible by 128 and K divisible by 64"), false;
  uint64_t elements;
  if (!checked_mul(rows, columns, "NVFP4 element count", &elements)) return false;
  g->rows = rows;
  g->columns = columns;
  g->groups_per_row = columns / 16;
  g->k_tiles = columns / 64;
  g->code_plane_bytes = elements / 2;
  if (!align_up(g->code_plane_bytes, kTensorAlignment, "NVFP4 scale plane offset", &g->scale_plane_offset)) return false;
  g->scale_plane_bytes = elements / 16;
  if (!checked_add(g->scale_plane_offset, g->scale_plane_bytes, "NVFP4 weight divisor offset", &g->weight_divisor_offset))
    return false;
  return checked_add(g->weight_divisor_offset, 4, "NVFP4 tensor encoded size", &g->encoded_bytes);
}

bool trellis_geometry(uint32_t format, const uint64_t *shape, uint32_t rank, b200q_trellis_geometry *g) {
  const uint64_t k2 = trellis_k2(format);
  if (k2 == 0) return fail("trellis-tile16-v1 requires a TRELLIS format"), false;
  if (!require_rank2("trellis-tile16-v1", shape, rank)) return false;
  const uint64_t rows = shape[0], columns = shape[1];
  if (rows % 128 != 0 || columns % 128 != 0)
    return fail("trellis-tile16-v1 requires both dimensions divisible by 128"), false;
  uint64_t elements, suh_bytes, svh_bytes;
  if (!checked_mul(rows, columns, "trellis element count", &elements)) return false;
  // 16 K int16 words per tile of 256 weights: elements 2K / 16 bytes
  if (!checked_mul(elements / 16, k2, "trellis plane bytes", &g->trellis_bytes)) return false;
  g->rows = rows;
  g->columns = columns;
  g->k2 = k2;
  g->suh_offset = g->trellis_bytes;
  if (!checked_mul(columns, 2, "suh bytes", &suh_bytes) || !checked_add(g->suh_offset, suh_bytes, "svh offset", &g->svh_offset))
    return false;
  if (!checked_mul(rows, 2, "svh bytes", &svh_bytes) || !checked_add(g->svh_offset, svh_bytes, "trellis data bytes", &g->data_bytes))
    return false;
  return align_up(g->data_bytes, kDirectIoAlignment, "trellis record bytes", &g->encoded_bytes);
}

bool row_split_bytes(uint32_t format, const uint64_t *shape, uint32_t rank, uint64_t *bytes) {
  if (!require_rank2("row-split-k128-v1", shape, rank)) return false;
  uint64_t group, low_bpg, high_bpg;
  switch (format) {
    case B200Q_FORMAT_Q4G64_F16S: group = 64, low_bpg = 32, high_bpg = 0; break;
    case B200Q_FORMAT_Q5G64_F16S: group = 64, low_bpg = 32, high_bpg = 8; break;
    case B200Q_FORMAT_Q6G64_F16S: group = 64, low_bpg = 32, high_bpg = 16; break;
    case B200Q_FORMAT_W8G32_F16S: group = 32, low_bpg = 32, high_bpg = 0; break;
    default: return fail("row-split-k128-v1 requires a grouped quantized format"), false;
  }
  uint64_t padded, groups, low, high, scale, high_offset, aligned_high, scale_offset;
  if (!align_up(shape[1], kKAlignment, "padded K", &padded)) return false;
  if (!checked_mul(shape[0], padded / group, "physical group count", &groups)) return false;
  if (!checked_mul(groups, low_bpg, "base plane bytes", &low) || !checked_mul(groups, high_bpg, "high plane bytes", &high) ||
      !checked_mul(groups, 2, "scale plane bytes", &scale))
    return false;
  if (!align_up(low, kTensorAlignment, "high plane offset", &high_offset) ||
      !align_up(high, kTensorAlignment, "scale plane alignment", &aligned_high) ||
      !checked_add(high_offset, aligned_high, "scale plane offset", &scale_offset))
    return false;
  return checked_add(scale_offset, scale, "tensor encoded size", bytes);
}

bool row_scale_bytes(uint32_t format, const uint64_t *shape, uint32_t rank, uint64_t *bytes) {
  if (format != B200Q_FORMAT_FP8_E4M3FN_ROW_BF16S) return fail("row-scale-v1 requires FP8_E4M3FN_ROW_BF16S"), false;
  if (!require_rank2("row-scale-v1", shape, rank)) return false;
  uint64_t codes, scale_offset, scales;
  if (!checked_mul(shape[0], shape[1], "FP8 element count", &codes) ||
      !align_up(codes, kTensorAlignment, "FP8 scale plane offset", &scale_offset) ||
      !checked_mul(shape[0], 2, "FP8 scale plane bytes", &scales))
    return false;
  return checked_add(scale_offset, scales, "FP8 tensor encoded size", bytes);
}

bool row_interleaved_bytes(uint32_t format, const uint64_t *shape, uint32_t rank, uint64_t *bytes) {
  if (format != B200Q_FORMAT_Q4G32_F16S) return fail("row-interleaved-v1 requires Q4G32_F16S"), false;
  if (!require_rank2("row-interleaved-v1", shape, rank)) return false;
  if (shape[1] % 32 != 0) return fail("row-interleaved-v1 requires a column count divisible by 32"), false;
  const uint64_t row_bytes = shape[1] / 2 + shape[1] / 32 * 2;
  return checked_mul(shape[0], row_bytes, "row-interleaved tensor encoded size", bytes);
}

bool encoded_size(uint32_t layout, uint32_t format, const uint64_t *shape, uint32_t rank, uint64_t *bytes) {
  switch (layout) {
    case B200Q_LAYOUT_CONTIGUOUS_LE_V1: {
      if (rank > 16) return fail("contiguous-le-v1 supports rank 0 through 16"), false;
      uint64_t elements = 1;
      for (uint32_t i = 0; i < rank; ++i) {
        if (shape[i] == 0) return fail("tensor shape dimensions must be positive"), false;
        if (!checked_mul(elements, shape[i], "tensor element count", &elements)) return false;
      }
      uint64_t word;
      switch (format) {
        case B200Q_FORMAT_BF16: word = 2; break;
        case B200Q_FORMAT_FP32:
        case B200Q_FORMAT_I32: word = 4; break;
        case B200Q_FORMAT_I64: word = 8; break;
        default: return fail("contiguous-le-v1 requires BF16, FP32, I32, or I64"), false;
      }
      return checked_mul(elements, word, "tensor encoded size", bytes);
    }
    case B200Q_LAYOUT_ROW_SPLIT_K128_V1: return row_split_bytes(format, shape, rank, bytes);
    case B200Q_LAYOUT_BLOCKSCALE_K16_M128X4_V1: {
      b200q_blockscale_geometry g;
      if (!blockscale_geometry(format, shape, rank, &g)) return false;
      *bytes = g.encoded_bytes;
      return true;
    }
    case B200Q_LAYOUT_ROW_SCALE_V1: return row_scale_bytes(format, shape, rank, bytes);
    case B200Q_LAYOUT_TRELLIS_TILE16_V1: {
      b200q_trellis_geometry g;
      if (!trellis_geometry(format, shape, rank, &g)) return false;
      *bytes = g.encoded_bytes;
      return true;
    }
    case B200Q_LAYOUT_ROW_INTERLEAVED_V1: return row_interleaved_bytes(format, shape, rank, bytes);
    default: return fail("unknown tensor layout"), false;
  }
}

// ---- JSON: the subset a directory uses, parsed strictly ----------------------------------------

struct Json {
  enum Type { kNull, kBool, kNumber, kString, kArray, kObject } type = kNull;
  bool boolean = false;
  bool is_unsigned = false;  // a number written as a plain non-negative integer that fits 64 bits
  uint64_t number = 0;
  std::string string;
  std::vector<Json> items;
  std::vector<std::pair<std::string, Json>> members;  // in file order; duplicates are an error at parse

  const Json *get(const char *key) const {
    for (const auto &m : members)
      if (m.first == key) return &m.second;
    return nullptr;
  }
};

class JsonParser {
 public:
  JsonParser(const char *begin, const char *end) : p_(begin), end_(end) {}

  bool parse(Json *out) {
    if (!value(out, 0)) return false;
    space();
    if (p_ != end_) return error("trailing characters");
    return true;
  }
  const std::string &message() const { return message_; }

 private:
  const char *p_, *end_;
  std::string message_;

  bool error(const char *what) {
    if (message_.empty()) message_ = what;
    return false;
  }
  void space() {
    while (p_ != end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
  }
  bool literal(const char *text) {
    const size_t n = strlen(text);
    if (static_cast<size_t>(end_ - p_) < n || memcmp(p_, text, n) != 0) return error("invalid literal");
    p_ += n;
    return true;
  }
  static void utf8(uint32_t cp, std::string *s) {
    if (cp < 0x80) {
      s->push_back(static_cast<char>(cp));
    } else if (cp < 0x800) {
      s->push_back(static_cast<char>(0xC0 | (cp >> 6)));
      s->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
      s->push_back(static_cast<char>(0xE0 | (cp >> 12)));
      s->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      s->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
      s->push_back(static_cast<char>(0xF0 | (cp >> 18)));
      s->push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
      s->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      s->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
  }
  bool hex4(uint32_t *cp) {
    if (end_ - p_ < 4) return error("short \\u escape");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
      const char c = *p_++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= static_cast<uint32_t>(c - '0');
      else if (c >= 'a' && c <= 'f') v |= static_cast<uint32_t>(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') v |= static_cast<uint32_t>(c - 'A' + 10);
      else return error("bad \\u escape");
    }
    *cp = v;
    return true;
  }
  bool string(std::string *out) {
    ++p_;  // the opening quote
    while (true) {
      if (p_ == end_) return error("unterminated string");
      const unsigned char c = static_cast<unsigned char>(*p_++);
      if (c == '"') return true;
      if (c < 0x20) return error("control character in string");
      if (c != '\\') {
        out->push_back(static_cast<char>(c));
        continue;
      }
      if (p_ == end_) return error("unterminated escape");
      const char e = *p_++;
      switch (e) {
        case '"': out->push_back('"'); break;
        case '\\': out->push_back('\\'); break;
        case '/': out->push_back('/'); break;
        case 'b': out->push_back('\b'); break;
        case 'f': out->push_back('\f'); break;
        case 'n': out->push_back('\n'); break;
        case 'r': out->push_back('\r'); break;
        case 't': out->push_back('\t'); break;
        case 'u': {
          uint32_t cp;
          if (!hex4(&cp)) return false;
          if (cp >= 0xD800 && cp < 0xDC00) {  // a surrogate pair
            uint32_t low;
            if (end_ - p_ < 2 || p_[0] != '\\' || p_[1] != 'u') return error("lone surrogate");
            p_ += 2;
            if (!hex4(&low)) return false;
            if (low < 0xDC00 || low > 0xDFFF) return error("lone surrogate");
            cp = 0x10000 + ((cp - 0xD800) << 10) + (low - 0xDC00);
          } else if (cp >= 0xDC00 && cp < 0xE000) {
            return error("lone surrogate");
          }
          utf8(cp, out);
          break;
        }
        default: return error("bad escape");
      }
    }
  }
  bool number(Json *out) {
    const char *start = p_;
    bool integer = true;
    if (p_ != end_ && *p_ == '-') {
      integer = false;
      ++p_;
    }
    if (p_ == end_ || *p_ < '0' || *p_ > '9') return error("invalid number");
    if (*p_ == '0') {
      ++p_;
    } else {
      while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
    }
    if (p_ != end_ && *p_ == '.') {
      integer = false;
      ++p_;
      if (p_ == end_ || *p_ < '0' || *p_ > '9') return error("invalid number");
      while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
    }
    if (p_ != end_ && (*p_ == 'e' || *p_ == 'E')) {
      integer = false;
      ++p_;
      if (p_ != end_ && (*p_ == '+' || *p_ == '-')) ++p_;
      if (p_ == end_ || *p_ < '0' || *p_ > '9') return error("invalid number");
      while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
    }
    out->type = Json::kNumber;
    if (integer) {
      uint64_t v = 0;
      bool fits = true;
      for (const char *q = start; q != p_; ++q) {
        const uint64_t d = static_cast<uint64_t>(*q - '0');
        if (v > (UINT64_MAX - d) / 10) {
          fits = false;
          break;
        }
        v = v * 10 + d;
      }
      out->is_unsigned = fits;
      out->number = fits ? v : 0;
    }
    return true;
  }
  bool value(Json *out, int depth) {
    if (depth > 64) return error("nesting too deep");
    space();
    if (p_ == end_) return error("unexpected end");
    switch (*p_) {
      case '{': {
        ++p_;
        out->type = Json::kObject;
        space();
        if (p_ != end_ && *p_ == '}') {
          ++p_;
          return true;
        }
        while (true) {
          space();
          if (p_ == end_ || *p_ != '"') return error("expected a member name");
          std::string key;
          if (!string(&key)) return false;
          space();
          if (p_ == end_ || *p_ != ':') return error("expected ':'");
          ++p_;
          if (out->get(key.c_str()) != nullptr) return error("duplicate member");
          out->members.emplace_back(std::move(key), Json());
          if (!value(&out->members.back().second, depth + 1)) return false;
          space();
          if (p_ == end_) return error("unterminated object");
          if (*p_ == ',') {
            ++p_;
            continue;
          }
          if (*p_ == '}') {
            ++p_;
            return true;
          }
          return error("expected ',' or '}'");
        }
      }
      case '[': {
        ++p_;
        out->type = Json::kArray;
        space();
        if (p_ != end_ && *p_ == ']') {
          ++p_;
          return true;
        }
        while (true) {
          out->items.emplace_back();
          if (!value(&out->items.back(), depth + 1)) return false;
          space();
          if (p_ == end_) return error("unterminated array");
          if (*p_ == ',') {
            ++p_;
            continue;
          }
          if (*p_ == ']') {
            ++p_;
            return true;
          }
          return error("expected ',' or ']'");
        }
      }
      case '"': out->type = Json::kString; return string(&out->string);
      case 't': out->type = Json::kBool; out->boolean = true; return literal("true");
      case 'f': out->type = Json::kBool; out->boolean = false; return literal("false");
      case 'n': out->type = Json::kNull; return literal("null");
      default: return number(out);
    }
  }
};

// ---- SHA-256 (FIPS 180-4) ----------------------------------------------------------------------

class Sha256 {
 public:
  Sha256() {
    static const uint32_t init[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au,
                                     0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
    memcpy(h_, init, sizeof(h_));
  }
  void update(const void *data, size_t n) {
    const uint8_t *p = static_cast<const uint8_t *>(data);
    total_ += n;
    while (n > 0) {
      const size_t take = (64 - fill_) < n ? (64 - fill_) : n;
      memcpy(block_ + fill_, p, take);
      fill_ += take;
      p += take;
      n -= take;
      if (fill_ == 64) {
        compress();
        fill_ = 0;
      }
    }
  }
  void update_u64(uint64_t v) {
    uint8_t le[8];
    for (int i = 0; i < 8; ++i) le[i] = static_cast<uint8_t>(v >> (8 * i));
    update(le, 8);
  }
  void update_str0(const char *s) { update(s, strlen(s) + 1); }  // the bytes and a terminating zero
  void finish(uint8_t out[32]) {
    const uint64_t bits = total_ * 8;
    const uint8_t one = 0x80, zero = 0;
    update(&one, 1);
    while (fill_ != 56) update(&zero, 1);
    uint8_t be[8];
    for (int i = 0; i < 8; ++i) be[i] = static_cast<uint8_t>(bits >> (56 - 8 * i));
    update(be, 8);
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 4; ++j) out[4 * i + j] = static_cast<uint8_t>(h_[i] >> (24 - 8 * j));
  }

 private:
  uint32_t h_[8];
  uint8_t block_[64];
  size_t fill_ = 0;
  uint64_t total_ = 0;

  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void compress() {
    static const uint32_t k[64] = {
        0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u,
        0xd807aa98u, 0x12835b01u, 0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u,
        0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu, 0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau,
        0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u,
        0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u,
        0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u, 0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u,
        0x19a4c116u, 0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu, 0x682e6ff3u,
        0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u, 0xc67178f2u};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (static_cast<uint32_t>(block_[4 * i]) << 24) | (static_cast<uint32_t>(block_[4 * i + 1]) << 16) |
             (static_cast<uint32_t>(block_[4 * i + 2]) << 8) | block_[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h_[0], b = h_[1], c = h_[2], d = h_[3], e = h_[4], f = h_[5], g = h_[6], h = h_[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = h + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + k[i] + w[i];
      const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
      h = g, g = f, f = e, e = d + t1, d = c, c = b, b = a, a = t1 + t2;
    }
    h_[0] += a, h_[1] += b, h_[2] += c, h_[3] += d, h_[4] += e, h_[5] += f, h_[6] += g, h_[7] += h;
  }
};

// ---- the directory -----------------------------------------------------------------------------

struct Entry {
  std::string name;
  uint32_t kind = 0, format = 0, layout = 0;
  std::vector<uint64_t> shape;
  uint64_t offset = 0, bytes = 0;
};

bool require_members(const Json &value, std::initializer_list<const char *> members, const char *label) {
  if (value.type != Json::kObject) return fail("%s must be a JSON object", label), false;
  if (value.members.size() != members.size()) return fail("%s has missing or extra members", label), false;
  for (const char *m : members)
    if (value.get(m) == nullptr) return fail("%s has missing or extra members", label), false;
  return true;
}

bool require_string(const Json &value, const char *label, std::string *out) {
  if (value.type != Json::kString || value.string.empty()) return fail("%s must be a nonempty string", label), false;
  *out = value.string;
  return true;
}

bool require_unsigned(const Json &value, const char *label, bool positive, uint64_t *out) {
  if (value.type != Json::kNumber || !value.is_unsigned || (positive && value.number == 0))
    return fail("%s must be an integer", label), false;
  *out = value.number;
  return true;
}

uint32_t format_by_name(const std::string &name) {
  for (uint32_t i = 1; i < kFormatCount; ++i)
    if (name == kFormatNames[i]) return i;
  fail("unknown tensor format: %s", name.c_str());
  return 0;
}

uint32_t layout_by_name(const std::string &name) {
  for (uint32_t i = 1; i < kLayoutCount - 1; ++i)  // the last entry is the resource encoding
    if (name == kLayoutNames[i]) return i;
  fail("unknown tensor layout: %s", name.c_str());
  return 0;
}

bool parse_object(const Json &value, Entry *e) {
  if (value.type != Json::kObject) return fail("each object entry must be a JSON object"), false;
  const Json *kind = value.get("kind");
  if (kind == nullptr || kind->type != Json::kString) return fail("object kind must be 'tensor' or 'resource'"), false;
  std::string text;
  if (kind->string == "tensor") {
    if (!require_members(value, {"name", "kind", "shape", "format", "layout", "offset", "bytes"}, "tensor entry")) return false;
    e->kind = B200Q_ARTIFACT_TENSOR;
    if (!require_string(*value.get("name"), "tensor name", &e->name)) return false;
    if (!require_string(*value.get("format"), "tensor format", &text) || (e->format = format_by_name(text)) == 0) return false;
    if (!require_string(*value.get("layout"), "tensor layout", &text) || (e->layout = layout_by_name(text)) == 0) return false;
    if (!require_unsigned(*value.get("offset"), "tensor offset", false, &e->offset)) return false;
    if (!require_unsigned(*value.get("bytes"), "tensor bytes", true, &e->bytes)) return false;
    const Json &shape = *value.get("shape");
    if (shape.type != Json::kArray) return fail("tensor shape must be an array"), false;
    for (const Json &dim : shape.items) {
      uint64_t d;
      if (!require_unsigned(dim, "shape dimension", true, &d)) return false;
      e->shape.push_back(d);
    }
    uint64_t encoded;
    if (!encoded_size(e->layout, e->format, e->shape.data(), static_cast<uint32_t>(e->shape.size()), &encoded)) return false;
    if (encoded != e->bytes)
      return fail("tensor %s stores %llu bytes; layout requires %llu", e->name.c_str(), static_cast<unsigned long long>(e->bytes),
                  static_cast<unsigned long long>(encoded)),
             false;
    return true;
  }
  if (kind->string == "resource") {
    if (!require_members(value, {"name", "kind", "encoding", "offset", "bytes"}, "resource entry")) return false;
    e->kind = B200Q_ARTIFACT_RESOURCE;
    if (!require_string(*value.get("name"), "resource name", &e->name)) return false;
    if (!require_string(*value.get("encoding"), "resource encoding", &text)) return false;
    if (text != "raw-bytes-v1") return fail("unknown resource encoding: %s", text.c_str()), false;
    e->layout = B200Q_LAYOUT_RAW_BYTES_V1;
    if (!require_unsigned(*value.get("offset"), "resource offset", false, &e->offset)) return false;
    return require_unsigned(*value.get("bytes"), "resource bytes", true, &e->bytes);
  }
  return fail("object kind must be 'tensor' or 'resource'"), false;
}

}  // namespace

struct b200q_artifact {
  int fd = -1;
  const uint8_t *map = nullptr;
  uint64_t file_bytes = 0, payload_start = 0;
  std::string model_id, weights_id;
  std::vector<Entry> objects;
  std::unordered_map<std::string, size_t> index;

  ~b200q_artifact() {
    if (map != nullptr) munmap(const_cast<uint8_t *>(map), file_bytes);
    if (fd >= 0) close(fd);
  }
};

namespace {

void describe(const b200q_artifact &a, const Entry &e, b200q_artifact_object *out) {
  memset(out, 0, sizeof(*out));
  out->name = e.name.c_str();
  out->kind = e.kind;
  out->format = e.format;
  out->layout = e.layout;
  out->rank = static_cast<uint32_t>(e.shape.size());
  for (size_t i = 0; i < e.shape.size(); ++i) out->shape[i] = e.shape[i];
  out->offset = e.offset;
  out->bytes = e.bytes;
  out->file_offset = a.payload_start + e.offset;
  out->data = a.map + out->file_offset;
}

const Entry *lookup(const b200q_artifact *a, const char *name) {
  if (a == nullptr || name == nullptr) {
    fail("null artifact or name");
    return nullptr;
  }
  const auto it = a->index.find(name);
  if (it == a->index.end()) {
    fail("unknown artifact object: %s", name);
    return nullptr;
  }
  return &a->objects[it->second];
}

bool read_divisor(const b200q_artifact *a, const char *name, float *out) {
  const Entry *e = lookup(a, name);
  if (e == nullptr) return false;
  if (e->kind != B200Q_ARTIFACT_TENSOR || e->format != B200Q_FORMAT_FP32 || e->layout != B200Q_LAYOUT_CONTIGUOUS_LE_V1 ||
      !e->shape.empty())
    return fail("object %s is not a rank-0 FP32 scalar", name), false;
  memcpy(out, a->map + a->payload_start + e->offset, 4);  // little-endian host
  if (!std::isfinite(*out) || !(*out > 0.0f)) return fail("divisor %s is not finite and positive", name), false;
  return true;
}

bool ends_with(const std::string &s, const char *suffix) {
  const size_t n = strlen(suffix);
  return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

bool divisor_name(const std::string &parent, std::string *out) {
  static const char *const kSites[6][2] = {{"/gdn/query_key_value_z", "/gdn/input_projection"},
                                           {"/gdn/output", "/gdn/output_projection"},
                                           {"/attention/query_key_gate_value", "/attention/input_projection"},
                                           {"/attention/output", "/attention/output_projection"},
                                           {"/mlp/gate_up", "/mlp/gate_up_projection"},
                                           {"/mlp/down", "/mlp/down_projection"}};
  for (const auto &site : kSites) {
    if (ends_with(parent, site[0])) {
      *out = parent.substr(0, parent.size() - strlen(site[0])) + site[1] + "/input_scale_divisor";
      return true;
    }
  }
  return fail("%s is not one of the NVFP4 projections that carry an activation divisor", parent.c_str()), false;
}

}  // namespace

extern "C" {

const char *b200q_artifact_last_error(void) { return g_error; }

uint32_t b200q_artifact_format_by_name(const char *name) { return name ? format_by_name(name) : (fail("null name"), 0u); }

uint32_t b200q_artifact_layout_by_name(const char *name) {
  if (name == nullptr) return fail("null name"), 0u;
  if (strcmp(name, "raw-bytes-v1") == 0) return B200Q_LAYOUT_RAW_BYTES_V1;
  return layout_by_name(name);
}

const char *b200q_artifact_format_name(uint32_t format) { return format < kFormatCount ? kFormatNames[format] : nullptr; }
const char *b200q_artifact_layout_name(uint32_t layout) { return layout < kLayoutCount ? kLayoutNames[layout] : nullptr; }
uint32_t b200q_artifact_trellis_k2(uint32_t format) { return trellis_k2(format); }
uint64_t b200q_artifact_alignment(uint32_t layout) { return layout_alignment(layout); }

int32_t b200q_artifact_encoded_size(uint32_t layout, uint32_t format, const uint64_t *shape, uint32_t rank, uint64_t *bytes) {
  if (bytes == nullptr || (rank != 0 && shape == nullptr)) return fail("null argument");
  return encoded_size(layout, format, shape, rank, bytes) ? 0 : -1;
}

int32_t b200q_artifact_blockscale_geometry(uint32_t format, const uint64_t *shape, uint32_t rank, b200q_blockscale_geometry *out) {
  if (out == nullptr || (rank != 0 && shape == nullptr)) return fail("null argument");
  return blockscale_geometry(format, shape, rank, out) ? 0 : -1;
}

int32_t b200q_artifact_trellis_geometry(uint32_t format, const uint64_t *shape, uint32_t rank, b200q_trellis_geometry *out) {
  if (out == nullptr || (rank != 0 && shape == nullptr)) return fail("null argument");
  return trellis_geometry(format, shape, rank, out) ? 0 : -1;
}

int32_t b200q_artifact_open(const char *path, b200q_artifact **out) {
  if (path == nullptr || out == nullptr) return fail("null argument");
  *out = nullptr;
  std::unique_ptr<b200q_artifact> a(new b200q_artifact);
  a->fd = open(path, O_RDONLY | O_CLOEXEC);
  if (a->fd < 0) return fail("open %s: %s", path, strerror(errno));
  struct stat st;
  if (fstat(a->fd, &st) != 0) return fail("stat %s: %s", path, strerror(errno));
  a->file_bytes = static_cast<uint64_t>(st.st_size);
  if (a->file_bytes < kPrefixBytes) return fail("artifact is shorter than the v2 prefix");
  void *map = mmap(nullptr, a->file_bytes, PROT_READ, MAP_PRIVATE, a->fd, 0);
  if (map == MAP_FAILED) return fail("mmap %s: %s", path, strerror(errno));
  a->map = static_cast<const uint8_t *>(map);

  if (memcmp(a->map, kV1Magic, 8) == 0)
    return fail("NInfer artifact v1 is no longer supported; migrate it with: python3 -m tools.artifact.migrate_v1_to_v2 <artifact>");
  if (memcmp(a->map, kMagic, 8) != 0) return fail("artifact magic is not NInfer v2");
  uint64_t json_bytes = 0;
  for (int i = 0; i < 8; ++i) json_bytes |= static_cast<uint64_t>(a->map[8 + i]) << (8 * i);
  if (json_bytes == 0) return fail("json_bytes must be positive");
  uint64_t metadata_end;
  if (!checked_add(kPrefixBytes, json_bytes, "JSON range", &metadata_end) ||
      !align_up(metadata_end, kPayloadAlignment, "payload offset", &a->payload_start))
    return -1;
  if (metadata_end > a->file_bytes || a->payload_start > a->file_bytes)
    return fail("declared JSON or payload start extends beyond the file");

  Json directory;
  JsonParser parser(reinterpret_cast<const char *>(a->map) + kPrefixBytes, reinterpret_cast<const char *>(a->map) + metadata_end);
  if (!parser.parse(&directory)) return fail("invalid JSON directory: %s", parser.message().c_str());
  if (!require_members(directory, {"identity", "objects"}, "directory root")) return -1;
  const Json &identity = *directory.get("identity");
  if (!require_members(identity, {"model_id", "weights_id"}, "artifact identity")) return -1;
  if (!require_string(*identity.get("model_id"), "model_id", &a->model_id) ||
      !require_string(*identity.get("weights_id"), "weights_id", &a->weights_id))
    return -1;
  const Json &objects = *directory.get("objects");
  if (objects.type != Json::kArray || objects.items.empty()) return fail("objects must be a nonempty array");

  const uint64_t payload_bytes = a->file_bytes - a->payload_start;
  uint64_t cursor = 0;
  a->objects.reserve(objects.items.size());
  for (const Json &raw : objects.items) {
    Entry e;
    if (!parse_object(raw, &e)) return -1;
    const uint64_t alignment = layout_alignment(e.layout);
    if (e.offset < cursor) return fail("object %s overlaps or is out of order", e.name.c_str());
    if (e.offset % alignment != 0)
      return fail("object %s is not %llu-byte aligned", e.name.c_str(), static_cast<unsigned long long>(alignment));
    uint64_t end;
    if (!checked_add(e.offset, e.bytes, "object payload range", &end)) return -1;
    if (end > payload_bytes) return fail("object %s extends beyond the file", e.name.c_str());
    if (!a->index.emplace(e.name, a->objects.size()).second) return fail("duplicate object name: %s", e.name.c_str());
    a->objects.push_back(std::move(e));
    cursor = end;
  }
  *out = a.release();
  return 0;
}

void b200q_artifact_close(b200q_artifact *artifact) { delete artifact; }

const char *b200q_artifact_model_id(const b200q_artifact *a) { return a ? a->model_id.c_str() : nullptr; }
const char *b200q_artifact_weights_id(const b200q_artifact *a) { return a ? a->weights_id.c_str() : nullptr; }
uint64_t b200q_artifact_object_count(const b200q_artifact *a) { return a ? a->objects.size() : 0; }
uint64_t b200q_artifact_payload_offset(const b200q_artifact *a) { return a ? a->payload_start : 0; }
uint64_t b200q_artifact_file_bytes(const b200q_artifact *a) { return a ? a->file_bytes : 0; }

int32_t b200q_artifact_object_at(const b200q_artifact *a, uint64_t index, b200q_artifact_object *out) {
  if (a == nullptr || out == nullptr) return fail("null argument");
  if (index >= a->objects.size())
    return fail("object index %llu is outside the directory of %zu objects", static_cast<unsigned long long>(index), a->objects.size());
  describe(*a, a->objects[index], out);
  return 0;
}

int32_t b200q_artifact_find(const b200q_artifact *a, const char *name, b200q_artifact_object *out) {
  if (out == nullptr) return fail("null argument");
  const Entry *e = lookup(a, name);
  if (e == nullptr) return -1;
  describe(*a, *e, out);
  return 0;
}

int32_t b200q_artifact_content_hash(const b200q_artifact *a, uint8_t digest[32]) {
  if (a == nullptr || digest == nullptr) return fail("null argument");
  Sha256 h;
  h.update_str0("ignis-artifact-directory-v1");  // the domain tag, with its terminating zero
  h.update_str0(a->model_id.c_str());
  h.update_str0(a->weights_id.c_str());
  h.update_u64(a->file_bytes);
  h.update_u64(a->payload_start);
  h.update_u64(a->objects.size());
  for (const Entry &e : a->objects) {
    h.update_str0(e.name.c_str());
    h.update_str0(e.kind == B200Q_ARTIFACT_TENSOR ? "tensor" : "resource");
    h.update_u64(e.offset);
    h.update_u64(e.bytes);
    if (e.kind == B200Q_ARTIFACT_TENSOR) {
      h.update_str0(kFormatNames[e.format]);
      h.update_str0(kLayoutNames[e.layout]);
      h.update_u64(e.shape.size());
      for (uint64_t d : e.shape) h.update_u64(d);
    } else {
      h.update_str0(kLayoutNames[e.layout]);
    }
  }
  h.finish(digest);
  return 0;
}

int32_t b200q_artifact_divisor_name(const char *parent, char *out, uint64_t capacity) {
  if (parent == nullptr || out == nullptr) return fail("null argument");
  std::string name;
  if (!divisor_name(parent, &name)) return -1;
  if (name.size() + 1 > capacity) return fail("the divisor name needs %zu bytes", name.size() + 1);
  memcpy(out, name.c_str(), name.size() + 1);
  return 0;
}

int32_t b200q_artifact_nvfp4_weight(const b200q_artifact *a, const char *name, const char *divisor, const void *payload,
                                    b200q_nvfp4_weight *out) {
  if (out == nullptr) return fail("null argument");
  const Entry *e = lookup(a, name);
  if (e == nullptr) return -1;
  if (e->kind != B200Q_ARTIFACT_TENSOR || e->format != B200Q_FORMAT_NVFP4 || e->layout != B200Q_LAYOUT_BLOCKSCALE_K16_M128X4_V1)
    return fail("object %s is not an NVFP4 block-scale tensor", name);
  if (e->shape.size() != 2) return fail("object %s is not rank-two", name);
  b200q_blockscale_geometry g;
  if (!blockscale_geometry(e->format, e->shape.data(), 2, &g)) return -1;
  if (g.rows > UINT32_MAX || g.columns > UINT32_MAX) return fail("object %s is wider than the kernels' 32-bit extents", name);
  const uint8_t *host = a->map + a->payload_start + e->offset;
  const uint8_t *base = payload != nullptr ? static_cast<const uint8_t *>(payload) : host;
  if (payload != nullptr && reinterpret_cast<uintptr_t>(payload) % kTensorAlignment != 0)
    return fail("the payload copy of %s is not 256-byte aligned", name);
  float weight_divisor, input_divisor = 1.0f;
  memcpy(&weight_divisor, host + g.weight_divisor_offset, 4);
  if (!std::isfinite(weight_divisor) || !(weight_divisor > 0.0f)) return fail("the weight divisor of %s is not finite and positive", name);
  if (divisor == nullptr) {
    std::string derived;
    if (!divisor_name(name, &derived) || !read_divisor(a, derived.c_str(), &input_divisor)) return -1;
  } else if (divisor[0] != '\0') {
    if (!read_divisor(a, divisor, &input_divisor)) return -1;
  }
  out->codes = base;
  out->scales = base + g.scale_plane_offset;
  out->n = static_cast<uint32_t>(g.rows);
  out->k = static_cast<uint32_t>(g.columns);
  out->weight_scale_divisor = weight_divisor;
  out->input_scale_divisor = input_divisor;
  return 0;
}

int32_t b200q_artifact_trellis_weight(const b200q_artifact *a, const char *name, const void *payload, ignis_trellis_weight *out) {
  if (out == nullptr) return fail("null argument");
  const Entry *e = lookup(a, name);
  if (e == nullptr) return -1;
  if (e->kind != B200Q_ARTIFACT_TENSOR || e->layout != B200Q_LAYOUT_TRELLIS_TILE16_V1 || trellis_k2(e->format) == 0)
    return fail("object %s is not a trellis tensor", name);
  b200q_trellis_geometry g;
  if (!trellis_geometry(e->format, e->shape.data(), static_cast<uint32_t>(e->shape.size()), &g)) return -1;
  if (g.rows > UINT32_MAX || g.columns > UINT32_MAX) return fail("object %s is wider than the kernels' 32-bit extents", name);
  if (payload != nullptr && reinterpret_cast<uintptr_t>(payload) % kTensorAlignment != 0)
    return fail("the payload copy of %s is not 256-byte aligned", name);
  const uint8_t *base = payload != nullptr ? static_cast<const uint8_t *>(payload) : a->map + a->payload_start + e->offset;
  out->trellis = base;
  out->suh = base + g.suh_offset;
  out->svh = base + g.svh_offset;
  out->k2 = static_cast<uint32_t>(g.k2);
  out->in = static_cast<uint32_t>(g.columns);
  out->out = static_cast<uint32_t>(g.rows);
  out->tile_stride = 0;
  return 0;
}

}  // extern "C"
