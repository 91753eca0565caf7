// Entry points of include/b200q_nvfp4.h: argument checks, route choice and launches.
#include "../../include/b200q_nvfp4.h"

#include "nvfp4_internal.cuh"

#include <cmath>

namespace b200q {
namespace {

bool aligned(const void *p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// A16_ONLY or ALLOW_A4 in the low byte, optionally one B200Q_NVFP4_PROBLEM_* class above it.
bool policy_ok(uint32_t policy) {
  return (policy & ~(0xFFu | B200Q_NVFP4_PROBLEM_MASK)) == 0u && (policy & 0xFFu) <= B200Q_NVFP4_ALLOW_A4 &&
         (policy & B200Q_NVFP4_PROBLEM_MASK) <= B200Q_NVFP4_PROBLEM_RESIDUAL;
}

int32_t check_weight(ErrorSlot &slot, const b200q_nvfp4_weight *w, const char *what) {
  if (w == nullptr) return fail(slot, "%s: weight is NULL", what);
  if (w->codes == nullptr || w->scales == nullptr) return fail(slot, "%s: weight planes are NULL", what);
  if (w->n == 0 || (w->n % 128u) != 0) return fail(slot, "%s: n = %u is not a positive multiple of 128", what, w->n);
  if (w->k == 0 || (w->k % 64u) != 0) return fail(slot, "%s: k = %u is not a positive multiple of 64", what, w->k);
  if (!aligned(w->codes, 32)) return fail(slot, "%s: the code plane is not 32-byte aligned", what);
  if (!aligned(w->scales, 16)) return fail(slot, "%s: the scale plane is not 16-byte aligned", what);
  if (!std::isfinite(w->weight_scale_divisor) || !(w->weight_scale_divisor > 0.0f)) {
    return fail(slot, "%s: weight_scale_divisor must be finite and positive", what);
  }
  return 0;
}

const DeviceState *prepared_state(ErrorSlot &slot, const char *what) {
  const DeviceState *dev = device_state(slot);
  if (dev == nullptr) return nullptr;
  if (!dev->prepared) {
    fail(slot, "%s: the device was not prepared (call b200q_nvfp4_prepare at load)", what);
    return nullptr;
  }
  return dev;
}

// The decode route over `count` weights that share x, in passes of at most 32 tokens.
// `y` holds `peers` pointers per weight (weight i's at y[i * peers ..]); a plain product has one.
PeerSync make_sync(const DeviceState &dev, const b200q_peer_sync *s) {
  PeerSync out = {};
  if (s != nullptr) {
    out.flags_peers = s->flags_peers;
    out.state = s->state;
    out.peers = s->peers;
    out.rank = s->rank;
    out.polls = static_cast<uint32_t>(dev.peer_barrier_polls);
  }
  return out;
}

int32_t decode_route(ErrorSlot &slot, const DeviceState &dev, const b200q_nvfp4_weight *const *w, uint32_t count,
                     const void *x, uint32_t tokens, void *const *y, const uint32_t *ldy, uint32_t epilogue,
                     cudaStream_t stream, uint32_t peers = 1, const b200q_peer_sync *wait_for = nullptr) {
  const uint32_t k = w[0]->k;
  const bool swiglu = (epilogue & kEpilogueSwiglu) != 0u;
  const size_t out_elem = (epilogue & kEpilogueF32) ? 4u : 2u;
  uint32_t groups = 0;
  for (uint32_t i = 0; i < count; ++i) groups += w[i]->n / 32u;
  if (dev.a16_mma != 0 && tokens > 16u && !swiglu && peers == 1u && wait_for == nullptr && a16mma_takes(k, x)) {
    // beyond two token tiles the warp-level MMAs of the decode kernel are the limit: the weights
    // are decoded once per tile of up to 256 tokens and multiplied on the tensor cores
    {
      const uint32_t t0 = 0, pass = tokens;
      GemvWeight gw[kMaxGroup];
      for (uint32_t i = 0; i < count; ++i) {
        gw[i].codes = static_cast<const uint8_t *>(w[i]->codes);
        gw[i].scales = static_cast<const uint8_t *>(w[i]->scales);
        gw[i].y[0] = static_cast<uint8_t *>(y[i]) + static_cast<size_t>(t0) * ldy[i] * out_elem;
        gw[i].peers = 1;
        gw[i].n = w[i]->n;
        gw[i].ldy = ldy[i];
        gw[i].inv_dw = 1.0f / w[i]->weight_scale_divisor;
        gw[i].block_begin = 0;
      }
      if (a16mma_launch(slot, dev, gw, count, static_cast<const uint16_t *>(x) + static_cast<size_t>(t0) * k, k, pass, epilogue,
                        stream) != 0) {
        return -1;
      }
    }
    return 0;
  }
  for (uint32_t t0 = 0; t0 < tokens; t0 += B200Q_NVFP4_DECODE_MAX_TOKENS) {
    const uint32_t pass = tokens - t0 < B200Q_NVFP4_DECODE_MAX_TOKENS ? tokens - t0 : B200Q_NVFP4_DECODE_MAX_TOKENS;
    const int nt = pass <= 8 ? 1 : (pass <= 16 ? 2 : 4);
    GemvParams p = {};
    p.x = static_cast<const uint16_t *>(x) + static_cast<size_t>(t0) * k;
    p.count = count;
    p.k = k;
    p.ksteps = (k + 255u) / 256u;
    p.tokens = pass;
    p.epilogue = epilogue;
    if (t0 == 0) p.wait = make_sync(dev, wait_for);   // a call of several passes waits before its first
    const GemvPlan plan = gemv_plan(dev, groups, p.ksteps, nt, swiglu);
    const uint32_t rows_per_cta = static_cast<uint32_t>(swiglu ? plan.rm / 2 : plan.rm);
    uint32_t ctas = 0;
    for (uint32_t i = 0; i < count; ++i) {
      GemvWeight &g = p.w[i];
      g.codes = static_cast<const uint8_t *>(w[i]->codes);
      g.scales = static_cast<const uint8_t *>(w[i]->scales);
      for (uint32_t pp = 0; pp < peers; ++pp) {
        g.y[pp] = static_cast<uint8_t *>(y[i * peers + pp]) + static_cast<size_t>(t0) * ldy[i] * out_elem;
      }
      g.peers = peers;
      g.n = w[i]->n;
      g.ldy = ldy[i];
      g.inv_dw = 1.0f / w[i]->weight_scale_divisor;
      g.block_begin = ctas;
      const uint32_t out_groups = swiglu ? w[i]->n / 64u : w[i]->n / 32u;
      ctas += (out_groups + rows_per_cta - 1) / rows_per_cta * static_cast<uint32_t>(plan.kc);
    }
    if (gemv_launch(slot, dev, p, nt, plan, ctas, stream) != 0) return -1;
  }
  return 0;
}

// Tokens from which the reference's AllowA4 policy quantizes the activations, by problem
// (nvfp4_dispatch.cpp:31-39): its fused GDN input always, attention inputs from 4 tokens, gate|up
// from 5, the projections back to the residual stream from 8. The reference resolves this by the
// problem the weight was registered as; a caller says which problem a call is with the
// B200Q_NVFP4_PROBLEM_* bits of `policy`. Without them the problem is told from the shape's
// proportions (so other model sizes of the same family resolve alike), and one literal shape for
// the GDN input whose proportions equal an attention input's.
uint32_t a4_min_tokens(uint32_t policy, uint32_t n_total, uint32_t k) {
  switch (policy & B200Q_NVFP4_PROBLEM_MASK) {
    case B200Q_NVFP4_PROBLEM_GDN_INPUT: return 1;
    case B200Q_NVFP4_PROBLEM_ATTN_INPUT: return 4;
    case B200Q_NVFP4_PROBLEM_GATE_UP: return 5;
    case B200Q_NVFP4_PROBLEM_RESIDUAL: return 8;
    default: break;
  }
  if (n_total < k) return 8;
  if (n_total >= 4u * k) return 5;
  if (n_total == 16384u && k == 5120u) return 1;
  return 4;
}

// Calls of up to 32 tokens. B200Q_NVFP4_ALLOW_A4 from the reference's per-problem thresholds: the
// activations are quantized inside the W4A4 decode kernel (no workspace). Everything else: the A16
// routes.
int32_t narrow_route(ErrorSlot &slot, const DeviceState &dev, const b200q_nvfp4_weight *const *w, uint32_t count, const void *x,
                     uint32_t tokens, void *const *y, const uint32_t *ldy, uint32_t epilogue, uint32_t policy,
                     cudaStream_t stream) {
  if ((policy & 0xFFu) == B200Q_NVFP4_ALLOW_A4 && dev.a4_decode != 0 && tokens <= kA4DecodeMaxTokens) {
    uint32_t n_total = 0;
    bool takes = true;
    for (uint32_t i = 0; i < count; ++i) {
      n_total += w[i]->n;
      takes = takes && w4a4_decode_takes(w[i]->n, w[i]->k, tokens, epilogue) && std::isfinite(w[i]->input_scale_divisor) &&
              w[i]->input_scale_divisor > 0.0f;
    }
    if (takes && tokens >= a4_min_tokens(policy, n_total, w[0]->k)) {
      A4Item items[kMaxGroup];
      for (uint32_t i = 0; i < count; ++i) {
        items[i] = A4Item{static_cast<const uint8_t *>(w[i]->codes), static_cast<const uint8_t *>(w[i]->scales), y[i], w[i]->n, ldy[i],
                          w[i]->weight_scale_divisor, w[i]->input_scale_divisor};
      }
      return w4a4_decode_launch(slot, dev, items, count, static_cast<const uint16_t *>(x), w[0]->k, tokens, epilogue, stream);
    }
  }
  return decode_route(slot, dev, w, count, x, tokens, y, ldy, epilogue, stream);
}

int32_t linear_group_impl(const b200q_nvfp4_weight *const *w, uint32_t count, const void *x, uint32_t tokens,
                          void *const *y, const uint32_t *ldy, uint32_t epilogue, uint32_t policy,
                          const b200q_nvfp4_workspace *workspace, void *stream, const char *what) {
  ErrorSlot &slot = nvfp4_error();
  if (w == nullptr || y == nullptr || ldy == nullptr) return fail(slot, "%s: NULL argument array", what);
  if (count == 0 || count > B200Q_NVFP4_MAX_GROUP) return fail(slot, "%s: count = %u is outside 1..%d", what, count, B200Q_NVFP4_MAX_GROUP);
  if (tokens == 0) return fail(slot, "%s: tokens must be positive", what);
  if (!policy_ok(policy)) return fail(slot, "%s: unknown policy 0x%x", what, policy);
  if ((epilogue & ~(kEpilogueAdd | kEpilogueF32 | kEpilogueSwiglu)) != 0u) return fail(slot, "%s: unknown epilogue 0x%x", what, epilogue);
  if (x == nullptr || !aligned(x, 16)) return fail(slot, "%s: x is NULL or not 16-byte aligned", what);
  const bool swiglu = (epilogue & kEpilogueSwiglu) != 0u;
  for (uint32_t i = 0; i < count; ++i) {
    if (check_weight(slot, w[i], what) != 0) return -1;
    if (w[i]->k != w[0]->k) return fail(slot, "%s: the weights of a group must share k", what);
    if (y[i] == nullptr) return fail(slot, "%s: output %u is NULL", what, i);
    const uint32_t width = swiglu ? w[i]->n / 2u : w[i]->n;
    if (ldy[i] < width) return fail(slot, "%s: ldy[%u] = %u is narrower than the output (%u)", what, i, ldy[i], width);
    if (swiglu && (w[i]->n % 256u) != 0) return fail(slot, "%s: a fused gate_up parent needs n a multiple of 256", what);
  }
  const DeviceState *dev = prepared_state(slot, what);
  if (dev == nullptr) return -1;
  // Wide calls under B200Q_NVFP4_ALLOW_A4 quantize the activations into the workspace and take the
  // prefill kernels; everything else takes the A16 routes.
  if ((policy & 0xFFu) == B200Q_NVFP4_ALLOW_A4 && tokens > B200Q_NVFP4_DECODE_MAX_TOKENS && count == 1 &&
      !(swiglu && (epilogue & kEpilogueAdd)) && w4a4_shape_ok(w[0]->n, w[0]->k)) {
    const b200q_nvfp4_weight *w0 = w[0];
    if (!std::isfinite(w0->input_scale_divisor) || !(w0->input_scale_divisor > 0.0f)) {
      return fail(slot, "%s: input_scale_divisor must be finite and positive for the A4 route", what);
    }
    const uint64_t need = w4a4_workspace_bytes(w0->k, tokens);
    if (workspace == nullptr || workspace->base == nullptr || workspace->bytes < need || !aligned(workspace->base, 256)) {
      return fail(slot, "%s: the A4 route needs a 256-byte aligned workspace of %llu bytes", what,
                  static_cast<unsigned long long>(need));
    }
    if (!aligned(y[0], 16) || (ldy[0] % 8u) != 0) return fail(slot, "%s: the A4 route needs y 16-byte aligned and ldy a multiple of 8", what);
    return w4a4_launch(slot, *dev, static_cast<const uint8_t *>(w0->codes), static_cast<const uint8_t *>(w0->scales), w0->n,
                       w0->k, w0->weight_scale_divisor, w0->input_scale_divisor, static_cast<const uint16_t *>(x), tokens,
                       y[0], ldy[0], epilogue, static_cast<uint8_t *>(workspace->base), static_cast<cudaStream_t>(stream));
  }
  return narrow_route(slot, *dev, w, count, x, tokens, y, ldy, epilogue, policy, static_cast<cudaStream_t>(stream));
}

}  // namespace
}  // namespace b200q

using namespace b200q;

namespace b200q {
int32_t prepare_nvfp4_kernels(ErrorSlot &slot) {
  if (gemv_prepare(slot) != 0) return -1;
  if (a16mma_prepare(slot) != 0) return -1;
  if (w4a4_decode_prepare(slot) != 0) return -1;
  return w4a4_prepare(slot);
}
}  // namespace b200q

extern "C" {

int32_t b200q_nvfp4_prepare(void) { return prepare_all(nvfp4_error()); }

uint64_t b200q_nvfp4_workspace_bytes(uint32_t n, uint32_t k, uint32_t policy, uint32_t tokens) {
  if (n == 0 || (n % 128u) != 0 || k == 0 || (k % 64u) != 0 || tokens == 0) return 0;
  if (!policy_ok(policy)) return 0;
  // The decode route keeps its partial sums in distributed shared memory and needs no global
  // scratch (one aligned line, so a workspace pointer is never NULL); the A4 route keeps the
  // quantized activations there.
  if ((policy & 0xFFu) == B200Q_NVFP4_ALLOW_A4 && tokens > B200Q_NVFP4_DECODE_MAX_TOKENS && w4a4_shape_ok(n, k)) {
    return w4a4_workspace_bytes(k, tokens);
  }
  return 256;
}

int32_t b200q_nvfp4_workspace_init(const b200q_nvfp4_workspace *workspace, void *stream) {
  ErrorSlot &slot = nvfp4_error();
  if (workspace == nullptr || workspace->base == nullptr || workspace->bytes < 256) {
    return fail(slot, "b200q_nvfp4_workspace_init: workspace is NULL or shorter than 256 bytes");
  }
  if (!aligned(workspace->base, 256)) return fail(slot, "b200q_nvfp4_workspace_init: base is not 256-byte aligned");
  const cudaError_t err = cudaMemsetAsync(workspace->base, 0, 256, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(slot, "b200q_nvfp4_workspace_init: %s", cudaGetErrorString(err));
  return 0;
}

int32_t b200q_nvfp4_workspace_status(const b200q_nvfp4_workspace *workspace, void *stream, uint32_t *status) {
  ErrorSlot &slot = nvfp4_error();
  if (workspace == nullptr || workspace->base == nullptr || status == nullptr) {
    return fail(slot, "b200q_nvfp4_workspace_status: NULL argument");
  }
  cudaError_t err = cudaMemcpyAsync(status, workspace->base, sizeof(uint32_t), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (err == cudaSuccess) err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(slot, "b200q_nvfp4_workspace_status: %s", cudaGetErrorString(err));
  return 0;
}

int32_t b200q_nvfp4_linear(const b200q_nvfp4_weight *w, const void *x, uint32_t tokens, void *y, uint32_t ldy,
                           uint32_t epilogue, uint32_t policy, const b200q_nvfp4_workspace *workspace, void *stream) {
  if ((epilogue & ~(B200Q_NVFP4_ADD | B200Q_NVFP4_OUT_F32)) != 0u) {
    return fail(nvfp4_error(), "b200q_nvfp4_linear: unknown epilogue 0x%x", epilogue);
  }
  const b200q_nvfp4_weight *ws[1] = {w};
  void *ys[1] = {y};
  const uint32_t lds[1] = {ldy};
  return linear_group_impl(ws, 1, x, tokens, ys, lds, epilogue, policy, workspace, stream, "b200q_nvfp4_linear");
}

int32_t b200q_nvfp4_linear_group(const b200q_nvfp4_weight *const *w, uint32_t count, const void *x, uint32_t tokens,
                                 void *const *y, const uint32_t *ldy, uint32_t epilogue, uint32_t policy,
                                 const b200q_nvfp4_workspace *workspace, void *stream) {
  if ((epilogue & ~(B200Q_NVFP4_ADD | B200Q_NVFP4_OUT_F32)) != 0u) {
    return fail(nvfp4_error(), "b200q_nvfp4_linear_group: unknown epilogue 0x%x", epilogue);
  }
  return linear_group_impl(w, count, x, tokens, y, ldy, epilogue, policy, workspace, stream, "b200q_nvfp4_linear_group");
}

int32_t b200q_nvfp4_device_status(void *stream, uint32_t *status) {
  ErrorSlot &slot = nvfp4_error();
  if (status == nullptr) return fail(slot, "b200q_nvfp4_device_status: status is NULL");
  uint32_t a16 = 0, a4 = 0, noalloc = 0;
  if (a16mma_status(slot, static_cast<cudaStream_t>(stream), &a16) != 0) return -1;
  if (w4a4_decode_status(slot, static_cast<cudaStream_t>(stream), &a4) != 0) return -1;
  if (w4a4_noalloc_status(slot, static_cast<cudaStream_t>(stream), &noalloc) != 0) return -1;
  *status = a16 | a4 | noalloc;
  return 0;
}

int32_t b200q_nvfp4_linear_split(const b200q_nvfp4_weight *parent, uint32_t count, const uint32_t *row_begin, const uint32_t *rows,
                                 const void *x, uint32_t tokens, void *const *y, const uint32_t *ldy, uint32_t epilogue,
                                 uint32_t policy, const b200q_nvfp4_workspace *workspace, void *stream) {
  const char *what = "b200q_nvfp4_linear_split";
  ErrorSlot &slot = nvfp4_error();
  if (row_begin == nullptr || rows == nullptr || y == nullptr || ldy == nullptr) return fail(slot, "%s: NULL argument array", what);
  if (count == 0 || count > B200Q_NVFP4_MAX_GROUP) return fail(slot, "%s: count = %u is outside 1..%d", what, count, B200Q_NVFP4_MAX_GROUP);
  if ((epilogue & ~static_cast<uint32_t>(B200Q_NVFP4_OUT_F32)) != 0u) return fail(slot, "%s: only STORE (optionally OUT_F32) is served", what);
  if (check_weight(slot, parent, what) != 0) return -1;
  // every range as a weight of its own: whole 128-row tiles are contiguous in both planes
  b200q_nvfp4_weight part[B200Q_NVFP4_MAX_GROUP];
  const b200q_nvfp4_weight *parts[B200Q_NVFP4_MAX_GROUP];
  const uint64_t row_bytes = parent->k / 2u, tile_bytes = static_cast<uint64_t>(parent->k / 64u) * 512u;
  for (uint32_t i = 0; i < count; ++i) {
    if (rows[i] == 0 || (rows[i] % 128u) != 0 || (row_begin[i] % 128u) != 0 ||
        static_cast<uint64_t>(row_begin[i]) + rows[i] > parent->n) {
      return fail(slot, "%s: range %u = [%u, +%u) is not whole 128-row tiles inside the parent's %u rows", what, i, row_begin[i],
                  rows[i], parent->n);
    }
    part[i] = *parent;
    part[i].codes = static_cast<const uint8_t *>(parent->codes) + row_begin[i] * row_bytes;
    part[i].scales = static_cast<const uint8_t *>(parent->scales) + (row_begin[i] / 128u) * tile_bytes;
    part[i].n = rows[i];
    parts[i] = &part[i];
  }
  const bool wide = (policy & 0xFFu) == B200Q_NVFP4_ALLOW_A4 && tokens > B200Q_NVFP4_DECODE_MAX_TOKENS && w4a4_shape_ok(parent->n, parent->k);
  if (!wide || count == 1) {
    return linear_group_impl(parts, count, x, tokens, y, ldy, epilogue, policy, workspace, stream, what);
  }
  // wide: one quantization of x, then a tensor-core product per range over the same operand
  if (tokens == 0) return fail(slot, "%s: tokens must be positive", what);
  if (x == nullptr || !aligned(x, 16)) return fail(slot, "%s: x is NULL or not 16-byte aligned", what);
  if (!std::isfinite(parent->input_scale_divisor) || !(parent->input_scale_divisor > 0.0f)) {
    return fail(slot, "%s: input_scale_divisor must be finite and positive for the A4 route", what);
  }
  const uint64_t need = w4a4_workspace_bytes(parent->k, tokens);
  if (workspace == nullptr || workspace->base == nullptr || workspace->bytes < need || !aligned(workspace->base, 256)) {
    return fail(slot, "%s: the A4 route needs a 256-byte aligned workspace of %llu bytes", what, static_cast<unsigned long long>(need));
  }
  const DeviceState *dev = prepared_state(slot, what);
  if (dev == nullptr) return -1;
  for (uint32_t i = 0; i < count; ++i) {
    if (y[i] == nullptr || !aligned(y[i], 16) || (ldy[i] % 8u) != 0 || ldy[i] < rows[i]) {
      return fail(slot, "%s: output %u must be 16-byte aligned with ldy a multiple of 8 and at least its rows", what, i);
    }
  }
  uint8_t *base = static_cast<uint8_t *>(workspace->base);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (uint32_t i = 0; i < count; ++i) {
    const b200q_nvfp4_weight &w = part[i];
    const int32_t rc = i == 0 ? w4a4_launch(slot, *dev, static_cast<const uint8_t *>(w.codes), static_cast<const uint8_t *>(w.scales), w.n, w.k,
                                            w.weight_scale_divisor, w.input_scale_divisor, static_cast<const uint16_t *>(x), tokens,
                                            y[i], ldy[i], epilogue, base, s)
                              : w4a4_launch_prequantized(slot, *dev, static_cast<const uint8_t *>(w.codes),
                                                         static_cast<const uint8_t *>(w.scales), w.n, w.k, w.weight_scale_divisor,
                                                         w.input_scale_divisor, tokens, y[i], ldy[i], epilogue, base, s);
    if (rc != 0) return -1;
  }
  return 0;
}

namespace {
int32_t check_sync(ErrorSlot &slot, const b200q_peer_sync *s, const char *what, const char *which) {
  if (s == nullptr) return 0;
  if (s->flags_peers == nullptr || s->state == nullptr) return fail(slot, "%s: %s has a NULL pointer", what, which);
  if (s->peers == 0 || s->peers > kMaxPeers || s->rank >= s->peers) {
    return fail(slot, "%s: %s has peers = %u, rank = %u out of range", what, which, s->peers, s->rank);
  }
  return 0;
}

int32_t scatter_impl(const b200q_nvfp4_weight *const *w, uint32_t count, const void *x, uint32_t tokens, void *const *y_peers,
                     uint32_t peers, const uint32_t *ldy, const uint32_t *col_offset, uint32_t epilogue,
                     const b200q_peer_sync *wait_for, void *stream, const char *what) {
  ErrorSlot &slot = nvfp4_error();
  if (w == nullptr || y_peers == nullptr || ldy == nullptr || col_offset == nullptr) return fail(slot, "%s: NULL argument array", what);
  if (count == 0 || count > B200Q_NVFP4_MAX_GROUP) return fail(slot, "%s: count = %u is outside 1..%d", what, count, B200Q_NVFP4_MAX_GROUP);
  if (peers == 0 || peers > kMaxPeers) return fail(slot, "%s: peers = %u is outside 1..%u", what, peers, kMaxPeers);
  if (tokens == 0) return fail(slot, "%s: tokens must be positive", what);
  if ((epilogue & ~static_cast<uint32_t>(B200Q_NVFP4_OUT_F32)) != 0u) return fail(slot, "%s: only STORE (optionally OUT_F32) is served", what);
  if (x == nullptr || !aligned(x, 16)) return fail(slot, "%s: x is NULL or not 16-byte aligned", what);
  if (check_sync(slot, wait_for, what, "rejoin") != 0) return -1;
  const size_t out_elem = (epilogue & kEpilogueF32) ? 4u : 2u;
  void *targets[B200Q_NVFP4_MAX_GROUP * kMaxPeers];
  for (uint32_t i = 0; i < count; ++i) {
    if (check_weight(slot, w[i], what) != 0) return -1;
    if (w[i]->k != w[0]->k) return fail(slot, "%s: the weights of a group must share k", what);
    if (ldy[i] < col_offset[i] + w[i]->n) return fail(slot, "%s: ldy[%u] = %u is narrower than col_offset + n", what, i, ldy[i]);
    for (uint32_t pp = 0; pp < peers; ++pp) {
      if (y_peers[i * peers + pp] == nullptr) return fail(slot, "%s: output %u of rank %u is NULL", what, i, pp);
      targets[i * peers + pp] = static_cast<uint8_t *>(y_peers[i * peers + pp]) + static_cast<size_t>(col_offset[i]) * out_elem;
    }
  }
  const DeviceState *dev = prepared_state(slot, what);
  if (dev == nullptr) return -1;
  return decode_route(slot, *dev, w, count, x, tokens, targets, ldy, epilogue, static_cast<cudaStream_t>(stream), peers, wait_for);
}
}  // namespace

int32_t b200q_nvfp4_linear_group_scatter(const b200q_nvfp4_weight *const *w, uint32_t count, const void *x, uint32_t tokens,
                                         void *const *y_peers, uint32_t peers, const uint32_t *ldy, const uint32_t *col_offset,
                                         uint32_t epilogue, void *stream) {
  return scatter_impl(w, count, x, tokens, y_peers, peers, ldy, col_offset, epilogue, nullptr, stream, "b200q_nvfp4_linear_group_scatter");
}

int32_t b200q_nvfp4_linear_group_gather(const b200q_nvfp4_weight *const *w, uint32_t count, const void *x, uint32_t tokens,
                                        void *const *y_peers, uint32_t peers, const uint32_t *ldy, const uint32_t *col_offset,
                                        uint32_t epilogue, const b200q_peer_sync *rejoin, void *stream) {
  return scatter_impl(w, count, x, tokens, y_peers, peers, ldy, col_offset, epilogue, rejoin, stream, "b200q_nvfp4_linear_group_gather");
}

uint64_t b200q_nvfp4_mlp_workspace_bytes(uint32_t gate_up_n, uint32_t k, uint32_t policy, uint32_t tokens) {
  if (gate_up_n == 0 || (gate_up_n % 256u) != 0 || k == 0 || (k % 64u) != 0 || tokens == 0) return 0;
  if (!policy_ok(policy)) return 0;
  const uint32_t inter = gate_up_n / 2u;
  if ((policy & 0xFFu) == B200Q_NVFP4_ALLOW_A4 && tokens > B200Q_NVFP4_DECODE_MAX_TOKENS && (k % 256u) == 0 && (inter % 256u) == 0) {
    return w4a4_mlp_workspace_bytes(k, inter, tokens);
  }
  return 256u + static_cast<uint64_t>(tokens) * inter * 2u;  // the status line, then h as BF16
}

int32_t b200q_nvfp4_mlp(const b200q_nvfp4_weight *gate_up, const b200q_nvfp4_weight *down, const void *x, uint32_t tokens, void *y,
                        uint32_t ldy, uint32_t epilogue, uint32_t policy, const b200q_nvfp4_workspace *workspace, void *stream) {
  const char *what = "b200q_nvfp4_mlp";
  ErrorSlot &slot = nvfp4_error();
  if ((epilogue & ~(B200Q_NVFP4_ADD | B200Q_NVFP4_OUT_F32)) != 0u) return fail(slot, "%s: unknown epilogue 0x%x", what, epilogue);
  if (!policy_ok(policy)) return fail(slot, "%s: unknown policy 0x%x", what, policy);
  if (check_weight(slot, gate_up, what) != 0 || check_weight(slot, down, what) != 0) return -1;
  if ((gate_up->n % 256u) != 0) return fail(slot, "%s: a fused gate_up parent needs n a multiple of 256", what);
  const uint32_t inter = gate_up->n / 2u;
  if (down->k != inter) return fail(slot, "%s: down.k = %u is not gate_up.n / 2 = %u", what, down->k, inter);
  if (tokens == 0) return fail(slot, "%s: tokens must be positive", what);
  if (x == nullptr || !aligned(x, 16)) return fail(slot, "%s: x is NULL or not 16-byte aligned", what);
  if (y == nullptr || !aligned(y, 16) || (ldy % 8u) != 0 || ldy < down->n) {
    return fail(slot, "%s: y must be 16-byte aligned with ldy a multiple of 8 and at least down.n", what);
  }
  const uint64_t need = b200q_nvfp4_mlp_workspace_bytes(gate_up->n, gate_up->k, policy, tokens);
  if (workspace == nullptr || workspace->base == nullptr || workspace->bytes < need || !aligned(workspace->base, 256)) {
    return fail(slot, "%s: needs a 256-byte aligned workspace of %llu bytes", what, static_cast<unsigned long long>(need));
  }
  const DeviceState *dev = prepared_state(slot, what);
  if (dev == nullptr) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t *base = static_cast<uint8_t *>(workspace->base);
  if ((policy & 0xFFu) == B200Q_NVFP4_ALLOW_A4 && tokens > B200Q_NVFP4_DECODE_MAX_TOKENS && (gate_up->k % 256u) == 0 && (inter % 256u) == 0) {
    for (const b200q_nvfp4_weight *w : {gate_up, down}) {
      if (!std::isfinite(w->input_scale_divisor) || !(w->input_scale_divisor > 0.0f)) {
        return fail(slot, "%s: input_scale_divisor must be finite and positive for the A4 route", what);
      }
    }
    return w4a4_mlp_launch(slot, *dev, static_cast<const uint8_t *>(gate_up->codes), static_cast<const uint8_t *>(gate_up->scales),
                           gate_up->n, gate_up->k, gate_up->weight_scale_divisor, gate_up->input_scale_divisor,
                           static_cast<const uint8_t *>(down->codes), static_cast<const uint8_t *>(down->scales), down->n,
                           down->weight_scale_divisor, down->input_scale_divisor, static_cast<const uint16_t *>(x), tokens, y, ldy,
                           epilogue, base, s);
  }
  // narrow calls: two products, h (BF16) in the workspace behind the status line
  void *h = base + 256;
  const b200q_nvfp4_weight *w0[1] = {gate_up};
  void *y0[1] = {h};
  const uint32_t ld0[1] = {inter};
  if (narrow_route(slot, *dev, w0, 1, x, tokens, y0, ld0, kEpilogueSwiglu, policy, s) != 0) return -1;
  const b200q_nvfp4_weight *w1[1] = {down};
  void *y1[1] = {y};
  const uint32_t ld1[1] = {ldy};
  return narrow_route(slot, *dev, w1, 1, h, tokens, y1, ld1, epilogue, policy, s);
}

int32_t b200q_nvfp4_linear_swiglu(const b200q_nvfp4_weight *gate_up, const void *x, uint32_t tokens, void *h, uint32_t ldh,
                                  uint32_t policy, const b200q_nvfp4_workspace *workspace, void *stream) {
  const b200q_nvfp4_weight *ws[1] = {gate_up};
  void *ys[1] = {h};
  const uint32_t lds[1] = {ldh};
  return linear_group_impl(ws, 1, x, tokens, ys, lds, kEpilogueSwiglu, policy, workspace, stream, "b200q_nvfp4_linear_swiglu");
}

int32_t b200q_nvfp4_dequantize(const b200q_nvfp4_weight *w, float *out, void *stream) {
  ErrorSlot &slot = nvfp4_error();
  if (check_weight(slot, w, "b200q_nvfp4_dequantize") != 0) return -1;
  if (out == nullptr || !aligned(out, 16)) return fail(slot, "b200q_nvfp4_dequantize: out is NULL or not 16-byte aligned");
  if (prepared_state(slot, "b200q_nvfp4_dequantize") == nullptr) return -1;
  return dequantize_launch(slot, static_cast<const uint8_t *>(w->codes), static_cast<const uint8_t *>(w->scales), w->n, w->k,
                           w->weight_scale_divisor, out, static_cast<cudaStream_t>(stream));
}

int32_t b200q_nvfp4_quantize_activations(const void *x, uint32_t tokens, uint32_t k, float input_scale_divisor, void *codes,
                                         void *scales, void *stream) {
  ErrorSlot &slot = nvfp4_error();
  if (x == nullptr || codes == nullptr || scales == nullptr) return fail(slot, "b200q_nvfp4_quantize_activations: NULL argument");
  if (tokens == 0 || k == 0 || (k % 16u) != 0) return fail(slot, "b200q_nvfp4_quantize_activations: tokens must be positive and k a positive multiple of 16");
  if (!aligned(x, 16) || !aligned(codes, 8)) return fail(slot, "b200q_nvfp4_quantize_activations: x must be 16-byte and codes 8-byte aligned");
  if (!std::isfinite(input_scale_divisor) || !(input_scale_divisor > 0.0f)) {
    return fail(slot, "b200q_nvfp4_quantize_activations: input_scale_divisor must be finite and positive");
  }
  if (prepared_state(slot, "b200q_nvfp4_quantize_activations") == nullptr) return -1;
  return quantize_activations_launch(slot, static_cast<const uint16_t *>(x), tokens, k, input_scale_divisor,
                                     static_cast<uint8_t *>(codes), static_cast<uint8_t *>(scales),
                                     static_cast<cudaStream_t>(stream));
}

int32_t b200q_nvfp4_quantize_operand(const void *x_rows, uint32_t tokens_total, uint32_t token_begin, uint32_t token_count,
                                     uint32_t k, float input_scale_divisor, const b200q_nvfp4_workspace *workspace, void *stream) {
  const char *what = "b200q_nvfp4_quantize_operand";
  ErrorSlot &slot = nvfp4_error();
  if (x_rows == nullptr || !aligned(x_rows, 16)) return fail(slot, "%s: x_rows is NULL or not 16-byte aligned", what);
  if (k == 0 || (k % 256u) != 0) return fail(slot, "%s: k = %u is not a positive multiple of 256", what, k);
  if (token_count == 0 || (token_begin % 128u) != 0 || static_cast<uint64_t>(token_begin) + token_count > tokens_total) {
    return fail(slot, "%s: tokens [%u, +%u) must start on a multiple of 128 inside the call's %u tokens", what, token_begin,
                token_count, tokens_total);
  }
  if (token_begin + token_count < tokens_total && (token_count % 128u) != 0) {
    return fail(slot, "%s: only the call's last range may end off a multiple of 128", what);
  }
  if (!std::isfinite(input_scale_divisor) || !(input_scale_divisor > 0.0f)) return fail(slot, "%s: input_scale_divisor must be finite and positive", what);
  const uint64_t need = w4a4_workspace_bytes(k, tokens_total);
  if (workspace == nullptr || workspace->base == nullptr || workspace->bytes < need || !aligned(workspace->base, 256)) {
    return fail(slot, "%s: needs a 256-byte aligned workspace of %llu bytes", what, static_cast<unsigned long long>(need));
  }
  const DeviceState *dev = prepared_state(slot, what);
  if (dev == nullptr) return -1;
  return w4a4_quantize_range(slot, *dev, static_cast<const uint16_t *>(x_rows), tokens_total, token_begin, token_count, k,
                             input_scale_divisor, static_cast<uint8_t *>(workspace->base), static_cast<cudaStream_t>(stream));
}

int32_t b200q_nvfp4_linear_prequantized(const b200q_nvfp4_weight *w, uint32_t tokens, void *y, uint32_t ldy, uint32_t epilogue,
                                        const b200q_nvfp4_workspace *workspace, void *stream) {
  const char *what = "b200q_nvfp4_linear_prequantized";
  ErrorSlot &slot = nvfp4_error();
  if (check_weight(slot, w, what) != 0) return -1;
  if (!w4a4_shape_ok(w->n, w->k)) return fail(slot, "%s: k must be a multiple of 256", what);
  if ((epilogue & ~(B200Q_NVFP4_ADD | B200Q_NVFP4_OUT_F32)) != 0u) return fail(slot, "%s: unknown epilogue 0x%x", what, epilogue);
  if (tokens == 0) return fail(slot, "%s: tokens must be positive", what);
  if (!std::isfinite(w->input_scale_divisor) || !(w->input_scale_divisor > 0.0f)) {
    return fail(slot, "%s: input_scale_divisor must be finite and positive", what);
  }
  if (y == nullptr || !aligned(y, 16) || (ldy % 8u) != 0 || ldy < w->n) return fail(slot, "%s: y must be 16-byte aligned, ldy a multiple of 8 and at least n", what);
  const uint64_t need = w4a4_workspace_bytes(w->k, tokens);
  if (workspace == nullptr || workspace->base == nullptr || workspace->bytes < need || !aligned(workspace->base, 256)) {
    return fail(slot, "%s: needs the 256-byte aligned workspace of %llu bytes the operand was quantized into", what,
                static_cast<unsigned long long>(need));
  }
  const DeviceState *dev = prepared_state(slot, what);
  if (dev == nullptr) return -1;
  return w4a4_launch_prequantized(slot, *dev, static_cast<const uint8_t *>(w->codes), static_cast<const uint8_t *>(w->scales), w->n, w->k,
                                  w->weight_scale_divisor, w->input_scale_divisor, tokens, y, ldy, epilogue,
                                  static_cast<uint8_t *>(workspace->base), static_cast<cudaStream_t>(stream));
}

const char *b200q_nvfp4_last_error(void) { return nvfp4_error().text; }

}  // extern "C"
