// The NVFP4 members of the reference's C++ ops API over the C ABI of b200q_nvfp4.h.
//
// The reference's leaf calls its NVFP4 linear through C++ (ninfer::ops::linear, linear_add,
// linear_swiglu and their *_workspace_capacity_bytes: kernel/vendor/include/ninfer/ops/linear.h:
// 20-119, linear_add.h:69-73, linear_swiglu.h:21-82), with ninfer::Tensor / ninfer::Weight
// (kernel/vendor/src/core/tensor.h:11-75) and a WorkspaceArena (core/arena.h:46-98, :150). This
// header gives the same functions - names, argument order and meaning, error behaviour (they throw
// std::invalid_argument where the reference's dispatcher does, nvfp4_dispatch.cpp:20-49, :75-95) -
// as templates over the caller's tensor, weight and arena types, so that the leaf's dispatcher
// (kernel/src/linear.cu:112-150) forwards its NVFP4 branch with one line,
//
//     case QType::NVFP4: return b200q::ops::linear(x, w, out, policy, workspace, stream);
//
// and the header itself needs nothing of the reference's tree. What a type must offer:
//   Tensor  .data (void*), .ne[4] (int32, dimension zero fastest), .nb[4] (int64 strides in
//           bytes); activations and outputs are BF16, [K, T] and [N, T] (token-major in memory)
//   Weight  .qdata, .scales (device pointers), .n, .k (int32), .weight_scale_divisor,
//           .input_scale_divisor (float)
//   Arena   .alloc_bytes(bytes, align) returning something with .data and .bytes, and .scope()
//           returning a guard that gives the bytes back when it goes out of scope
//   Stream  cudaStream_t (anything convertible to void*)
#ifndef B200Q_NINFER_OPS_HPP_
#define B200Q_NINFER_OPS_HPP_

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "b200q_nvfp4.h"

namespace b200q {
namespace ops {

/// The reference's LinearPolicy (ninfer/ops/linear.h:20-24), same enumerators in the same order.
enum class LinearPolicy : std::uint8_t { A16Only, AllowA8, AllowA4 };

namespace detail {

inline std::uint32_t policy_word(LinearPolicy policy, std::uint32_t problem) {
  switch (policy) {
    case LinearPolicy::A16Only: return B200Q_NVFP4_A16_ONLY | problem;
    case LinearPolicy::AllowA4: return B200Q_NVFP4_ALLOW_A4 | problem;
    default: throw std::invalid_argument("nvfp4 linear: unsupported policy");  // NVFP4 admits A16Only and AllowA4
  }
}

template <class Weight>
b200q_nvfp4_weight view(const Weight &w) {
  if (w.n <= 0 || w.k <= 0) throw std::invalid_argument("nvfp4 linear: unsupported shape");
  return b200q_nvfp4_weight{w.qdata, w.scales, static_cast<std::uint32_t>(w.n), static_cast<std::uint32_t>(w.k),
                            w.weight_scale_divisor, w.input_scale_divisor};
}

/// [rows, T] BF16, contiguous, non-null, 16-byte aligned, every extent positive; returns T.
template <class Tensor>
std::uint32_t columns(const Tensor &t, std::int32_t rows, const char *what) {
  if (t.data == nullptr) throw std::invalid_argument(std::string("nvfp4 linear: null ") + what);
  if (reinterpret_cast<std::uintptr_t>(t.data) % 16 != 0)
    throw std::invalid_argument(std::string("nvfp4 linear: ") + what + " is not 16-byte aligned");
  if (t.ne[0] != rows || t.ne[1] <= 0 || t.ne[2] != 1 || t.ne[3] != 1)
    throw std::invalid_argument(std::string("nvfp4 linear: ") + what + " has the wrong shape");
  if (t.nb[0] != 2 || t.nb[1] != 2 * static_cast<std::int64_t>(rows))
    throw std::invalid_argument(std::string("nvfp4 linear: ") + what + " is not contiguous BF16");
  return static_cast<std::uint32_t>(t.ne[1]);
}

inline void check(std::int32_t rc) {
  if (rc != 0) throw std::invalid_argument(b200q_nvfp4_last_error());
}

/// The C ABI answers 256 (one status line, which such calls never touch and which may be absent)
/// for the routes that keep nothing in global memory; the reference's contract for those is zero.
constexpr std::uint64_t kNoTransientBytes = 256;

/// Runs `call(workspace*)` with `bytes` of the arena (none for a route that needs none), given
/// back on return.
template <class Arena, class Stream, class Call>
void with_workspace(Arena &arena, std::uint64_t bytes, Stream stream, Call call) {
  if (bytes <= kNoTransientBytes) {
    call(static_cast<const b200q_nvfp4_workspace *>(nullptr));
    return;
  }
  auto scope = arena.scope();
  auto span = arena.alloc_bytes(static_cast<std::size_t>(bytes), 256);
  if (span.data == nullptr || span.bytes < bytes) throw std::invalid_argument("nvfp4 W4A4 linear requires caller workspace");
  const b200q_nvfp4_workspace ws{span.data, span.bytes};
  check(b200q_nvfp4_workspace_init(&ws, reinterpret_cast<void *>(stream)));  // the arena's bytes are not zero: clear the status line
  call(&ws);
  (void)scope;
}

inline std::size_t capacity(std::int32_t output_rows, std::int32_t input_rows, std::uint32_t policy, std::int32_t min_tokens,
                            std::int32_t max_tokens) {
  if (min_tokens <= 0 || max_tokens < min_tokens) throw std::invalid_argument("nvfp4 linear workspace: invalid token interval");
  if (output_rows <= 0 || input_rows <= 0) throw std::invalid_argument("nvfp4 linear: unsupported shape");
  // the need grows with the token count, so the interval's need is its upper end's
  const std::uint64_t bytes = b200q_nvfp4_workspace_bytes(static_cast<std::uint32_t>(output_rows), static_cast<std::uint32_t>(input_rows),
                                                          policy, static_cast<std::uint32_t>(max_tokens));
  if (bytes == 0) throw std::invalid_argument("nvfp4 linear: unsupported shape");
  return bytes <= kNoTransientBytes ? 0 : static_cast<std::size_t>(bytes);
}

}  // namespace detail

/// ninfer::ops::linear_workspace_capacity_bytes for QType::NVFP4 (ninfer/ops/linear.h:31-35): the
/// transient bytes Linear needs for every T in [min_tokens, max_tokens]; 0 when the resolved
/// route needs none. `problem`: one of B200Q_NVFP4_PROBLEM_* or 0.
inline std::size_t linear_workspace_capacity_bytes(std::int32_t output_rows, std::int32_t input_rows, LinearPolicy policy,
                                                   std::int32_t min_tokens, std::int32_t max_tokens, std::uint32_t problem = 0) {
  return detail::capacity(output_rows, input_rows, detail::policy_word(policy, problem), min_tokens, max_tokens);
}

/// ninfer::ops::linear (ninfer/ops/linear.h:99-100): out[N, T] = BF16(w[N, K] x[K, T]).
template <class Tensor, class Weight, class Arena, class Stream>
void linear(const Tensor &x, const Weight &w, Tensor &out, LinearPolicy policy, Arena &workspace, Stream stream,
            std::uint32_t problem = 0) {
  const b200q_nvfp4_weight view = detail::view(w);
  const std::uint32_t word = detail::policy_word(policy, problem);
  const std::uint32_t tokens = detail::columns(x, w.k, "x");
  if (detail::columns(out, w.n, "out") != tokens) throw std::invalid_argument("nvfp4 linear: x and out disagree on T");
  detail::with_workspace(workspace, b200q_nvfp4_workspace_bytes(view.n, view.k, word, tokens), stream, [&](const b200q_nvfp4_workspace *ws) {
    detail::check(b200q_nvfp4_linear(&view, x.data, tokens, out.data, view.n, B200Q_NVFP4_STORE, word, ws, reinterpret_cast<void *>(stream)));
  });
}

/// The A16-only overload (ninfer/ops/linear.h:113): no workspace.
template <class Tensor, class Weight, class Stream>
void linear(const Tensor &x, const Weight &w, Tensor &out, Stream stream) {
  const b200q_nvfp4_weight view = detail::view(w);
  const std::uint32_t tokens = detail::columns(x, w.k, "x");
  if (detail::columns(out, w.n, "out") != tokens) throw std::invalid_argument("nvfp4 linear: x and out disagree on T");
  detail::check(b200q_nvfp4_linear(&view, x.data, tokens, out.data, view.n, B200Q_NVFP4_STORE, B200Q_NVFP4_A16_ONLY, nullptr,
                                   reinterpret_cast<void *>(stream)));
}

/// ninfer::ops::linear_add (ninfer/ops/linear_add.h:72-73): residual[N, T] += w x, one rounding.
template <class Tensor, class Weight, class Arena, class Stream>
void linear_add(const Tensor &x, const Weight &w, Tensor &residual, LinearPolicy policy, Arena &workspace, Stream stream) {
  const b200q_nvfp4_weight view = detail::view(w);
  const std::uint32_t word = detail::policy_word(policy, B200Q_NVFP4_PROBLEM_RESIDUAL);
  const std::uint32_t tokens = detail::columns(x, w.k, "x");
  if (detail::columns(residual, w.n, "residual") != tokens) throw std::invalid_argument("nvfp4 linear: x and residual disagree on T");
  detail::with_workspace(workspace, b200q_nvfp4_workspace_bytes(view.n, view.k, word, tokens), stream, [&](const b200q_nvfp4_workspace *ws) {
    detail::check(b200q_nvfp4_linear(&view, x.data, tokens, residual.data, view.n, B200Q_NVFP4_ADD, word, ws, reinterpret_cast<void *>(stream)));
  });
}

/// ninfer::ops::linear_swiglu_workspace_capacity_bytes for NVFP4 (ninfer/ops/linear_swiglu.h:33-36).
inline std::size_t linear_swiglu_workspace_capacity_bytes(std::int32_t gate_up_rows, std::int32_t input_rows, LinearPolicy policy,
                                                          std::int32_t min_tokens, std::int32_t max_tokens) {
  return detail::capacity(gate_up_rows, input_rows, detail::policy_word(policy, B200Q_NVFP4_PROBLEM_GATE_UP), min_tokens, max_tokens);
}

/// ninfer::ops::linear_swiglu (ninfer/ops/linear_swiglu.h:73-74): out[N/2, T] = BF16(silu(g) * u),
/// g | u = gate_up x.
template <class Tensor, class Weight, class Arena, class Stream>
void linear_swiglu(const Tensor &x, const Weight &gate_up, Tensor &out, LinearPolicy policy, Arena &workspace, Stream stream) {
  const b200q_nvfp4_weight view = detail::view(gate_up);
  const std::uint32_t word = detail::policy_word(policy, B200Q_NVFP4_PROBLEM_GATE_UP);
  const std::uint32_t tokens = detail::columns(x, gate_up.k, "x");
  if (gate_up.n % 2 != 0 || detail::columns(out, gate_up.n / 2, "out") != tokens)
    throw std::invalid_argument("nvfp4 linear: x and out disagree on T");
  detail::with_workspace(workspace, b200q_nvfp4_workspace_bytes(view.n, view.k, word, tokens), stream, [&](const b200q_nvfp4_workspace *ws) {
    detail::check(b200q_nvfp4_linear_swiglu(&view, x.data, tokens, out.data, view.n / 2, word, ws, reinterpret_cast<void *>(stream)));
  });
}

}  // namespace ops
}  // namespace b200q

#endif  // B200Q_NINFER_OPS_HPP_
