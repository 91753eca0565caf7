// The C++ ops shim (include/b200q_ninfer_ops.hpp) driven the way the reference's leaf would drive
// it, with stand-ins for ninfer::Tensor, ninfer::Weight and the WorkspaceArena that carry the same
// member names (kernel/vendor/src/core/tensor.h:11-75, core/arena.h:46-98).
//
//   ops_shim_driver host   argument checks and their exceptions, workspace capacities
//   ops_shim_driver gpu    (built with -DWITH_CUDA) linear under A16Only and AllowA4, linear_add and
//                          linear_swiglu on device 0 against results known in closed form
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <initializer_list>
#include <stdexcept>
#include <string>
#include <vector>

#include "b200q_ninfer_ops.hpp"

#ifdef WITH_CUDA
#include <cuda_runtime_api.h>
#endif

namespace standin {

struct Tensor {  // BF16, dimension zero fastest
  void *data = nullptr;
  std::int32_t ne[4] = {1, 1, 1, 1};
  std::int64_t nb[4] = {0, 0, 0, 0};
  Tensor() = default;
  Tensor(void *p, std::int32_t rows, std::int32_t cols) : data(p) {
    ne[0] = rows, ne[1] = cols;
    nb[0] = 2, nb[1] = 2 * static_cast<std::int64_t>(rows), nb[2] = nb[3] = nb[1] * cols;
  }
};

struct Weight {
  const void *qdata = nullptr;
  const void *scales = nullptr;
  std::int32_t n = 0, k = 0;
  float weight_scale_divisor = 0.0f, input_scale_divisor = 0.0f;
};

struct Span {
  void *data = nullptr;
  std::size_t bytes = 0;
};

class Arena {  // a bump allocator over one region, with the reference's scope() guard
 public:
  class Scope {
   public:
    explicit Scope(Arena &a) : arena_(&a), saved_(a.used_) {}
    Scope(Scope &&o) noexcept : arena_(o.arena_), saved_(o.saved_) { o.arena_ = nullptr; }
    ~Scope() {
      if (arena_ != nullptr) arena_->used_ = saved_;
    }

   private:
    Arena *arena_;
    std::size_t saved_;
  };
  Arena(void *base, std::size_t capacity) : base_(static_cast<char *>(base)), capacity_(capacity) {}
  Span alloc_bytes(std::size_t bytes, std::size_t align = 256) {
    const std::size_t start = (used_ + align - 1) / align * align;
    if (start + bytes > capacity_) throw std::runtime_error("arena exhausted");
    used_ = start + bytes;
    peak_ = used_ > peak_ ? used_ : peak_;
    return Span{base_ + start, bytes};
  }
  Scope scope() { return Scope(*this); }
  std::size_t used() const { return used_; }
  std::size_t peak() const { return peak_; }

 private:
  char *base_;
  std::size_t capacity_, used_ = 0, peak_ = 0;
};

}  // namespace standin

#define CHECK(cond)                                                             \
  do {                                                                          \
    if (!(cond)) {                                                              \
      std::fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
      std::exit(1);                                                             \
    }                                                                           \
  } while (0)

template <class F>
static std::string thrown(F f) {
  try {
    f();
  } catch (const std::invalid_argument &e) {
    return e.what();
  }
  return "";
}

using b200q::ops::LinearPolicy;
using standin::Arena;
using standin::Tensor;
using standin::Weight;

static void host_checks() {
  alignas(256) static std::uint16_t buffer[4096];
  Weight w;
  w.qdata = buffer, w.scales = buffer, w.n = 128, w.k = 64, w.weight_scale_divisor = 1.0f, w.input_scale_divisor = 1.0f;
  Tensor x(buffer, 64, 4), out(buffer + 1024, 128, 4);
  Arena arena(nullptr, 0);
  void *stream = nullptr;
  // the reference's dispatcher refuses AllowA8 for NVFP4 (nvfp4_dispatch.cpp:27)
  CHECK(thrown([&] { b200q::ops::linear(x, w, out, LinearPolicy::AllowA8, arena, stream); }) == "nvfp4 linear: unsupported policy");
  Tensor null_x = x;
  null_x.data = nullptr;
  CHECK(thrown([&] { b200q::ops::linear(null_x, w, out, stream); }) == "nvfp4 linear: null x");
  Tensor odd = x;
  odd.data = reinterpret_cast<char *>(buffer) + 2;
  CHECK(thrown([&] { b200q::ops::linear(odd, w, out, stream); }).find("not 16-byte aligned") != std::string::npos);
  Tensor empty(buffer, 64, 0);  // T = 0 is invalid rather than a no-op (ninfer/ops/linear.h:56-58)
  CHECK(thrown([&] { b200q::ops::linear(empty, w, out, stream); }).find("wrong shape") != std::string::npos);
  Tensor wrong_k(buffer, 128, 4);
  CHECK(thrown([&] { b200q::ops::linear(wrong_k, w, out, stream); }).find("wrong shape") != std::string::npos);
  Tensor five(buffer + 1024, 128, 5);
  CHECK(thrown([&] { b200q::ops::linear(x, w, five, stream); }).find("disagree on T") != std::string::npos);
  Tensor strided = x;
  strided.nb[1] = 256;
  CHECK(thrown([&] { b200q::ops::linear(strided, w, out, stream); }).find("not contiguous") != std::string::npos);
  Weight bad = w;
  bad.n = 0;
  CHECK(thrown([&] { b200q::ops::linear(x, bad, out, stream); }) == "nvfp4 linear: unsupported shape");
  // a valid call without a prepared device: the C ABI's own refusal comes through as the exception's text
  CHECK(!thrown([&] { b200q::ops::linear(x, w, out, stream); }).empty());
  // capacities (linear_workspace_capacity_bytes, ninfer/ops/linear.h:31-35)
  CHECK(b200q::ops::linear_workspace_capacity_bytes(5120, 17408, LinearPolicy::A16Only, 1, 8192) == 0);
  const std::size_t small = b200q::ops::linear_workspace_capacity_bytes(5120, 17408, LinearPolicy::AllowA4, 1, 1024);
  const std::size_t large = b200q::ops::linear_workspace_capacity_bytes(5120, 17408, LinearPolicy::AllowA4, 1, 8192);
  CHECK(small > 0 && large > small);
  CHECK(b200q::ops::linear_swiglu_workspace_capacity_bytes(34816, 5120, LinearPolicy::AllowA4, 1, 4096) > 0);
  CHECK(thrown([&] { (void)b200q::ops::linear_workspace_capacity_bytes(5120, 17408, LinearPolicy::AllowA4, 0, 8); }) ==
        "nvfp4 linear workspace: invalid token interval");
  CHECK(thrown([&] { (void)b200q::ops::linear_workspace_capacity_bytes(5120, 17408, LinearPolicy::AllowA8, 1, 8); }) ==
        "nvfp4 linear: unsupported policy");
}

#ifdef WITH_CUDA
#define CUDA_OK(call) CHECK((call) == cudaSuccess)

static float bf16_to_float(std::uint16_t h) {
  const std::uint32_t bits = static_cast<std::uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

static std::uint16_t float_to_bf16(float f) {
  std::uint32_t bits;
  std::memcpy(&bits, &f, 4);
  bits += 0x7FFFu + ((bits >> 16) & 1u);
  return static_cast<std::uint16_t>(bits >> 16);
}

static void gpu_checks() {
  constexpr int N = 512, K = 512;
  CHECK(b200q_nvfp4_prepare() == 0);
  std::uint8_t *codes, *scales;
  CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&codes), N * K / 2));
  CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&scales), N * K / 16));
  CUDA_OK(cudaMemset(codes, 0x22, N * K / 2));   // every weight code is E2M1 1.0
  CUDA_OK(cudaMemset(scales, 0x38, N * K / 16)); // every block scale is E4M3 1.0
  Weight w;
  w.qdata = codes, w.scales = scales, w.n = N, w.k = K, w.weight_scale_divisor = 1.0f, w.input_scale_divisor = 1.0f;
  const std::size_t arena_bytes = 8u << 20;
  void *arena_base;
  CUDA_OK(cudaMalloc(&arena_base, arena_bytes));
  CUDA_OK(cudaMemset(arena_base, 0xFF, arena_bytes));   // an arena hands out bytes that are not zero
  Arena arena(arena_base, arena_bytes);
  cudaStream_t stream = nullptr;

  for (int tokens : {1, 8, 40, 200}) {
    std::vector<std::uint16_t> hx(static_cast<std::size_t>(tokens) * K), hy(static_cast<std::size_t>(tokens) * N);
    for (int t = 0; t < tokens; ++t)
      for (int c = 0; c < K; ++c) hx[static_cast<std::size_t>(t) * K + c] = float_to_bf16((t % 4 + 1) * 0.25f);  // 0.25 .. 1.0, by token
    std::uint16_t *x, *y;
    CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&x), hx.size() * 2));
    CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&y), hy.size() * 2));
    CUDA_OK(cudaMemcpy(x, hx.data(), hx.size() * 2, cudaMemcpyHostToDevice));
    Tensor tx(x, K, tokens), ty(y, N, tokens);
    // A16: exact. Every product term is the activation itself, K of them.
    b200q::ops::linear(tx, w, ty, stream);
    CUDA_OK(cudaMemcpy(hy.data(), y, hy.size() * 2, cudaMemcpyDeviceToHost));
    for (int t = 0; t < tokens; ++t)
      for (int r = 0; r < N; ++r) CHECK(bf16_to_float(hy[static_cast<std::size_t>(t) * N + r]) == K * (t % 4 + 1) * 0.25f);
    // linear_add on top of that: exactly twice the product (a power-of-two multiple stays exact in BF16)
    b200q::ops::linear_add(tx, w, ty, LinearPolicy::A16Only, arena, stream);
    CUDA_OK(cudaMemcpy(hy.data(), y, hy.size() * 2, cudaMemcpyDeviceToHost));
    for (int t = 0; t < tokens; ++t)
      for (int r = 0; r < N; ++r) CHECK(bf16_to_float(hy[static_cast<std::size_t>(t) * N + r]) == 2 * K * (t % 4 + 1) * 0.25f);
    // AllowA4: the activations go through FP4 with an E4M3 block scale; constant blocks lose at most the scale's rounding
    b200q::ops::linear(tx, w, ty, LinearPolicy::AllowA4, arena, stream, B200Q_NVFP4_PROBLEM_RESIDUAL);
    CUDA_OK(cudaMemcpy(hy.data(), y, hy.size() * 2, cudaMemcpyDeviceToHost));
    for (int t = 0; t < tokens; ++t)
      for (int r = 0; r < N; ++r) {
        const float want = K * (t % 4 + 1) * 0.25f, got = bf16_to_float(hy[static_cast<std::size_t>(t) * N + r]);
        CHECK(std::fabs(got - want) <= 0.07f * want);
      }
    CHECK(arena.used() == 0);   // every call gave its bytes back
    CUDA_OK(cudaFree(x));
    CUDA_OK(cudaFree(y));
  }
  CHECK(arena.peak() > 0);      // the wide AllowA4 calls did take a workspace from the arena

  {  // linear_swiglu: gate and up rows both give K * x = 1, so every output is BF16(silu(1))
    const int tokens = 8;
    std::vector<std::uint16_t> hx(static_cast<std::size_t>(tokens) * K, float_to_bf16(1.0f / K)), hh(static_cast<std::size_t>(tokens) * N / 2);
    std::uint16_t *x, *h;
    CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&x), hx.size() * 2));
    CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&h), hh.size() * 2));
    CUDA_OK(cudaMemcpy(x, hx.data(), hx.size() * 2, cudaMemcpyHostToDevice));
    Tensor tx(x, K, tokens), th(h, N / 2, tokens);
    b200q::ops::linear_swiglu(tx, w, th, LinearPolicy::A16Only, arena, stream);
    CUDA_OK(cudaMemcpy(hh.data(), h, hh.size() * 2, cudaMemcpyDeviceToHost));
    const float want = 1.0f / (1.0f + std::exp(-1.0f));
    for (std::uint16_t v : hh) CHECK(std::fabs(bf16_to_float(v) - want) <= want / 128.0f);   // within one BF16 step
    CUDA_OK(cudaFree(x));
    CUDA_OK(cudaFree(h));
  }
  std::uint32_t status = 1;
  CHECK(b200q_nvfp4_device_status(nullptr, &status) == 0 && status == 0);
  CUDA_OK(cudaFree(arena_base));
  CUDA_OK(cudaFree(codes));
  CUDA_OK(cudaFree(scales));
}
#endif

int main(int argc, char **argv) {
  if (argc >= 2 && std::strcmp(argv[1], "host") == 0) {
    host_checks();
#ifdef WITH_CUDA
  } else if (argc >= 2 && std::strcmp(argv[1], "gpu") == 0) {
    gpu_checks();
#endif
  } else {
    std::fprintf(stderr, "usage: %s host | gpu\n", argv[0]);
    return 2;
  }
  std::printf("ok\n");
  return 0;
}
