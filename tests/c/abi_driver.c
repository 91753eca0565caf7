/* A C99 program over the C ABI alone (no Python, no C++): what a maintainer's own binding sees.
 *
 *   abi_driver host <container.ninfer>   checks that need no device: struct sizes, size queries,
 *                                        argument errors and their texts, the container reader
 *   abi_driver gpu                       (built with -DWITH_CUDA) one NVFP4 product on device 0
 *                                        with weights and activations whose result is known in
 *                                        closed form, through b200q_nvfp4_linear
 *
 * Exit code 0 and a last line "ok" on success; the first failed check is printed and exits 1. */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "b200q_artifact.h"
#include "b200q_nvfp4.h"
#include "ignis_moe.h"
#include "ignis_trellis_linear.h"

#ifdef WITH_CUDA
#include <cuda_runtime_api.h>
#endif

/* sizes the reference's Rust mirrors pin (crates/core/src/trellis.rs:229-234, moe.rs:355-388) */
typedef char weight_is_32_bytes[sizeof(b200q_nvfp4_weight) == 32 ? 1 : -1];
typedef char workspace_is_16_bytes[sizeof(b200q_nvfp4_workspace) == 16 ? 1 : -1];
typedef char trellis_weight_is_40_bytes[sizeof(ignis_trellis_weight) == 40 ? 1 : -1];
typedef char trellis_workspace_is_16_bytes[sizeof(ignis_trellis_workspace) == 16 ? 1 : -1];
typedef char moe_slot_is_16_bytes[sizeof(struct ignis_moe_slot) == 16 ? 1 : -1];
typedef char moe_workspace_is_24_bytes[sizeof(struct ignis_moe_workspace) == 24 ? 1 : -1];
typedef char moe_plan_is_40_bytes[sizeof(struct ignis_moe_plan) == 40 ? 1 : -1];

#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
      exit(1);                                                             \
    }                                                                      \
  } while (0)

static int host_checks(const char *container) {
  uint64_t bytes = 0;
  b200q_nvfp4_weight w;
  uint16_t x[16];
  struct ignis_moe_plan plan;

  /* argument errors come back as -1 with a text, never as a crash */
  CHECK(b200q_nvfp4_linear(NULL, NULL, 1, NULL, 0, B200Q_NVFP4_STORE, B200Q_NVFP4_A16_ONLY, NULL, NULL) == -1);
  CHECK(strlen(b200q_nvfp4_last_error()) > 0);
  memset(&w, 0, sizeof(w));
  w.codes = x, w.scales = x, w.n = 100, w.k = 64, w.weight_scale_divisor = 1.0f, w.input_scale_divisor = 1.0f;
  CHECK(b200q_nvfp4_linear(&w, x, 1, x, 100, B200Q_NVFP4_STORE, B200Q_NVFP4_A16_ONLY, NULL, NULL) == -1);
  CHECK(strstr(b200q_nvfp4_last_error(), "128") != NULL); /* n must be a multiple of 128 */
  CHECK(ignis_trellis_linear(NULL, NULL, 1, NULL, 0, IGNIS_TRELLIS_STORE, NULL, NULL) == -1);
  CHECK(strlen(ignis_trellis_last_error()) > 0);

  /* size queries are host arithmetic */
  CHECK(b200q_nvfp4_workspace_bytes(5120, 5120, B200Q_NVFP4_ALLOW_A4, 8192) > 0);
  CHECK(b200q_nvfp4_workspace_bytes(5120, 5120, B200Q_NVFP4_A16_ONLY, 8) == 256); /* the status line alone */
  CHECK(b200q_nvfp4_workspace_bytes(5120, 5120, B200Q_NVFP4_ALLOW_A4, 8192) > 8192u * 5120u / 2u);
  CHECK(b200q_nvfp4_workspace_bytes(100, 64, B200Q_NVFP4_ALLOW_A4, 64) == 0);
  CHECK(ignis_moe_record_bytes(IGNIS_MOE_PROJ_GATE_UP, 5, &bytes) == 0 && bytes == 1032192u); /* [1280, 2560] at 2.5 bits */
  CHECK(ignis_moe_record_bytes(IGNIS_MOE_PROJ_DOWN, 8, &bytes) == 0 && bytes == 827392u);
  CHECK(ignis_moe_record_bytes(IGNIS_MOE_PROJ_DOWN, 7, &bytes) == -1);
  CHECK(ignis_moe_plan_bytes(8, 64, &plan) == 0 && plan.total >= plan.workspace + plan.acc);

  /* the container reader */
  {
    const uint64_t shape[2] = {34816, 5120};
    b200q_blockscale_geometry g;
    b200q_artifact *a = NULL;
    b200q_artifact_object obj;
    char name[128];
    uint64_t i, count;
    CHECK(b200q_artifact_blockscale_geometry(B200Q_FORMAT_NVFP4, shape, 2, &g) == 0);
    CHECK(g.code_plane_bytes == 89128960u && g.scale_plane_offset == 89128960u && g.encoded_bytes == 100270084u);
    CHECK(b200q_artifact_encoded_size(B200Q_LAYOUT_BLOCKSCALE_K16_M128X4_V1, B200Q_FORMAT_BF16, shape, 2, &bytes) == -1);
    CHECK(b200q_artifact_divisor_name("text/layers/9/mlp/down", name, sizeof(name)) == 0);
    CHECK(strcmp(name, "text/layers/9/mlp/down_projection/input_scale_divisor") == 0);
    CHECK(b200q_artifact_open("/nonexistent/file.ninfer", &a) == -1 && a == NULL);
    CHECK(strstr(b200q_artifact_last_error(), "open") != NULL);
    CHECK(b200q_artifact_open(container, &a) == 0 && a != NULL);
    count = b200q_artifact_object_count(a);
    CHECK(count >= 2);
    for (i = 0; i < count; ++i) {
      CHECK(b200q_artifact_object_at(a, i, &obj) == 0);
      printf("object %s: %llu bytes at %llu\n", obj.name, (unsigned long long)obj.bytes, (unsigned long long)obj.file_offset);
      if (obj.kind == B200Q_ARTIFACT_TENSOR && obj.format == B200Q_FORMAT_NVFP4) {
        CHECK(b200q_artifact_nvfp4_weight(a, obj.name, NULL, NULL, &w) == 0);
        CHECK(w.codes == obj.data && w.n == obj.shape[0] && w.k == obj.shape[1]);
        CHECK(w.weight_scale_divisor > 0.0f && w.input_scale_divisor > 0.0f);
      }
    }
    CHECK(b200q_artifact_find(a, "no/such/object", &obj) == -1);
    b200q_artifact_close(a);
  }
  return 0;
}

#ifdef WITH_CUDA
#define CUDA_OK(call) CHECK((call) == cudaSuccess)

static int gpu_checks(void) {
  enum { N = 256, K = 512, TOKENS = 8 };
  const size_t code_bytes = (size_t)N * K / 2, scale_bytes = (size_t)N * K / 16;
  uint8_t *codes, *scales;
  uint16_t *x, *y;
  uint16_t hx[TOKENS * K], hy[TOKENS * N];
  b200q_nvfp4_weight w;
  uint32_t status = 1;
  int t, c;

  CHECK(b200q_nvfp4_prepare() == 0);
  CUDA_OK(cudaMalloc((void **)&codes, code_bytes));
  CUDA_OK(cudaMalloc((void **)&scales, scale_bytes));
  CUDA_OK(cudaMalloc((void **)&x, sizeof(hx)));
  CUDA_OK(cudaMalloc((void **)&y, sizeof(hy)));
  CUDA_OK(cudaMemset(codes, 0x22, code_bytes));   /* every E2M1 code is 2: the value 1.0 */
  CUDA_OK(cudaMemset(scales, 0x38, scale_bytes)); /* every E4M3 scale is 1.0 (the swizzle moves equal bytes onto equal bytes) */
  for (t = 0; t < TOKENS; ++t)
    for (c = 0; c < K; ++c) hx[t * K + c] = (uint16_t)(t % 2 == 0 ? 0x3F80 : 0xBF80); /* BF16 +1, -1 by token */
  CUDA_OK(cudaMemcpy(x, hx, sizeof(hx), cudaMemcpyHostToDevice));
  w.codes = codes, w.scales = scales, w.n = N, w.k = K, w.weight_scale_divisor = 2.0f, w.input_scale_divisor = 1.0f;
  CHECK(b200q_nvfp4_linear(&w, x, TOKENS, y, N, B200Q_NVFP4_STORE, B200Q_NVFP4_A16_ONLY, NULL, NULL) == 0);
  CUDA_OK(cudaMemcpy(hy, y, sizeof(hy), cudaMemcpyDeviceToHost));
  for (t = 0; t < TOKENS; ++t)
    for (c = 0; c < N; ++c) CHECK(hy[t * N + c] == (t % 2 == 0 ? 0x4380 : 0xC380)); /* K / 2 = +-256 in BF16 */
  CHECK(b200q_nvfp4_device_status(NULL, &status) == 0 && status == 0);
  CUDA_OK(cudaFree(codes));
  CUDA_OK(cudaFree(scales));
  CUDA_OK(cudaFree(x));
  CUDA_OK(cudaFree(y));
  return 0;
}
#endif

int main(int argc, char **argv) {
  if (argc >= 3 && strcmp(argv[1], "host") == 0) {
    if (host_checks(argv[2]) != 0) return 1;
#ifdef WITH_CUDA
  } else if (argc >= 2 && strcmp(argv[1], "gpu") == 0) {
    if (gpu_checks() != 0) return 1;
#endif
  } else {
    fprintf(stderr, "usage: %s host <container.ninfer> | gpu\n", argv[0]);
    return 2;
  }
  printf("ok\n");
  return 0;
}
