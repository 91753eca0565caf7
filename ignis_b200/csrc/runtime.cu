// Error slots and per-device state shared by every op family.
#include "common.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace b200q {

ErrorSlot &nvfp4_error() {
  static thread_local ErrorSlot slot = {""};
  return slot;
}
ErrorSlot &trellis_error() {
  static thread_local ErrorSlot slot = {""};
  return slot;
}
ErrorSlot &moe_error() {
  static thread_local ErrorSlot slot = {""};
  return slot;
}

namespace {
constexpr int kMaxDevices = 64;
DeviceState g_state[kMaxDevices];
std::mutex g_mutex;

// A measurement switch read once per prepare, as the reference reads its own
// (kernel/src/process_environment.h:17-34): unset or unparsable gives `fallback`.
int env_int(const char *name, int fallback) {
  const char *v = std::getenv(name);
  if (v == nullptr || *v == '\0') return fallback;
  char *end = nullptr;
  const long parsed = std::strtol(v, &end, 10);
  return (end == v) ? fallback : static_cast<int>(parsed);
}
}  // namespace

DeviceState *device_state(ErrorSlot &slot) {
  int device = -1;
  const cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) {
    fail(slot, "no CUDA device: %s", cudaGetErrorString(err));
    return nullptr;
  }
  if (device < 0 || device >= kMaxDevices) {
    fail(slot, "device ordinal %d is outside the supported range", device);
    return nullptr;
  }
  return &g_state[device];
}

int32_t prepare_all(ErrorSlot &slot) {
  if (prepare_device(slot) != 0) return -1;
  if (prepare_nvfp4_kernels(slot) != 0) return -1;
  if (prepare_trellis_kernels(slot) != 0) return -1;
  return prepare_moe_kernels(slot);
}

int32_t prepare_device(ErrorSlot &slot) {
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState *state = device_state(slot);
  if (state == nullptr) return -1;
  // A repeated call re-reads the environment switches (tests and sweeps flip them between
  // calls); everything else it computes is a function of the device alone.
  int device = 0;
  cudaGetDevice(&device);
  cudaDeviceProp prop;
  cudaError_t err = cudaGetDeviceProperties(&prop, device);
  if (err != cudaSuccess) return fail(slot, "cudaGetDeviceProperties: %s", cudaGetErrorString(err));
  if (prop.major != 10) {
    return fail(slot, "this library is built for sm_100a only; device %d is sm_%d%d", device, prop.major, prop.minor);
  }
  DeviceState fresh;
  fresh.sm_count = prop.multiProcessorCount;
  fresh.pdl = env_int("B200Q_PDL", 1) != 0;
  fresh.gemv_rb = env_int("B200Q_GEMV_RM", 0);
  fresh.gemv_kc = env_int("B200Q_GEMV_KC", 0);
  fresh.gemv_ctas_per_sm = env_int("B200Q_GEMV_CTAS_PER_SM", 2);
  fresh.gemv_xu = env_int("B200Q_GEMV_XU", 8);
  fresh.a16_mma = env_int("B200Q_A16_MMA", 1);
  fresh.a4_decode = env_int("B200Q_A4_DECODE", 1);
  fresh.trellis_kc_max = env_int("B200Q_TRELLIS_KC_MAX", 8);
  fresh.a4_decode_pair = env_int("B200Q_A4_DECODE_PAIR", -1);
  fresh.a4_decode_kc = env_int("B200Q_A4_DECODE_KC", 0);
  fresh.a4_decode_groups = env_int("B200Q_A4_DECODE_GROUPS", 0);
  fresh.a4_decode_ctas = env_int("B200Q_A4_DECODE_CTAS", 2) == 1 ? 1 : 2;
  fresh.a16_mma_wide = env_int("B200Q_A16_MMA_WIDE", 1);
  fresh.w4a4_pair = env_int("B200Q_W4A4_PAIR", 1);
  fresh.sm_cap = env_int("IGNIS_TRELLIS_SM_CAP", 0);
  if (fresh.sm_cap < 0 || fresh.sm_cap > fresh.sm_count) fresh.sm_cap = 0;
  fresh.trellis_tc = env_int("B200Q_TRELLIS_TC", 1);
  fresh.moe_tc = env_int("B200Q_MOE_TC", 1);
  fresh.peer_barrier_polls = env_int("B200Q_PEER_BARRIER_POLLS", 1 << 22);
  if (fresh.peer_barrier_polls < 1) fresh.peer_barrier_polls = 1;
  for (int i = 0; i < 9; ++i) fresh.gemv_slots[i] = state->gemv_slots[i];
  fresh.prepared = true;
  *state = fresh;
  return 0;
}

}  // namespace b200q
