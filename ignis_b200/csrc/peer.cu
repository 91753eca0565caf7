// A barrier between the ranks of one node, on the device, over peer-mapped flag arrays: what turns
// a product that stores its column shard into every rank's buffer (b200q_nvfp4_linear_group_scatter)
// into an all-gather. No counterpart in the single-GPU reference.
//
// Every rank owns an array of `peers` 32-bit flags (slot s is written by rank s) that every other
// rank has mapped. Barrier number `epoch` (1, 2, ... per flag array): thread s of one warp stores
// `epoch` into slot `rank` of rank s's array with a system-scope release, then waits, with a
// system-scope acquire load, until slot s of its own array has reached `epoch`. The kernel runs in
// stream order behind the product, so the product's peer stores are complete and visible before
// the flag that announces them. The wait is bounded: when it runs out the kernel records which
// peers were missing in status[0] and returns, and the host decides what to do. With epoch 0 the
// kernel numbers the barrier itself from status[1], so a launch captured in a CUDA graph counts on
// at every replay (all ranks must then use epoch 0 for every barrier on that flag array).
#include "../../include/b200q_nvfp4.h"

#include "common.cuh"

namespace b200q {
namespace {

// `polls`: how often a thread looks at its flag before it gives up; with the sleep below the
// default (2^22, B200Q_PEER_BARRIER_POLLS at prepare) is about two seconds.
__global__ void __launch_bounds__(32) peer_barrier_kernel(uint32_t *const *flags_peers, uint32_t peers, uint32_t rank,
                                                          uint32_t epoch, uint32_t *status, uint32_t polls) {
  griddep_launch_dependents();
  griddep_wait();  // the product before this kernel has finished and flushed its stores
  const uint32_t s = threadIdx.x;
  if (epoch == 0u) {  // numbered on the device, so a captured launch counts on at every replay
    uint32_t next = 0;
    if (s == 0) next = atomicAdd(status + 1, 1u) + 1u;
    epoch = __shfl_sync(0xFFFFFFFFu, next, 0);
  }
  if (s >= peers) return;
  __threadfence_system();
  st_release_sys(flags_peers[s] + rank, epoch);
  bool seen = false;
  const uint32_t *mine = flags_peers[rank] + s;
  for (uint32_t poll = 0; poll < polls; ++poll) {
    if (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) >= 0) {
      seen = true;
      break;
    }
    __nanosleep(400);
  }
  if (!seen) atomicOr(status, 1u << s);
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int32_t b200q_peer_barrier(uint32_t *const *flags_peers, uint32_t peers, uint32_t rank, uint32_t epoch,
                                      uint32_t *status, void *stream) {
  ErrorSlot &slot = nvfp4_error();
  if (flags_peers == nullptr || status == nullptr) return fail(slot, "b200q_peer_barrier: NULL argument");
  if (peers == 0 || peers > 8u || rank >= peers) return fail(slot, "b200q_peer_barrier: peers = %u, rank = %u are out of range", peers, rank);
  const DeviceState *dev = device_state(slot);
  if (dev == nullptr) return -1;
  if (!dev->prepared) return fail(slot, "b200q_peer_barrier: the device was not prepared (call b200q_nvfp4_prepare at load)");
  const cudaError_t err = launch(peer_barrier_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), dev->pdl != 0,
                                 flags_peers, peers, rank, epoch, status, static_cast<uint32_t>(dev->peer_barrier_polls));
  if (err != cudaSuccess) return fail(slot, "b200q_peer_barrier: launch failed: %s", cudaGetErrorString(err));
  return 0;
}
