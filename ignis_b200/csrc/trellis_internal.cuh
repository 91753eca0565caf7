// What the dense trellis entry points (trellis_linear.cu) use of the tensor-core prefill route
// (trellis_prefill.cu).
#ifndef B200Q_TRELLIS_INTERNAL_CUH
#define B200Q_TRELLIS_INTERNAL_CUH

#include "../../include/ignis_trellis_linear.h"

#include "common.cuh"

namespace b200q {

int32_t trellis_tc_prepare(ErrorSlot &slot);
// Workspace bytes of a call of `tokens` tokens over `weights` weights of `in` inputs on that route.
uint64_t trellis_tc_workspace_bytes(uint32_t in, uint32_t weights, uint32_t tokens);
// Whether a call takes the route: more than 64 tokens and a workspace that holds the rotated rows.
bool trellis_tc_takes(const DeviceState &dev, uint32_t in, uint32_t tokens, uint32_t weights, const ignis_trellis_workspace *workspace);
// y = x W through `epilogue` (0 store, 1 add), or with `up` the SwiGLU of the pair into y.
int32_t trellis_tc_linear(ErrorSlot &slot, const DeviceState &dev, const ignis_trellis_weight *w, const ignis_trellis_weight *up,
                          const void *x, uint32_t tokens, void *y, uint32_t ldy, uint32_t epilogue,
                          const ignis_trellis_workspace *workspace, cudaStream_t stream, const char *what);
int32_t trellis_tc_status(ErrorSlot &slot, cudaStream_t stream, uint32_t *status);

}  // namespace b200q

#endif
