// Instantiations of the all-reduce fused with the optimizer update, one per
// update rule (float32; the rules of dragon/kernels/training/cuda/sgd_kernel.cu
// and adam_kernel.cu).
#include "../../include/dgn.h"
#include "dgn_update.cuh"

namespace dgn {

const void* update_kernel_fn(int kind) {
  switch (kind) {
    case DGN_UPDATE_MOMENTUM_SGD: return (const void*)ar_update_kernel<kUpdMomentumSGD>;
    case DGN_UPDATE_NESTEROV_SGD: return (const void*)ar_update_kernel<kUpdNesterovSGD>;
    case DGN_UPDATE_ADAM: return (const void*)ar_update_kernel<kUpdAdam>;
    case DGN_UPDATE_ADAMW: return (const void*)ar_update_kernel<kUpdAdamW>;
    default: return nullptr;
  }
}

}  // namespace dgn
