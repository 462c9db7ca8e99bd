// Instantiations of the sharded-optimizer kernels for the three element types
// the reference's ZeRO update accepts (float16, bfloat16, float32:
// dragon/operators/training/zero_update_op.h:83-96).
#include "../../include/dgn.h"
#include "dgn_zero.cuh"

namespace dgn {

// which: 0 reduce-scatter into the gradient shard, 1 update + all-gather,
//        2 master initialisation.
template <typename T>
static const void* zero_kernels_of(int which) {
  switch (which) {
    case 0: return (const void*)zero_reduce_kernel<T>;
    case 1: return (const void*)zero_update_kernel<T>;
    case 2: return (const void*)zero_init_master_kernel<T>;
    default: return nullptr;
  }
}

const void* zero_kernel_fn(int dtype, int which) {
  switch (dtype) {
    case DGN_F16: return zero_kernels_of<__half>(which);
    case DGN_BF16: return zero_kernels_of<__nv_bfloat16>(which);
    case DGN_F32: return zero_kernels_of<float>(which);
    default: return nullptr;
  }
}

}  // namespace dgn
