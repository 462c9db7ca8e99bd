/* Stand-in for dragon/kernels/training/op_kernels.h (TEST INFRASTRUCTURE ONLY):
 * the primary templates that the reference's CPU optimizer files specialise
 * (dragon/kernels/training/op_kernels.h:28-101), and an empty CPUContext,
 * which those loops take but never touch. */
#ifndef ORACLE_REF_STUB_OP_KERNELS_H_
#define ORACLE_REF_STUB_OP_KERNELS_H_

#include "dragon/core/types.h"

namespace dragon {

class CPUContext {};

namespace kernels {

template <typename T, typename CopyT, class Context>
void Adam(const int N, const float lr, const float beta1, const float beta2, const float eps, const float wd,
          const T* x, const T* g, T* m, T* v, T* y, CopyT* y_copy, Context* ctx);

template <typename T, typename CopyT, class Context>
void AdamW(const int N, const float lr, const float beta1, const float beta2, const float eps, const float wd,
           const T* x, const T* g, T* m, T* v, T* y, CopyT* y_copy, Context* ctx);

template <typename T, typename CopyT, class Context>
void MomentumSGD(const int N, const float lr, const float momentum, const float wd, const T* x, const T* g, T* m,
                 T* y, CopyT* y_copy, Context* ctx);

template <typename T, typename CopyT, class Context>
void NesterovSGD(const int N, const float lr, const float momentum, const float wd, const T* x, const T* g, T* m,
                 T* y, CopyT* y_copy, Context* ctx);

}  // namespace kernels
}  // namespace dragon

#endif
