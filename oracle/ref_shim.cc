// C entry points over pieces of the reference that compile on their own
// (TEST INFRASTRUCTURE ONLY): the 16-bit float converters of
// dragon/utils/conversions.h:42-149 and the CPU optimizer loops of
// dragon/kernels/training/cpu/adam_kernel.cc:11-57 and sgd_kernel.cc:10-45.
// The Makefile beside this file compiles those reference sources where they
// lie, with oracle/ref_stub in front of the include path, into
// oracle/_ref/libdragon_ref.so; tests use it to pin the restatement in
// collective_oracle.c to the reference's own arithmetic.
#include <cstdint>

#include "dragon/kernels/training/op_kernels.h"
#include "dragon/utils/conversions.h"

using namespace dragon;

extern "C" {

void ref_f32_to_f16(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = convert::To<float16>(in[i]).x;
}
void ref_f16_to_f32(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    float16 h;
    h.x = in[i];
    out[i] = convert::To<float>(h);
  }
}
void ref_f32_to_bf16(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = convert::To<bfloat16>(in[i]).x;
}
void ref_bf16_to_f32(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    bfloat16 h;
    h.x = in[i];
    out[i] = convert::To<float>(h);
  }
}

// copy_kind: 0 none, 1 float16, 2 bfloat16 (the y_copy output of the loops).
static CPUContext g_ctx;

void ref_adamw(int n, float lr, float beta1, float beta2, float eps, float wd, const float* x, const float* g,
               float* m, float* v, float* y, uint16_t* y_copy, int copy_kind) {
  if (copy_kind == 2)
    kernels::AdamW<float, bfloat16, CPUContext>(n, lr, beta1, beta2, eps, wd, x, g, m, v, y,
                                                reinterpret_cast<bfloat16*>(y_copy), &g_ctx);
  else
    kernels::AdamW<float, float16, CPUContext>(n, lr, beta1, beta2, eps, wd, x, g, m, v, y,
                                               copy_kind == 1 ? reinterpret_cast<float16*>(y_copy) : nullptr, &g_ctx);
}

void ref_adam(int n, float lr, float beta1, float beta2, float eps, float wd, const float* x, const float* g,
              float* m, float* v, float* y, uint16_t* y_copy, int copy_kind) {
  if (copy_kind == 2)
    kernels::Adam<float, bfloat16, CPUContext>(n, lr, beta1, beta2, eps, wd, x, g, m, v, y,
                                               reinterpret_cast<bfloat16*>(y_copy), &g_ctx);
  else
    kernels::Adam<float, float16, CPUContext>(n, lr, beta1, beta2, eps, wd, x, g, m, v, y,
                                              copy_kind == 1 ? reinterpret_cast<float16*>(y_copy) : nullptr, &g_ctx);
}

void ref_momentum_sgd(int n, float lr, float momentum, float wd, const float* x, const float* g, float* m, float* y,
                      uint16_t* y_copy, int copy_kind, int nesterov) {
  float16* hc = copy_kind == 1 ? reinterpret_cast<float16*>(y_copy) : nullptr;
  bfloat16* bc = reinterpret_cast<bfloat16*>(y_copy);
  if (nesterov) {
    if (copy_kind == 2) kernels::NesterovSGD<float, bfloat16, CPUContext>(n, lr, momentum, wd, x, g, m, y, bc, &g_ctx);
    else kernels::NesterovSGD<float, float16, CPUContext>(n, lr, momentum, wd, x, g, m, y, hc, &g_ctx);
  } else {
    if (copy_kind == 2) kernels::MomentumSGD<float, bfloat16, CPUContext>(n, lr, momentum, wd, x, g, m, y, bc, &g_ctx);
    else kernels::MomentumSGD<float, float16, CPUContext>(n, lr, momentum, wd, x, g, m, y, hc, &g_ctx);
  }
}

}  // extern "C"
