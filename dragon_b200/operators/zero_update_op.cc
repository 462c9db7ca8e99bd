// Operator body of `ZeroAdamW` for the CUDA context.
//
// What differs from dragon/operators/training/zero_update_op_base.cc:
//  * gradients are read from, and parameters written to, the tensors
//    themselves: there is no "BufferShared" send/receive buffer and no concat
//    or split copy (:73-83,118-119,141-142);
//  * the overflow verdict is agreed on the device, so the run neither reads
//    the flag back nor calls the host all-reduce (:121-131); the optional last
//    output is incremented by the kernel and must live in device memory;
//  * the state tensors are laid out on the 16-byte vectors of the flat bucket:
//    element i of the reference's "master" / "m" / "v" sits at index
//    dgn_zero_state_offset() + i.
#include "zero_update_op.h"

#include <cuda_runtime.h>

#include <cmath>
#include <string>

namespace dragon {

template <class Context>
template <typename T>
void ZeroUpdateOpBase<Context>::DoRunWithType() {
  GetArguments();
  const int n = InputSize();
  CHECK(OutputSize() >= n) << "\nEvery gradient needs its parameter as an output.";
  void* stream = this->ctx()->cuda_stream();
  const int dtype = DgnTypeOf<T>::value;
  vector<const void*> grads(n);
  vector<void*> params(n);
  vector<int64_t> counts(n);
  int64_t total = 0;
  for (int i = 0; i < n; ++i) {
    Tensor* P = Output(i);
    CHECK(Input(i).count() == P->count()) << "\nGradient " << i << " does not match its parameter.";
    grads[i] = Input(i).template data<T, Context>();
    params[i] = P->template mutable_data<T, Context>();
    counts[i] = P->count();
    total += counts[i];
  }
  Tensor* IsInfAll = OutputSize() > n ? Output(-1) : nullptr;
  const int64_t state_count = dgn_zero_state_count(coll_impl_.comm_size(), total, dtype);
  CHECK(state_count > 0) << "\nEmpty bucket.";

  // Master copies and moments: created on the first run, kept afterwards.
  Tensor* X = GetState("master");
  Tensor* M = GetState("m");
  Tensor* V = GetState("v");
  const bool fresh = X->raw_data() == nullptr;
  float* x = X->Reshape({state_count})->template mutable_data<float, Context>();
  float* m = M->Reshape({state_count})->template mutable_data<float, Context>();
  float* v = V->Reshape({state_count})->template mutable_data<float, Context>();
  if (fresh) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CHECK(cudaMemsetAsync(m, 0, sizeof(float) * state_count, s) == cudaSuccess) << "\nCUDA: memset failed.";
    CHECK(cudaMemsetAsync(v, 0, sizeof(float) * state_count, s) == cudaSuccess) << "\nCUDA: memset failed.";
    coll_impl_.ZeroInitMaster(params, counts, dtype, x, stream);
  }
  // The scratch tensor of the reference, "BufferKernel", is shared by all
  // operators of one device and stream, which run one after another there.
  // Virtual ranks of one device run inside ONE launch, so each rank gets its own.
  Tensor* dX = this->ctx()->workspace()->CreateTensor("BufferKernel:" + std::to_string(coll_impl_.comm_rank()));
  float* dx = dX->Reshape({state_count})->template mutable_data<float, Context>();

  dgn_adamw_args args = KernelArguments();
  args.grad_scale = grad_scale_;
  args.clip_norm = clip_norm_;
  args.clip_value = clip_value_;
  const float* lrs = nullptr;
  if (use_lr_scales_ > 0) {
    CHECK_EQ(static_cast<int>(lr_scales_.size()), n) << "\nBad number of <lr_scales>.";
    lrs = lr_scales_.data();
  }
  float* found_inf = IsInfAll ? IsInfAll->Reshape({1})->template mutable_data<float, Context>() : nullptr;
  coll_impl_.ZeroAdamW(grads, params, counts, dtype, x, m, v, dx, lrs, args, found_inf, stream);
}

template <class Context>
void ZeroAdamWOp<Context>::GetArguments() {
  lr_ = this->template GetHyper<float>("lr");
  beta1_ = this->template GetHyper<float>("beta1");
  beta2_ = this->template GetHyper<float>("beta2");
  eps_ = this->template GetHyper<float>("eps");
  t_++;
  correction_ = static_cast<float>(std::sqrt(1.f - std::pow(beta2_, t_)) / (1.f - std::pow(beta1_, t_)));
  ZeroUpdateOpBase<Context>::GetArguments();
}

template <class Context>
dgn_adamw_args ZeroAdamWOp<Context>::KernelArguments() {
  dgn_adamw_args a;
  a.lr = lr_ * correction_;
  a.beta1 = beta1_;
  a.beta2 = beta2_;
  a.eps = eps_;
  a.weight_decay = lr_ * this->weight_decay_;
  a.grad_scale = 1.f;
  a.clip_norm = 0.f;
  a.clip_value = 0.f;
  return a;
}

DEPLOY_CUDA_OPERATOR(ZeroAdamW);

OPERATOR_SCHEMA(ZeroAdamW).AllowInplace([](int, int) -> bool { return false; });

}  // namespace dragon
