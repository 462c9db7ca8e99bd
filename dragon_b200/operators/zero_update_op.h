// The `ZeroAdamW` operator: AdamW with the optimizer state and the update
// sharded over the process group, with Dragon's argument names, hyper tensors
// and state tensors (dragon/operators/training/zero_update_op.h:20-125):
//   arguments   bucket_name ""  use_lr_scales 0  lr_scales []  weight_decay -1
//               backend "MPI"  comm 0  group 0  ranks []
//   hyper       host tensors "<name>/lr", "/beta1", "/beta2", "/eps",
//               "/grad_scale", "/clip_norm", "/clip_value" and, unless the
//               argument is given, "/weight_decay"
//   state       "<name>/<bucket_name>/master", "/m", "/v" (fp32)
//   inputs      the gradients of the bucket; outputs: its parameters, plus an
//               optional last float output that counts overflowed steps
// The body of the reference (zero_update_op_base.cc:103-143) -- concat copies,
// ReduceScatter, CheckFinite with a host all-reduce, Cast, Scale, clip, the
// AdamW kernel, AllGather, split copies -- is one dgn_zero_adamw call here.
#ifndef DRAGON_B200_OPERATORS_ZERO_UPDATE_OP_H_
#define DRAGON_B200_OPERATORS_ZERO_UPDATE_OP_H_

#include "collective_op_impl.h"
#include "dragon_shim.h"

namespace dragon {

template <class Context>
class ZeroUpdateOpBase : public Operator<Context> {
 public:
  ZeroUpdateOpBase(const OperatorDef& def, Workspace* ws) : Operator<Context>(def, ws) {
    bucket_name_ = OP_SINGLE_ARG(string, "bucket_name", "");
    lr_scales_ = OP_REPEATED_ARG(float, "lr_scales");
    use_lr_scales_ = OP_SINGLE_ARG(int64_t, "use_lr_scales", 0);
    coll_impl_.SetBackend(OP_SINGLE_ARG(string, "backend", "MPI"));
    coll_impl_.SetComm(OP_SINGLE_ARG(int64_t, "comm", 0), OP_SINGLE_ARG(int64_t, "group", 0),
                       OP_REPEATED_ARG(int64_t, "ranks"));
  }
  USE_OPERATOR_FUNCTIONS;

  // float16 / bfloat16 / float32 gradients (float64 is refused by the library).
  void RunOnDevice() override { DispatchHelper<dtypes::Floating>::Call(this, Input(0)); }

  template <typename T>
  void DoRunWithType();

 protected:
  // A hyper-parameter: the first element of the host tensor "<name>/<key>".
  template <typename T>
  T GetHyper(const string& key) {
    const Tensor* h = this->workspace()->GetTensor(this->name() + "/" + key);
    return h->template data<T, CPUContext>()[0];
  }

  // A state tensor of this bucket: "<name>/<bucket_name>/<key>".
  Tensor* GetState(const string& key) {
    return this->workspace()->CreateTensor(this->name() + "/" + bucket_name_ + "/" + key);
  }

  // Gradient transform and decay; the `weight_decay` argument, if given, wins over the hyper tensor.
  virtual void GetArguments() {
    const float wd_arg = OP_SINGLE_ARG(float, "weight_decay", -1.f);
    weight_decay_ = wd_arg < 0.f ? GetHyper<float>("weight_decay") : wd_arg;
    grad_scale_ = GetHyper<float>("grad_scale");
    clip_norm_ = GetHyper<float>("clip_norm");
    clip_value_ = GetHyper<float>("clip_value");
  }

  // What the update kernel receives; the gradient transform is filled in by the base.
  virtual dgn_adamw_args KernelArguments() = 0;

  CollectiveOpImpl coll_impl_;
  string bucket_name_;
  vector<float> lr_scales_;
  int64_t use_lr_scales_ = 0;
  float grad_scale_ = 1.f, weight_decay_ = 0.f, clip_norm_ = 0.f, clip_value_ = 0.f;
};

template <class Context>
class ZeroAdamWOp final : public ZeroUpdateOpBase<Context> {
 public:
  ZeroAdamWOp(const OperatorDef& def, Workspace* ws) : ZeroUpdateOpBase<Context>(def, ws), t_(0) {}

  // The step count advances on every run, skipped or not, and the kernel
  // takes lr * correction and lr * weight_decay (zero_update_op.h:108-116,
  // adam_op.cc:52,56).
  void GetArguments() override;
  dgn_adamw_args KernelArguments() override;

 protected:
  int64_t t_;
  float lr_ = 0.f, beta1_ = 0.f, beta2_ = 0.f, eps_ = 0.f, correction_ = 1.f;
};

}  // namespace dragon

#endif  // DRAGON_B200_OPERATORS_ZERO_UPDATE_OP_H_
