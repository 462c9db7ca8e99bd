// The `Collective` operator: ALLREDUCE / ALLGATHER / REDUCESCATTER / BROADCAST
// over a process group, with Dragon's argument names and defaults
// (dragon/operators/distributed/collective_op.h:21-54):
//   operation ""  reduction "SUM"  root 0  comm 0  group 0  backend "MPI"
//   ranks []  bucket_size 0
// `root` is read here; the reference declares it in its Python wrappers but
// drops it before the operator sees it.
#ifndef DRAGON_B200_OPERATORS_COLLECTIVE_OP_H_
#define DRAGON_B200_OPERATORS_COLLECTIVE_OP_H_

#include "collective_op_impl.h"
#include "dragon_shim.h"

namespace dragon {

template <class Context>
class CollectiveOp final : public Operator<Context> {
 public:
  CollectiveOp(const OperatorDef& def, Workspace* ws) : Operator<Context>(def, ws) { ReadArguments(); }
  USE_OPERATOR_FUNCTIONS;

  // One message per bucket of inputs (ALLREDUCE) or per input (everything else).
  void RunOnDevice() override;

  template <typename T>
  void DoRunWithType();

 protected:
  // Names and defaults of the reference's constructor.
  void ReadArguments() {
    operation_ = OP_SINGLE_ARG(string, "operation", "");
    reduction_ = OP_SINGLE_ARG(string, "reduction", "SUM");
    const bool buckets = operation_ == "ALLREDUCE";  // the other operations move one tensor per message
    bucket_size_ = buckets ? OP_SINGLE_ARG(int64_t, "bucket_size", 0) : 0;
    const int64_t root = OP_SINGLE_ARG(int64_t, "root", 0);
    coll_impl_.SetBackend(OP_SINGLE_ARG(string, "backend", "MPI"));
    coll_impl_.SetReduction(reduction_);
    coll_impl_.SetComm(OP_SINGLE_ARG(int64_t, "comm", 0), OP_SINGLE_ARG(int64_t, "group", 0),
                       OP_REPEATED_ARG(int64_t, "ranks"), root);
  }

  // Number of consecutive inputs, from src_index_, that travel as one message.
  int BucketLength(size_t elem_bytes);

  CollectiveOpImpl coll_impl_;
  string operation_, reduction_;
  int64_t bucket_size_ = 0;
  int src_index_ = 0;
};

}  // namespace dragon

#endif  // DRAGON_B200_OPERATORS_COLLECTIVE_OP_H_
