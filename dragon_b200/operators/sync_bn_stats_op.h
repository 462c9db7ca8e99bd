// The statistics exchange of synchronized batch normalization as an operator
// of its own: what BatchNormOp::RunTraining and the gradient operator do
// between computing their per-channel partial sums and using them
// (dragon/operators/normalization/batch_norm_op.cc:29-43 and :168-170):
//
//     int64_t N = N_;  coll_impl_.AllReduce(&N, &N, 1);             // host, blocking
//     coll_impl_.AllReduce(params, params, C_ * 2, ctx());          // device, 2C floats
//
// Arguments as BatchNormOp reads them (batch_norm_op.h:29-35): comm, group,
// ranks, backend; plus
//   batch_size       this rank's N
//   count_on_device  0: the reference's sequence -- the count goes through the
//                       host all-reduce (the run blocks until every rank has
//                       arrived), the 2C floats through the low-latency device
//                       kernel; Output(1), a one-element int64 HOST tensor,
//                       receives the global count.
//                    1: no host round trip -- Input(0) holds 2C + 1 floats, the
//                       last one float(batch_size); one device all-reduce (SUM)
//                       leaves the global count there (exact up to 2^24).
// Input(0) / Output(0): the float statistics, reduced in place.
#ifndef DRAGON_B200_OPERATORS_SYNC_BN_STATS_OP_H_
#define DRAGON_B200_OPERATORS_SYNC_BN_STATS_OP_H_

#include "collective_op_impl.h"
#include "dragon_shim.h"

namespace dragon {

template <class Context>
class SyncBNStatsOp final : public Operator<Context> {
 public:
  SyncBNStatsOp(const OperatorDef& def, Workspace* ws) : Operator<Context>(def, ws) {
    batch_size_ = OP_SINGLE_ARG(int64_t, "batch_size", 0);
    count_on_device_ = OP_SINGLE_ARG(int64_t, "count_on_device", 0);
    coll_impl_.SetBackend(OP_SINGLE_ARG(string, "backend", "MPI"));
    coll_impl_.SetReduction("SUM");
    coll_impl_.SetComm(OP_SINGLE_ARG(int64_t, "comm", 0), OP_SINGLE_ARG(int64_t, "group", 0),
                       OP_REPEATED_ARG(int64_t, "ranks"));
  }
  USE_OPERATOR_FUNCTIONS;

  void RunOnDevice() override;

 protected:
  CollectiveOpImpl coll_impl_;
  int64_t batch_size_ = 0, count_on_device_ = 0;
};

}  // namespace dragon

#endif  // DRAGON_B200_OPERATORS_SYNC_BN_STATS_OP_H_
