#include "sync_bn_stats_op.h"

namespace dragon {

template <class Context>
void SyncBNStatsOp<Context>::RunOnDevice() {
  Tensor* stats = Output(0);
  CHECK(Input(0).raw_data() == stats->raw_data()) << "\nThe statistics are reduced in place.";
  float* params = stats->template mutable_data<float, Context>();
  const int64_t count = stats->count();
  void* stream = this->ctx()->cuda_stream();
  if (count_on_device_ > 0) {
    CHECK(count >= 3 && (count - 1) % 2 == 0) << "\nExpected 2C + 1 floats, got " << count << ".";
    if (coll_impl_.comm_size() > 1) coll_impl_.AllReduce(params, params, count, stream);
    return;
  }
  CHECK(count >= 2 && count % 2 == 0) << "\nExpected 2C floats, got " << count << ".";
  int64_t N = batch_size_;
  if (coll_impl_.comm_size() > 1) {
    coll_impl_.AllReduce(&N, &N, 1);                      // batch_norm_op.cc:31, host, blocking
    coll_impl_.AllReduce(params, params, count, stream);  // batch_norm_op.cc:43, 2C floats
  }
  if (OutputSize() > 1) {
    Tensor* total = Output(1);
    CHECK(total->device_id() < 0) << "\nThe global count is a host tensor.";
    total->Reshape({1});
    *total->template mutable_data<int64_t, Context>() = N;
  }
}

template class SyncBNStatsOp<CUDAContext>;
REGISTER_CUDA_OPERATOR(SyncBNStats, SyncBNStatsOp<CUDAContext>);
OPERATOR_SCHEMA(SyncBNStats).AllowInplace([](int in, int out) -> bool { return in == 0 && out == 0; });

}  // namespace dragon
