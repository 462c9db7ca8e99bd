// Operator body of `Collective` for the CUDA context.
//
// What differs from dragon/operators/distributed/collective_op.cc:
//  * a bucket is handed to the collective as a tensor list; there is no
//    "BufferShared" scratch tensor and no concat / split copy (:7-35);
//  * the MEAN scale is part of the reduction kernel; the second loop over the
//    inputs with one Scale launch per tensor (:95-100) is gone;
//  * buckets are closed BEFORE the tensor that would overflow them and a
//    tensor larger than bucket_size is a bucket of its own (the reference
//    includes the overflowing tensor and never advances past an oversize
//    first tensor).
#include "collective_op.h"

#include <cuda_runtime.h>

namespace dragon {

template <class Context>
int CollectiveOp<Context>::BucketLength(size_t elem_bytes) {
  if (bucket_size_ <= 0) return 1;
  const DType dtype = Input(src_index_).dtype();
  int64_t bytes = 0;
  int n = 0;
  for (; src_index_ + n < InputSize(); ++n) {
    const Tensor& X = Input(src_index_ + n);
    if (X.dtype() != dtype) break;  // one element type per message
    const int64_t b = X.count() * static_cast<int64_t>(elem_bytes);
    if (n > 0 && bytes + b > bucket_size_) break;
    bytes += b;
  }
  return n;
}

template <class Context>
template <typename T>
void CollectiveOp<Context>::DoRunWithType() {
  void* stream = this->ctx()->cuda_stream();
  Tensor& X = Input(src_index_);
  if (operation_ == "ALLREDUCE") {
    const int n = BucketLength(sizeof(T));
    vector<const void*> src(n);
    vector<void*> dest(n);
    vector<int64_t> counts(n);
    for (int i = 0; i < n; ++i) {
      Tensor& Xi = Input(src_index_ + i);
      Tensor* Yi = Output(src_index_ + i);
      src[i] = Xi.template data<T, Context>();
      dest[i] = Yi->ReshapeLike(Xi)->template mutable_data<T, Context>();
      counts[i] = Xi.count();
    }
    coll_impl_.AllReduce<T>(src, dest, counts, stream);
    src_index_ += n;
    return;
  }
  Tensor* Y = Output(src_index_);
  if (operation_ == "ALLGATHER") {
    auto dest_dims = X.dims();
    dest_dims.insert(dest_dims.begin(), coll_impl_.comm_size());
    const T* x = X.template data<T, Context>();
    coll_impl_.AllGather(x, Y->Reshape(dest_dims)->template mutable_data<T, Context>(), X.count(), stream);
  } else if (operation_ == "REDUCESCATTER") {
    auto dest_dims = X.dims();
    CHECK(!dest_dims.empty() && dest_dims[0] % coll_impl_.comm_size() == 0)
        << "\nThe first dimension must be divisible by the group size.";
    dest_dims[0] /= coll_impl_.comm_size();
    const T* x = X.template data<T, Context>();
    const int64_t count = X.count() / coll_impl_.comm_size();
    coll_impl_.ReduceScatter(x, Y->Reshape(dest_dims)->template mutable_data<T, Context>(), count, stream);
  } else if (operation_ == "BROADCAST") {
    const T* x = X.template data<T, Context>();
    T* y = Y->ReshapeLike(X)->template mutable_data<T, Context>();
    if (x != y && coll_impl_.comm_rank() == coll_impl_.comm_root()) {
      // Out of place: the root's value starts in the output, then travels in place.
      cudaError_t e = cudaMemcpyAsync(y, x, X.nbytes(), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
      CHECK(e == cudaSuccess) << "\nCUDA: " << cudaGetErrorString(e);
    }
    coll_impl_.Broadcast(y, y, X.count(), stream);
  } else {
    DRAGON_FATAL << "Unsupported operation: " << operation_;
  }
  src_index_ += 1;
}

template <class Context>
void CollectiveOp<Context>::RunOnDevice() {
  if (coll_impl_.comm_size() <= 1) return;  // nothing to exchange, outputs untouched
  for (src_index_ = 0; src_index_ < InputSize();) {
    DispatchHelper<dtypes::Numerical>::Call(this, Input(src_index_));
  }
}

DEPLOY_CUDA_OPERATOR(Collective);

OPERATOR_SCHEMA(Collective).AllowInplace([](int, int) -> bool { return true; });

}  // namespace dragon
