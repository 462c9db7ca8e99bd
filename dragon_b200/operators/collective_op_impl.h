// CollectiveOpImpl over the dgn C-ABI: the place where Dragon's
// CollectiveOpImpl (dragon/operators/distributed/collective_op_impl.h:22-158)
// switches between MPI_* and nccl* library calls.  Here every method is one
// call into libdgn.so, which launches one hand-written kernel on the stream.
#ifndef DRAGON_B200_OPERATORS_COLLECTIVE_OP_IMPL_H_
#define DRAGON_B200_OPERATORS_COLLECTIVE_OP_IMPL_H_

#include "dgn.h"
#include "dragon_shim.h"

namespace dragon {

template <typename T> struct DgnTypeOf;
template <> struct DgnTypeOf<uint8_t> { static constexpr int value = DGN_U8; };
template <> struct DgnTypeOf<int8_t> { static constexpr int value = DGN_I8; };
template <> struct DgnTypeOf<int> { static constexpr int value = DGN_I32; };
template <> struct DgnTypeOf<int64_t> { static constexpr int value = DGN_I64; };
template <> struct DgnTypeOf<float16> { static constexpr int value = DGN_F16; };
template <> struct DgnTypeOf<bfloat16> { static constexpr int value = DGN_BF16; };
template <> struct DgnTypeOf<float> { static constexpr int value = DGN_F32; };
template <> struct DgnTypeOf<double> { static constexpr int value = DGN_F64; };

// A failed dgn call is fatal at the operator boundary, as MPI_CHECK /
// NCCL_CHECK are in the reference (utils/device/common_nccl.h:22-26).
#define DGN_CHECK(expr)                                                               \
  do {                                                                                \
    int rc__ = (expr);                                                                \
    CHECK(rc__ == DGN_OK) << "\nDGN: " << dgn_status_string(rc__) << ": " << dgn_last_error_string(); \
  } while (0)

class CollectiveOpImpl {
 public:
  explicit CollectiveOpImpl(const string& backend = "MPI") : backend_(backend) {}

  void SetBackend(const string& backend) { backend_ = backend; }

  // SUM / PROD / MIN / MAX as in the reference's maps
  // (collective_op_impl_mpi.cc:111-126) plus MEAN, which the maps lack
  // although the operator and its callers use it.
  void SetReduction(const string& reduction) {
    if (reduction == "SUM") redop_ = DGN_SUM;
    else if (reduction == "MEAN") redop_ = DGN_MEAN;
    else if (reduction == "PROD") redop_ = DGN_PROD;
    else if (reduction == "MIN") redop_ = DGN_MIN;
    else if (reduction == "MAX") redop_ = DGN_MAX;
    else DRAGON_FATAL << "Unsupported reduction: " << reduction;
  }

  // `comm` carries the dgn communicator handle where the reference carries an
  // MPI_Comm pointer (modules/python/mpi.h:110); 0 means "no group" and leaves
  // comm_size() at 0, which turns the operator into a no-op
  // (collective_op_impl_mpi.cc:10, collective_op.cc:89).  `root` is an index
  // into the group, i.e. already a group rank.
  void SetComm(const int64_t comm, const int64_t group, const vec64_t ranks, const int64_t root = 0) {
    if (comm == 0) return;
    CHECK(group != 0) << "\nSet comm from an invalid group.";
    comm_ = reinterpret_cast<dgn_comm_t>(static_cast<intptr_t>(comm));
    comm_size_ = dgn_comm_size(comm_);
    comm_rank_ = dgn_comm_rank(comm_);
    CHECK(comm_size_ >= 1) << "\nInvalid communicator handle.";
    CHECK(ranks.empty() || static_cast<int>(ranks.size()) == comm_size_)
        << "\nGroup has " << ranks.size() << " ranks, communicator has " << comm_size_ << ".";
    CHECK(root >= 0 && root < comm_size_) << "\nComm root is not in the group.";
    comm_root_ = static_cast<int>(root);
  }

  template <typename T>
  void Broadcast(const T* x, T* y, int64_t N, void* stream) {
    CHECK(x == y) << "\nUnsupported non-inplace broadcast.";
    DGN_CHECK(dgn_broadcast(comm_, y, N, DgnTypeOf<T>::value, comm_root_, stream));
  }

  // Host pointers, synchronous: the overload SyncBatchNorm and the ZeRO update
  // call for a count or a flag (collective_op_impl.h:91-94 in the reference).
  template <typename T>
  void AllReduce(const T* x, T* y, int64_t N) {
    DGN_CHECK(dgn_allreduce_host(comm_, x, y, N, DgnTypeOf<T>::value, redop_));
  }

  template <typename T>
  void AllReduce(const T* x, T* y, int64_t N, void* stream) {
    const void* in[1] = {x};
    void* out[1] = {y};
    int64_t n[1] = {N};
    DGN_CHECK(dgn_allreduce(comm_, in, out, n, 1, DgnTypeOf<T>::value, redop_, stream));
  }

  // A bucket of tensors as one message: no concat / split copies.
  template <typename T>
  void AllReduce(const vector<const void*>& x, const vector<void*>& y, const vector<int64_t>& N, void* stream) {
    DGN_CHECK(dgn_allreduce(comm_, x.data(), y.data(), N.data(), static_cast<int>(N.size()),
                            DgnTypeOf<T>::value, redop_, stream));
  }

  template <typename T>
  void ReduceScatter(const T* x, T* y, int64_t N, void* stream) {
    DGN_CHECK(dgn_reducescatter(comm_, x, y, N, DgnTypeOf<T>::value, redop_, stream));
  }

  template <typename T>
  void AllGather(const T* x, T* y, int64_t N, void* stream) {
    DGN_CHECK(dgn_allgather(comm_, x, y, N, DgnTypeOf<T>::value, stream));
  }

  // The sharded AdamW step of one bucket (the body of the reference's
  // ZeroUpdateOpBase::DoRunWithType, zero_update_op_base.cc:103-143, which
  // issues ReduceScatter and AllGather around its update kernels).
  void ZeroInitMaster(const vector<void*>& params, const vector<int64_t>& N, int dtype, float* master, void* stream) {
    DGN_CHECK(dgn_zero_init_master(comm_, const_cast<const void* const*>(params.data()), N.data(),
                                   static_cast<int>(N.size()), dtype, master, stream));
  }
  void ZeroAdamW(const vector<const void*>& grads, const vector<void*>& params, const vector<int64_t>& N, int dtype,
                 float* master, float* m, float* v, float* grad_shard, const float* lr_scales,
                 const dgn_adamw_args& args, float* found_inf, void* stream) {
    DGN_CHECK(dgn_zero_adamw(comm_, grads.data(), params.data(), N.data(), static_cast<int>(N.size()), dtype,
                             master, m, v, grad_shard, lr_scales, &args, found_inf, stream));
  }

  int comm_rank() const { return comm_rank_; }
  int comm_size() const { return comm_size_; }
  int comm_root() const { return comm_root_; }
  const string& backend() const { return backend_; }

 private:
  string backend_;
  dgn_comm_t comm_ = nullptr;
  int comm_rank_ = 0, comm_size_ = 0, comm_root_ = 0, redop_ = DGN_SUM;
};

}  // namespace dragon

#endif  // DRAGON_B200_OPERATORS_COLLECTIVE_OP_IMPL_H_
