/*
 * dgn.h -- C-ABI of the B200-native `Collective` path (ALLREDUCE SUM/MEAN,
 * ALLGATHER, BROADCAST, REDUCESCATTER over a process group).
 *
 * This is the boundary a Dragon build binds instead of its MPI / NCCL calls:
 * plain pointers, sizes and integer handles only.  Every entry point returns a
 * dgn_status; nothing aborts and nothing throws.  Device pointers are ordinary
 * CUDA device pointers valid on the communicator's device, `stream` is a
 * cudaStream_t passed as void*.  All collectives are asynchronous with respect
 * to the host: they enqueue their kernel on `stream` (one launch; two for the
 * sharded optimizer step) and return.
 *
 * Reference interfaces replaced (paths relative to the Dragon source tree):
 *   dragon/operators/distributed/collective_op_impl_mpi.cc:50-85   (MPI_Bcast /
 *       MPI_Allreduce / MPI_Reduce_scatter / MPI_Allgather call sites)
 *   dragon/operators/distributed/collective_op_impl_nccl.cc:34-67  (the four
 *       nccl* call sites) and :69-89 (unique-id broadcast + ncclCommInitRank)
 *   dragon/operators/distributed/collective_op.cc:7-51             (bucket
 *       concat/split copies and the per-tensor MEAN scale, both fused here)
 */
#ifndef DGN_H_
#define DGN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DGN_MAX_RANKS 8
#define DGN_HANDLE_BYTES 256

typedef struct dgn_comm* dgn_comm_t;

typedef enum {
  DGN_OK = 0,
  DGN_ERR_ARG = 1,      /* bad argument (null pointer, unknown dtype, ...) */
  DGN_ERR_CUDA = 2,     /* a CUDA runtime call failed; see dgn_last_error_string */
  DGN_ERR_TIMEOUT = 3,  /* a bounded device- or host-side wait ran out */
  DGN_ERR_PEER = 4,     /* a peer GPU is not reachable by P2P / IPC */
  DGN_ERR_STATE = 5,    /* call order violated (e.g. collective before connect) */
  DGN_ERR_UNSUPPORTED = 6
} dgn_status;

/* Element types: the `dtypes::Numerical` list the reference dispatches on
 * (dragon/core/types.h:69; dragon/operators/distributed/collective_op.cc:93). */
typedef enum {
  DGN_U8 = 0,
  DGN_I8 = 1,
  DGN_I32 = 2,
  DGN_I64 = 3,
  DGN_F16 = 4,
  DGN_BF16 = 5,
  DGN_F32 = 6,
  DGN_F64 = 7
} dgn_dtype;

/* Reductions.  SUM/PROD/MIN/MAX are the reference's op map
 * (collective_op_impl_mpi.cc:111-126).  MEAN is the operator-level
 * "SUM, then scale by 1.f/float(comm_size)" of collective_op.cc:40-51, fused
 * into the reduction epilogue; it is defined for floating-point types only. */
typedef enum {
  DGN_SUM = 0,
  DGN_MEAN = 1,
  DGN_PROD = 2,
  DGN_MIN = 3,
  DGN_MAX = 4
} dgn_redop;

/* Algorithm selector for dgn_comm_set_tuning / DGN_FORCE_VARIANT. */
typedef enum {
  DGN_VARIANT_AUTO = 0,
  DGN_VARIANT_ONESHOT = 1, /* every rank pushes its whole message to every peer */
  DGN_VARIANT_TWOSHOT = 2, /* reduce-scatter by peer stores + all-gather by peer loads */
  DGN_VARIANT_NVLS = 3,    /* staged through NVSwitch multicast (multimem): all-reduce ring, all-gather, broadcast */
  DGN_VARIANT_LL = 4,      /* one-shot with flag-in-data lines, no barrier (small messages) */
  DGN_VARIANT_LL2 = 5,     /* two-shot with flag-in-data lines (medium messages) */
  DGN_VARIANT_SYMM = 6,    /* NVSwitch multicast in place, on a buffer from dgn_comm_symm_alloc */
  DGN_VARIANT_RING = 7,    /* the same staged kernels with peer loads and stores (no switch needed; never chosen automatically) */
  DGN_VARIANT_RING_PULL = 8 /* all-gather only: staged, every rank loads the chunks from the sources' rings */
} dgn_variant;

/* ---- library ----------------------------------------------------------- */

/* Version as major*10000 + minor*100 + patch. */
int dgn_version(void);
/* Size in bytes of one element of `dtype`, or 0 if unknown. */
size_t dgn_dtype_size(int dtype);
/* Text of the last error raised on the calling thread. */
const char* dgn_last_error_string(void);
const char* dgn_status_string(int status);

/* ---- communicator bootstrap --------------------------------------------
 * Replaces "root creates an ncclUniqueId, MPI_Bcast, ncclCommInitRank"
 * (collective_op_impl_nccl.cc:69-89).  Three steps, so that the host
 * framework can move the handles with whatever byte channel it already has
 * (Dragon: MPI_Allgather on the group's MPI_Comm):
 *   1. dgn_comm_init_local   allocates this rank's symmetric workspace,
 *   2. dgn_comm_get_handle   fills DGN_HANDLE_BYTES describing it,
 *   3. dgn_comm_connect      takes all ranks' handles (rank order) and maps
 *                            every peer's workspace into this process.
 * `nranks` <= DGN_MAX_RANKS; `nranks` == 1 gives the local-copy path. */
int dgn_comm_init_local(int rank, int nranks, int device, dgn_comm_t* comm);
int dgn_comm_get_handle(dgn_comm_t comm, void* handle /* DGN_HANDLE_BYTES */);
int dgn_comm_connect(dgn_comm_t comm, const void* all_handles /* nranks * DGN_HANDLE_BYTES */);

/* Symmetric memory.  dgn_comm_init_symmetric is dgn_comm_init_local with an
 * arena of `symm_bytes` (environment DGN_SYMM_BYTES for the other bootstrap
 * calls) inside the memory that is bound to the communicator's NVSwitch
 * multicast object.  After dgn_comm_connect, dgn_comm_symm_alloc hands out
 * 256-byte aligned pieces of it; every rank must make the same sequence of
 * allocations, so that a buffer sits at the same offset on every rank.  An
 * all-reduce (SUM / MEAN; float32, float16, bfloat16) that runs in place on
 * such a buffer, over a whole number of 16-byte vectors, is done by the switch
 * on the buffers themselves -- nothing is staged and each rank moves about
 * S(1 + 1/n) bytes per direction instead of 2S(n-1)/n.  This is what NCCL
 * offers through ncclMemAlloc + buffer registration; Dragon would place its
 * "BufferShared" bucket tensor (collective_op.cc:19-21) there.  The arena
 * lives as long as the communicator; dgn_comm_symm_reset forgets all
 * allocations (the caller makes sure nothing uses them any more).  Where the
 * box exposes no multicast the capacity is 0 and dgn_comm_symm_alloc returns
 * DGN_ERR_UNSUPPORTED; ordinary device memory always works. */
int dgn_comm_init_symmetric(int rank, int nranks, int device, int64_t symm_bytes, dgn_comm_t* comm);
int64_t dgn_comm_symm_capacity(dgn_comm_t comm);
int dgn_comm_symm_alloc(dgn_comm_t comm, int64_t bytes, void** ptr);
int dgn_comm_symm_reset(dgn_comm_t comm);

/* Convenience bootstrap without any external channel: ranks meet through
 * files in `rendezvous_dir` (a directory all ranks of this node can write),
 * under the unique name `tag`.  Waits at most `timeout_ms` for the peers. */
int dgn_comm_create(int rank, int nranks, int device, const char* rendezvous_dir,
                    const char* tag, int timeout_ms, dgn_comm_t* comm);

/* `nranks` virtual ranks that all live on ONE device.  Each returned
 * communicator behaves like one rank; a collective is launched (as a single
 * cooperative kernel covering every virtual rank) when the last of the
 * `nranks` communicators has issued its call, so a single host thread may
 * call them one after another; calls queue per rank, so one rank may issue
 * several collectives before the others follow; the buffers of a queued call
 * must stay valid until the last rank has issued it.  All calls of one collective
 * must use the same stream.  Used to exercise the multi-rank kernels where fewer GPUs
 * than ranks are available. */
int dgn_comm_create_emulated(int nranks, int device, dgn_comm_t* comms /* [nranks] */);

/* The caller must make sure no peer still runs a collective on this
 * communicator (a host barrier after the last stream sync). */
int dgn_comm_destroy(dgn_comm_t comm);

int dgn_comm_rank(dgn_comm_t comm);
int dgn_comm_size(dgn_comm_t comm);
int dgn_comm_device(dgn_comm_t comm);

/* Error word written by kernels of this communicator: DGN_OK, or
 * DGN_ERR_TIMEOUT once a bounded device-side wait has run out.  Readable at
 * any time without synchronising.  A communicator that timed out refuses
 * further collectives with DGN_ERR_STATE. */
int dgn_comm_status(dgn_comm_t comm);

/* Upper bound, in milliseconds, on any single device-side wait for a peer
 * (default 5000; environment DGN_WAIT_LIMIT_MS). */
int dgn_comm_set_wait_limit_ms(dgn_comm_t comm, int ms);

/* Kernel-shape overrides (0 keeps the automatic choice): variant, number of
 * thread blocks, threads per block, bytes per block per round. */
int dgn_comm_set_tuning(dgn_comm_t comm, int variant, int blocks, int threads,
                        int64_t chunk_bytes);

/* Named launch parameters beyond dgn_comm_set_tuning (0 restores the automatic
 * choice): "flow_chunk_bytes", "flow_switch_blocks", "flow_in_blocks",
 * "flow_out_blocks", "flow_depth" shape the staged ring all-reduce;
 * "nvls_unroll" (1, 2, 4, 8 or 16) is the number of multimem loads a thread
 * keeps in flight and "nvls_pattern" (0 contiguous batches per warp, 1
 * grid-strided) how the in-place kernel deals its vectors; "nvls_min_bytes",
 * "symm_min_bytes", "nvls_bcast_min_bytes", "bcast_scatter_min_bytes" and
 * "allgather_pull_min_bytes", "nvls_allgather_min_bytes" move the size
 * thresholds of the corresponding variants; "gather_chunk_bytes",
 * "gather_push_blocks", "gather_forward_blocks" and "gather_mode" (1 the root
 * multicasts alone, 2 the root scatters and every rank multicasts its shard)
 * shape the staged all-gather / broadcast.  Every rank must set the same values.  An unknown name or a
 * negative value returns DGN_ERR_ARG. */
int dgn_comm_set_knob(dgn_comm_t comm, const char* name, int64_t value);

/* 1 if the NVSwitch-multicast variant was set up for this communicator. */
int dgn_comm_has_nvls(dgn_comm_t comm);

/* ---- collectives --------------------------------------------------------
 * Every rank of the communicator must issue the same sequence of
 * collectives with the same counts, dtype and reduction.  The kernels of one
 * communicator share its workspace and its device-resident protocol state, so
 * they must not overlap on the GPU: issue them on one stream, or order the
 * streams with events (dgn_allreduce_host waits for the latest collective
 * itself).  Different communicators are independent. */

/* ALLREDUCE over a list of tensors (replaces MPI_Allreduce /
 * ncclAllReduce at collective_op_impl_mpi.cc:60-66, _nccl.cc:43-50 together
 * with the bucket concat/split of collective_op.cc:7-35 and the MEAN scale of
 * collective_op.cc:40-51).  Tensor i has counts[i] elements; in_ptrs[i] may
 * equal out_ptrs[i] (in place).  The list is reduced as one message. */
int dgn_allreduce(dgn_comm_t comm, const void* const* in_ptrs, void* const* out_ptrs,
                  const int64_t* counts, int ntensors, int dtype, int redop, void* stream);

/* ALLGATHER: out holds nranks*count elements, rank r's block at r*count
 * (replaces MPI_Allgather / ncclAllGather, collective_op_impl_mpi.cc:79-85). */
int dgn_allgather(dgn_comm_t comm, const void* in, void* out, int64_t count, int dtype,
                  void* stream);

/* BROADCAST in place from group rank `root` (replaces MPI_Bcast /
 * ncclBroadcast, collective_op_impl_mpi.cc:50-57). */
int dgn_broadcast(dgn_comm_t comm, void* buf, int64_t count, int dtype, int root,
                  void* stream);

/* REDUCESCATTER: in holds nranks*count elements, out receives the reduced
 * block `rank` (replaces MPI_Reduce_scatter / ncclReduceScatter,
 * collective_op_impl_mpi.cc:69-76). */
int dgn_reducescatter(dgn_comm_t comm, const void* in, void* out, int64_t count, int dtype,
                      int redop, void* stream);

/* ALLREDUCE of a few values that live in HOST memory, synchronous: returns
 * when `out` holds the result (replaces the host overload
 * CollectiveOpImpl::AllReduce(x, y, N) -> MPI_Allreduce on host pointers,
 * collective_op_impl.h:91-94, which SyncBatchNorm uses for its batch count
 * and the ZeRO update for its overflow flag).  At most 4096 bytes.  The values
 * travel through the low-latency device kernel on a stream of the
 * communicator; collectives issued earlier on this communicator are waited
 * for first.  Not available on emulated communicators. */
int dgn_allreduce_host(dgn_comm_t comm, const void* in, void* out, int64_t count, int dtype, int redop);

/* ---- sharded (ZeRO-style) AdamW step --------------------------------------
 * One call replaces the body of the reference's ZeroAdamW operator for one
 * bucket (dragon/operators/training/zero_update_op_base.cc:103-143 with
 * adam_op.cc:48-81): concat copies, reduce-scatter, CheckFinite + host
 * all-reduce of the overflow flag, Cast, Scale, clip, AdamW on the fp32 master
 * shard, all-gather, split copies.  Here it is two kernels on `stream` and no
 * host synchronisation; gradients are read from, and parameters written to,
 * the tensors themselves.
 *
 * The bucket is the element-wise concatenation of its tensors, `total`
 * elements; rank r owns elements [r*rc, (r+1)*rc), rc = dgn_zero_shard_count
 * = ceil(total / nranks), the reference's partition
 * (zero_update_op_base.cc:24-31).  The fp32 state arrays of a rank (master, m,
 * v and the gradient scratch) hold dgn_zero_state_count floats each; element i
 * of the reference's state tensors lives at index dgn_zero_state_offset + i
 * (the arrays are aligned with the 16-byte vectors of the flat bucket, so up
 * to 16 / element size - 1 leading entries are padding).  All four must be
 * 16-byte aligned device pointers; m and v start as zeros. */
typedef struct {
  float lr;           /* step size the kernel applies: lr * sqrt(1 - beta2^t) / (1 - beta1^t) (adam_op.cc:52) */
  float beta1, beta2, eps;
  float weight_decay; /* decoupled decay the kernel applies: lr * weight_decay (adam_op.cc:56); <= 0: none */
  float grad_scale;   /* multiplies the reduced gradient (zero_update_op_base.cc:86-89); callers fold 1/nranks in */
  float clip_norm;    /* > 0: scale this rank's gradient shard down to that L2 norm (:90-95) */
  float clip_value;   /* > 0 and clip_norm <= 0: clamp gradients to [-clip_value, clip_value] (:96-99) */
} dgn_adamw_args;

int64_t dgn_zero_shard_count(int nranks, int64_t total);
int64_t dgn_zero_state_count(int nranks, int64_t total, int dtype);
int64_t dgn_zero_state_offset(int rank, int nranks, int64_t total, int dtype);

/* master <- fp32 copies of this rank's shard of the parameters (InitMaster,
 * zero_update_op_base.cc:21-44); padding entries become zero.  Local work. */
int dgn_zero_init_master(dgn_comm_t comm, const void* const* param_ptrs, const int64_t* counts,
                         int ntensors, int dtype, float* master, void* stream);

/* One AdamW step on the bucket.  dtype is DGN_F16, DGN_BF16 or DGN_F32; at
 * most 1024 non-empty tensors.  grad_shard is scratch of state_count floats.
 * lr_scales (host array, one per tensor, or NULL) are the per-parameter
 * learning-rate multipliers of the reference's `lr_scales` argument.
 * found_inf (device-visible float, or NULL) enables the overflow check: when
 * any rank's reduced shard holds a non-finite value, every rank adds 1 to
 * *found_inf and leaves master, m, v and the parameters untouched
 * (zero_update_op_base.cc:121-134); NULL skips the check, like an operator
 * without the extra output.  Every rank must pass the same hyper-parameters
 * and the same choice of found_inf / lr_scales. */
int dgn_zero_adamw(dgn_comm_t comm, const void* const* grad_ptrs, void* const* param_ptrs,
                   const int64_t* counts, int ntensors, int dtype, float* master, float* m, float* v,
                   float* grad_shard, const float* lr_scales, const dgn_adamw_args* args,
                   float* found_inf, void* stream);

/* ---- gradient all-reduce fused with the optimizer update -------------------
 * Data-parallel training without state sharding: every rank holds all
 * parameters and all optimizer state.  One call replaces, for one list of
 * float32 tensors, the reference's sequence "Collective ALLREDUCE SUM over the
 * gradients, then the update operator" (torch/core/optim/optimizer.py:134-164,
 * :250-272; operators/training/update_op_base.cc:21-38 for the gradient
 * transform; kernels/training/cuda/sgd_kernel.cu:10-51 and adam_kernel.cu:10-55
 * for the arithmetic).  It is ONE kernel: the two-shot all-reduce whose reduced
 * vectors go straight into the update of the parameter and state vectors at
 * the same position; the summed gradient is never written to memory and the
 * gradient tensors are left untouched.  Results are bit-identical on all ranks
 * and to the CPU restatement of the reference's loops. */
typedef enum {
  DGN_UPDATE_MOMENTUM_SGD = 0, /* m = momentum*m + g';  x -= lr*m           (g' = g + wd*x if wd > 0) */
  DGN_UPDATE_NESTEROV_SGD = 1, /* m = momentum*m + g';  x -= lr*(momentum*m + g') */
  DGN_UPDATE_ADAM = 2,         /* coupled decay: g' = g + wd*x */
  DGN_UPDATE_ADAMW = 3         /* decoupled decay: x -= wd*x + lr*m/(sqrt(v)+eps) */
} dgn_update_kind;

typedef struct {
  int kind;           /* dgn_update_kind */
  float lr;           /* as the kernel applies it (Adam kinds: lr * sqrt(1-beta2^t)/(1-beta1^t), adam_op.cc:52) */
  float momentum;     /* SGD kinds */
  float beta1, beta2, eps; /* Adam kinds */
  float weight_decay; /* as the kernel applies it (AdamW: lr * weight_decay, adam_op.cc:56); <= 0: none */
  float grad_scale;   /* multiplies the summed gradient; callers fold 1/nranks in (optimizer.py:261-262) */
  float clip_value;   /* > 0: clamp the scaled gradient to [-clip_value, clip_value]; clipping by norm is not fused */
} dgn_update_args;

/* Tensor i has counts[i] float32 elements in grad_ptrs[i], param_ptrs[i],
 * m_ptrs[i] and, for the Adam kinds, v_ptrs[i] (NULL otherwise).  At most 512
 * non-empty tensors per call.  dtype must be DGN_F32.  Every rank passes the
 * same hyper-parameters. */
int dgn_allreduce_update(dgn_comm_t comm, const void* const* grad_ptrs, void* const* param_ptrs,
                         void* const* m_ptrs, void* const* v_ptrs, const int64_t* counts, int ntensors,
                         int dtype, const dgn_update_args* args, void* stream);

/* ALLREDUCE of `nranks` buffers that all live on the CURRENT device, without
 * allocating anything.  (No counterpart in the reference: Dragon's collectives
 * always go through a communicator that owns library-allocated buffers.)
 *
 * For callers that must not call cudaMalloc -- a framework whose memory
 * planner already owns the whole device pool, a serving loop that cannot take
 * the allocator's device-wide synchronisation, a plug-in invoked where its
 * host forbids allocation.  Such callers cannot create a dgn communicator,
 * whose workspace is allocated; here the kernel's scratch memory is a fixed
 * 4,198,656-byte array inside the library image (each GPU that loads the
 * library holds it until the process exits).
 *
 * in_ptrs[r] / out_ptrs[r] (r < nranks <= 8) are device buffers of `count`
 * elements on the current device; every out buffer receives the reduction of
 * all in buffers (same order and rounding as dgn_allreduce); in_ptrs[r] may
 * equal out_ptrs[r].  Limit: count * element size <= 16384 bytes; larger
 * messages are rejected with DGN_ERR_ARG and a message.
 * The first call on a device looks up the array's device address; make that
 * call before any stream capture begins on that device.  The call enqueues a
 * memset of the scratch it uses and one kernel on `stream` and returns; it
 * calls no allocating routine.  All calls share the one array per device:
 * two calls whose work overlaps on the GPU (different streams, no ordering
 * between them) race and give undefined results -- order them.
 * DGN_OK from this call means "enqueued".  Should a block of the kernel give up
 * waiting (2 s; it cannot happen while the launch is intact, since all blocks
 * run in one cooperative grid), the outputs of that call are incomplete and an
 * error word in the array is set; nothing reports it by itself --
 * dgn_allreduce_static_status does. */
int dgn_allreduce_static(int nranks, const void* const* in_ptrs, void* const* out_ptrs,
                         int64_t count, int dtype, int redop, void* stream);

/* Error word of the static path on the CURRENT device (no counterpart in the
 * reference either): DGN_OK, or DGN_ERR_TIMEOUT if a block of any earlier
 * dgn_allreduce_static call on this device gave up.  The word stays set until
 * this function is called with clear != 0.  It copies 32 bytes back with a
 * blocking cudaMemcpy, so it also waits for the calls enqueued so far; it
 * allocates nothing. */
int dgn_allreduce_static_status(int clear);

/* ---- introspection for benchmarks and tests ------------------------------ */

/* The variant and launch shape the library would choose for one collective on a
 * communicator of `nranks` ranks (2..8) on GPUs with `num_sms` SMs, with or
 * without NVSwitch multicast, with a symmetric arena of `symm_bytes`, for a
 * buffer inside (in_symm != 0) or outside it; the environment knobs apply as
 * they do to a real communicator.  op: 0 ALLREDUCE, 1 REDUCESCATTER (count per
 * rank), 2 ALLGATHER (count per rank), 3 BROADCAST; the operation is taken to
 * be in place; ntensors > 1 describes a bucket.  Touches no device: tests and
 * documentation of the thresholds use it. */
int dgn_plan_query(int nranks, int num_sms, int has_nvls, int64_t symm_bytes, int in_symm, int op,
                   int dtype, int redop, int64_t count, int ntensors, int* variant, int* blocks,
                   int* threads, int64_t* chunk_bytes, int* rounds);

/* The same for the staged kernels (ar_flow_kernel, gather_flow_kernel), with
 * what the plan needs of the rings: op 0 ALLREDUCE (fp32 SUM), 2 ALLGATHER
 * (bytes per rank), 3 BROADCAST, one tensor of `bytes`.  `staged` is 0 when
 * another kernel serves the message (the other fields past chunk_vectors are
 * zero then).  A plan is memory-safe when ring_bytes_needed <=
 * ring_bytes_available, inbox_bytes_needed <= inbox_bytes_available, and at
 * least one block is left for every other role.  Touches no device. */
typedef struct dgn_staged_plan {
  int variant, blocks, threads, chunks;
  int64_t chunk_vectors;          /* 16-byte vectors per chunk (all-reduce) or per chunk and source */
  int staged;
  int depth;                      /* ring slots in use */
  int first_role_blocks;          /* reducing blocks (all-reduce), pushing blocks of a source (gather) */
  int second_role_blocks;         /* copy-in blocks (all-reduce), forwarding blocks (scattered broadcast) */
  int mode;                       /* gather: 1 scattered shards, 2 pulling */
  int64_t ring_bytes_needed, ring_bytes_available;
  int64_t inbox_bytes_needed, inbox_bytes_available, inbox_offset_in_half;
} dgn_staged_plan;
int dgn_plan_query_staged(int nranks, int num_sms, int has_nvls, int op, int64_t bytes,
                          dgn_staged_plan* out);

/* Number of kernels this library has launched from the calling process. */
int64_t dgn_launch_count(void);
/* Variant / grid the last collective of `comm` used (any pointer may be NULL). */
int dgn_comm_last_launch(dgn_comm_t comm, int* variant, int* blocks, int* threads,
                         int64_t* chunk_bytes, int* rounds);

#ifdef __cplusplus
}
#endif
#endif /* DGN_H_ */
