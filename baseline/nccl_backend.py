"""The reference's NCCL backend, restated call for call, as a comparison baseline.

Dragon's NCCL path is: root creates an ncclUniqueId, the id is broadcast,
ncclCommInitRank, then one ncclAllReduce / ncclAllGather / ncclBroadcast per
tensor or bucket on the op's stream (collective_op_impl_nccl.cc:34-89), plus,
at the operator level, one `Scale` launch per tensor for MEAN and
cudaMemcpyAsync concat/split copies for buckets (collective_op.cc:7-51).
This module makes exactly those calls through ctypes on the NCCL library that
ships with torch.  It is used by bench.py only; the product never calls NCCL.
"""

import ctypes
import glob
import os

import torch

_NCCL_DTYPE = {
    torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6,
    torch.float32: 7, torch.float64: 8, torch.bfloat16: 9,
}
NCCL_SUM = 0


class _UniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


def _find_library():
    cands = []
    try:
        import nvidia.nccl
        for p in nvidia.nccl.__path__:
            cands += glob.glob(os.path.join(p, "lib", "libnccl.so*"))
    except ImportError:
        pass
    cands += glob.glob(os.path.join(os.path.dirname(torch.__file__), "lib", "libnccl.so*"))
    cands += ["libnccl.so.2"]
    for c in cands:
        try:
            return ctypes.CDLL(c)
        except OSError:
            continue
    raise RuntimeError("no NCCL library found")


class NcclBackend(object):
    """ncclCommInitRank + the collectives, on raw pointers and a raw stream."""

    def __init__(self, rank, nranks, exchange_bytes):
        """`exchange_bytes(payload_or_None) -> payload` broadcasts rank 0's bytes."""
        self.lib = _find_library()
        self.rank, self.nranks = rank, nranks
        uid = _UniqueId()
        if rank == 0:
            self._check(self.lib.ncclGetUniqueId(ctypes.byref(uid)))
            raw = exchange_bytes(bytes(bytearray(uid.internal)))
        else:
            raw = exchange_bytes(None)
        ctypes.memmove(ctypes.byref(uid), raw, 128)
        self.comm = ctypes.c_void_p()
        self.lib.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, _UniqueId, ctypes.c_int]
        self._check(self.lib.ncclCommInitRank(ctypes.byref(self.comm), nranks, uid, rank))
        self.lib.ncclAllReduce.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                           ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        self.lib.ncclAllGather.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                           ctypes.c_void_p, ctypes.c_void_p]
        self.lib.ncclBroadcast.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                           ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        self.lib.ncclReduceScatter.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        self.lib.ncclCommDestroy.argtypes = [ctypes.c_void_p]

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError("NCCL call failed with {}".format(rc))

    def version(self):
        v = ctypes.c_int()
        self.lib.ncclGetVersion(ctypes.byref(v))
        return v.value

    def all_reduce_sum(self, src, dst, stream):
        self._check(self.lib.ncclAllReduce(src.data_ptr(), dst.data_ptr(), src.numel(), _NCCL_DTYPE[src.dtype],
                                           NCCL_SUM, self.comm, ctypes.c_void_p(stream)))

    def all_gather(self, src, dst, stream):
        self._check(self.lib.ncclAllGather(src.data_ptr(), dst.data_ptr(), src.numel(), _NCCL_DTYPE[src.dtype],
                                           self.comm, ctypes.c_void_p(stream)))

    def broadcast(self, buf, root, stream):
        self._check(self.lib.ncclBroadcast(buf.data_ptr(), buf.data_ptr(), buf.numel(), _NCCL_DTYPE[buf.dtype],
                                           root, self.comm, ctypes.c_void_p(stream)))

    def operator_all_reduce(self, tensors, reduction, stream, bucket=None):
        """What the reference operator enqueues for ALLREDUCE on `tensors`.

        bucket=None: one ncclAllReduce per tensor (bucket_size 0).  Otherwise
        `bucket` is a flat scratch tensor: concat copies, one ncclAllReduce,
        split copies.  MEAN adds one scale launch per tensor, on the inputs."""
        if bucket is None:
            for t in tensors:
                self.all_reduce_sum(t, t, stream)
        else:
            off = 0
            for t in tensors:
                bucket[off:off + t.numel()].copy_(t.view(-1), non_blocking=True)
                off += t.numel()
            flat = bucket[:off]
            self.all_reduce_sum(flat, flat, stream)
            off = 0
            for t in tensors:
                t.view(-1).copy_(bucket[off:off + t.numel()], non_blocking=True)
                off += t.numel()
        if reduction.upper() == "MEAN":
            alpha = 1.0 / float(self.nranks)
            for t in tensors:
                t.mul_(alpha)

    def operator_all_reduce_sgd(self, grads, params, momenta, hyper, stream, bucket=None):
        """What the reference's data-parallel SGD step enqueues
        (torch/core/optim/optimizer.py:134-164, :250-272): the bucketed SUM
        all-reduce of the gradients, then the update operator -- one Scale per
        tensor for grad_scale / dist_size and the momentum kernel.  The update of
        all tensors is ONE fused multi-tensor call here, where the reference
        launches one kernel per tensor: in the baseline's favour."""
        self.operator_all_reduce(grads, "SUM", stream, bucket)
        torch._foreach_mul_(grads, hyper["grad_scale"])
        torch._fused_sgd_(params, grads, momenta, weight_decay=hyper["weight_decay"], momentum=hyper["momentum"],
                          lr=hyper["lr"], dampening=0.0, nesterov=False, maximize=False, is_first_step=False)

    def reduce_scatter_sum(self, src, dst, stream):
        self._check(self.lib.ncclReduceScatter(src.data_ptr(), dst.data_ptr(), dst.numel(), _NCCL_DTYPE[src.dtype],
                                               NCCL_SUM, self.comm, ctypes.c_void_p(stream)))

    def operator_zero_adamw(self, grads, params, state, hyper, stream, check_finite=True):
        """What the reference's ZeroAdamW operator enqueues for one bucket
        (zero_update_op_base.cc:103-143): concat copies into the send half of a
        flat buffer, ncclReduceScatter, CheckFinite with a device-to-host read
        of the flag (the host all-reduce of the flag that follows is left out,
        in the baseline's favour), Cast, Scale, one fused AdamW kernel on the
        fp32 master shard, a cast of the new values, ncclAllGather, split
        copies.  `state` holds flat (n*rc + rc elements), master, m, v, step
        (fp32 shard tensors; step is a 1-element fp32 tensor)."""
        rc = state["master"].numel()
        flat = state["flat"]
        recv, send = flat[:rc], flat[rc:]
        if check_finite:
            send.zero_()
        off = 0
        for g in grads:
            send[off:off + g.numel()].copy_(g.view(-1), non_blocking=True)
            off += g.numel()
        self.reduce_scatter_sum(send, recv, stream)
        if check_finite and not bool(torch.isfinite(recv).all().item()):
            return False
        dx = recv.float()
        dx.mul_(hyper["grad_scale"])
        torch._fused_adamw_([state["master"]], [dx], [state["m"]], [state["v"]], [], [state["step"]],
                            lr=hyper["lr"], beta1=hyper["beta1"], beta2=hyper["beta2"],
                            weight_decay=hyper["weight_decay"], eps=hyper["eps"], amsgrad=False, maximize=False)
        recv.copy_(state["master"])
        self.all_gather(recv, send, stream)
        off = 0
        for p in params:
            p.view(-1).copy_(send[off:off + p.numel()], non_blocking=True)
            off += p.numel()
        return True

    def destroy(self):
        if self.comm:
            self.lib.ncclCommDestroy(self.comm)
            self.comm = None
