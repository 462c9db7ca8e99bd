"""Sharded (ZeRO-style) AdamW over the dgn C-ABI, for torch CUDA tensors.

Mirrors the host side of the reference's ZeRO optimizer:

* ``ZeroReduceBucket.new`` groups parameters by dtype (float16, bfloat16,
  float32) and fills buckets of at most ``bucket_size`` bytes walking the
  parameters in inverse order (torch/core/optim/zero.py:40-62);
* ``ZeroAdamW.step`` runs one ``ZeroAdamW`` operator per bucket
  (torch/core/optim/zero.py:83-112): ``grad_scale`` is divided by the group
  size, per-parameter ``lr_scale`` attributes become ``lr_scales``, and an
  optional ``found_inf`` tensor collects the overflow verdict;
* the operator's own bookkeeping (dragon/operators/training/zero_update_op.h:
  101-118): the step count ``t`` advances on every run, skipped or not, and the
  kernel receives ``lr * sqrt(1 - beta2^t) / (1 - beta1^t)`` and
  ``lr * weight_decay``.

All device work is two kernels per bucket inside libdgn.so (dgn_zero_adamw);
torch provides memory and the stream.
"""

import ctypes
import math

import numpy as np
import torch

from dragon_b200 import _C
from dragon_b200.comm import _stream_ptr, dgn_dtype

_ZERO_DTYPES = (torch.float16, torch.bfloat16, torch.float32)


class ZeroReduceBucket(object):
    """Parameters that are reduced, updated and gathered as one message."""

    def __init__(self, params, dtype):
        self.params = list(params)
        self.dtype = dtype

    @property
    def size(self):
        """Bytes of the managed parameters."""
        return sum(p.numel() * p.element_size() for p in self.params)

    @classmethod
    def new(cls, params, bucket_size=536870912):
        """Buckets for `params`: one dtype per bucket, float16 first."""
        by_dtype = {}
        for p in params:
            by_dtype.setdefault(p.dtype, []).append(p)
        buckets = []
        for dtype in _ZERO_DTYPES:
            if by_dtype.get(dtype):
                buckets.extend(cls.new_with_dtype(by_dtype[dtype], dtype, bucket_size))
        return buckets

    @classmethod
    def new_with_dtype(cls, params, dtype, bucket_size=536870912):
        buckets, cur = [cls([], dtype)], 0
        for p in list(params)[::-1]:  # inverse order, as gradients become ready
            nxt = cur + p.numel() * p.element_size()
            if nxt > bucket_size and buckets[-1].params:
                buckets.append(cls([], dtype))
                cur, nxt = 0, p.numel() * p.element_size()
            buckets[-1].params.append(p)
            cur = nxt
        return buckets if len(params) > 0 else []


class _BucketState(object):
    """What one ZeroAdamW operator instance keeps for its bucket: the fp32
    master shard, both moments, the gradient scratch and the step count."""

    def __init__(self, comm, bucket, stream):
        lib = _C.lib()
        self.dtype = dgn_dtype(bucket.dtype)
        self.params = bucket.params
        n = len(self.params)
        self.counts = (ctypes.c_int64 * n)(*[p.numel() for p in self.params])
        self.total = sum(p.numel() for p in self.params)
        self.param_ptrs = (ctypes.c_void_p * n)(*[p.data_ptr() for p in self.params])
        count = lib.dgn_zero_state_count(comm.size, self.total, self.dtype)
        dev = self.params[0].device
        self.master = torch.zeros(count, dtype=torch.float32, device=dev)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.grad_shard = torch.empty_like(self.master)
        self.offset = lib.dgn_zero_state_offset(comm.rank, comm.size, self.total, self.dtype)
        self.shard = lib.dgn_zero_shard_count(comm.size, self.total)
        self.t = 0
        _C.check(lib.dgn_zero_init_master(comm._h, self.param_ptrs, self.counts, n, self.dtype,
                                          self.master.data_ptr(), _stream_ptr(stream, comm.device)))

    def view(self, name):
        """The reference's state tensor `name` (master, m or v): shard_count values."""
        return getattr(self, name)[self.offset:self.offset + self.shard]


class ZeroAdamW(object):
    """AdamW with optimizer state and the update sharded over the group.

    ``params`` are torch CUDA tensors whose ``.grad`` holds this rank's
    gradient.  The process group is ``comm`` (a dragon_b200.comm.Communicator)
    or ``group`` (a dragon_b200.distributed ProcessGroup); with neither, the
    default group of dragon_b200.distributed is taken, as the reference's
    ``step`` takes ``dist_backend.get_group()`` (torch/core/optim/zero.py:114-118).
    Keyword arguments and defaults follow the reference
    (torch/core/optim/adam.py:165-174, optimizer.py:56-59)."""

    def __init__(self, params, comm=None, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 grad_scale=1, clip_norm=0, clip_value=0, bucket_size=536870912, group=None):
        params = list(params)
        if len(params) == 0:
            raise ValueError("<params> is an empty sequence.")
        for p in params:
            if p.dtype not in _ZERO_DTYPES:
                raise TypeError("Unsupported data type: {}".format(p.dtype))
        if comm is None:
            from dragon_b200.distributed import backend as dist_backend
            group = group or dist_backend.get_group()
            if group is None:
                raise ValueError("<group> is required.")
            comm = dist_backend.communicator(group)
            if comm is None:
                raise ValueError("This rank is not a member of the group.")
        self.comm = comm
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.grad_scale, self.clip_norm, self.clip_value = grad_scale, clip_norm, clip_value
        self.buckets = ZeroReduceBucket.new(params, bucket_size)
        self._states = [None] * len(self.buckets)

    def state(self, bucket_index):
        return self._states[bucket_index]

    def kernel_args(self, t):
        """Hyper-parameters as the operator hands them to its kernel at step t."""
        f32 = np.float32
        beta1, beta2 = float(f32(self.betas[0])), float(f32(self.betas[1]))
        correction = f32(math.sqrt(1.0 - beta2 ** t) / (1.0 - beta1 ** t))
        lr = f32(self.lr)
        return _C.AdamWArgs(lr=float(lr * correction), beta1=beta1, beta2=beta2, eps=float(f32(self.eps)),
                            weight_decay=float(lr * f32(self.weight_decay)),
                            grad_scale=float(f32(self.grad_scale / self.comm.size)),
                            clip_norm=float(f32(self.clip_norm)), clip_value=float(f32(self.clip_value)))

    def step(self, found_inf=None, stream=None):
        """One update of every bucket.  `found_inf` (a one-element float32 CUDA
        tensor, or None) receives +1 per bucket whose reduced gradients hold a
        non-finite value on any rank; such a bucket is left unchanged."""
        lib = _C.lib()
        sp = _stream_ptr(stream, self.comm.device)
        for i, bucket in enumerate(self.buckets):  # master copies first: local work, no peer involved
            if self._states[i] is None:
                self._states[i] = _BucketState(self.comm, bucket, stream)
        for i, bucket in enumerate(self.buckets):
            st = self._states[i]
            grads = [p.grad for p in bucket.params]
            if any(g is None or g.dtype != bucket.dtype or not g.is_contiguous() for g in grads):
                raise ValueError("every parameter of a bucket needs a contiguous gradient of its own dtype")
            n = len(grads)
            grad_ptrs = (ctypes.c_void_p * n)(*[g.data_ptr() for g in grads])
            scales = [float(getattr(p, "lr_scale", 1)) for p in bucket.params]
            lrs = (ctypes.c_float * n)(*scales) if any(x != 1 for x in scales) else None
            st.t += 1
            args = self.kernel_args(st.t)
            _C.check(lib.dgn_zero_adamw(
                self.comm._h, grad_ptrs, st.param_ptrs, st.counts, n, st.dtype, st.master.data_ptr(),
                st.m.data_ptr(), st.v.data_ptr(), st.grad_shard.data_ptr(), lrs, ctypes.byref(args),
                found_inf.data_ptr() if found_inf is not None else None, sp))
