"""Data-parallel SGD / Adam / AdamW whose gradient all-reduce and update are
one kernel (dgn_allreduce_update), for torch CUDA tensors.

Mirrors the torch frontend's optimizers where they meet the process group
(torch/core/optim/optimizer.py:134-164 and :250-272): gradients of one dtype
are all-reduced with SUM, then the update operator runs with
``grad_scale / dist_size``.  The update operators' own bookkeeping is kept:
the Adam kinds advance a step count and hand the kernel
``lr * sqrt(1 - beta2^t) / (1 - beta1^t)`` (operators/training/update_op.h:160-163),
AdamW hands it ``lr * weight_decay`` (adam_op.cc:30-36).  State tensors ``m``
and ``v`` start at zero.  float32 parameters only; clipping by norm is not fused
(the reference computes the norm of the summed gradient of each tensor between
the collective and the kernel).
"""

import ctypes
import math

import numpy as np
import torch

from dragon_b200 import _C
from dragon_b200.comm import _stream_ptr

_MAX_TENSORS = 512  # per call of dgn_allreduce_update


class _FusedOptimizer(object):
    def __init__(self, params, comm, group, grad_scale, clip_value, two_states):
        params = list(params)
        if len(params) == 0:
            raise ValueError("<params> is an empty sequence.")
        for p in params:
            if p.dtype != torch.float32:
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
        self.params = params
        self.grad_scale, self.clip_value = grad_scale, clip_value
        self.m = [torch.zeros_like(p) for p in params]
        self.v = [torch.zeros_like(p) for p in params] if two_states else None
        self.t = 0

    def kernel_args(self, t):  # pragma: no cover - overridden
        raise NotImplementedError

    def step(self, stream=None):
        """One fused all-reduce + update of every parameter that has a gradient."""
        idx = [i for i, p in enumerate(self.params) if p.grad is not None]
        for i in idx:
            g = self.params[i].grad
            if g.dtype != torch.float32 or not g.is_contiguous() or g.numel() != self.params[i].numel():
                raise ValueError("every parameter needs a contiguous float32 gradient of its own size")
        self.t += 1
        args = self.kernel_args(self.t)
        lib = _C.lib()
        sp = _stream_ptr(stream, self.comm.device)
        for lo in range(0, len(idx), _MAX_TENSORS):
            part = idx[lo:lo + _MAX_TENSORS]
            n = len(part)
            ptrs = lambda ts: (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])  # noqa: E731
            grads = ptrs([self.params[i].grad for i in part])
            params = ptrs([self.params[i] for i in part])
            m = ptrs([self.m[i] for i in part])
            v = ptrs([self.v[i] for i in part]) if self.v is not None else None
            counts = (ctypes.c_int64 * n)(*[self.params[i].numel() for i in part])
            _C.check(lib.dgn_allreduce_update(self.comm._h, grads, params, m, v, counts, n, _C.F32,
                                              ctypes.byref(args), sp))


class FusedSGD(_FusedOptimizer):
    """SGD with momentum, plain or Nesterov (torch/core/optim/sgd.py:60-95)."""

    def __init__(self, params, lr, momentum=0, weight_decay=0, nesterov=False, comm=None, group=None,
                 grad_scale=1, clip_value=0):
        if lr < 0:
            raise ValueError("Invalid learning rate: {}".format(lr))
        if momentum < 0:
            raise ValueError("Invalid momentum: {}".format(momentum))
        if nesterov and momentum <= 0:
            raise ValueError("Nesterov momentum requires a momentum and zero dampening.")
        super(FusedSGD, self).__init__(params, comm, group, grad_scale, clip_value, two_states=False)
        self.lr, self.momentum, self.weight_decay, self.nesterov = lr, momentum, weight_decay, nesterov

    def kernel_args(self, t):
        f32 = np.float32
        return _C.UpdateArgs(kind=_C.UPDATE_NESTEROV_SGD if self.nesterov else _C.UPDATE_MOMENTUM_SGD,
                             lr=float(f32(self.lr)), momentum=float(f32(self.momentum)), beta1=0.0, beta2=0.0,
                             eps=0.0, weight_decay=float(f32(self.weight_decay)),
                             grad_scale=float(f32(self.grad_scale / self.comm.size)),
                             clip_value=float(f32(self.clip_value)))


class FusedAdam(_FusedOptimizer):
    """Adam with coupled weight decay (torch/core/optim/adam.py:40-86)."""

    _kind = _C.UPDATE_ADAM

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, comm=None, group=None,
                 grad_scale=1, clip_value=0):
        if not 0 <= lr:
            raise ValueError("Invalid learning rate: {}".format(lr))
        if not 0 <= eps:
            raise ValueError("Invalid epsilon: {}".format(eps))
        if not 0 <= betas[0] < 1:
            raise ValueError("Invalid beta1: {}".format(betas[0]))
        if not 0 <= betas[1] < 1:
            raise ValueError("Invalid beta2: {}".format(betas[1]))
        super(FusedAdam, self).__init__(params, comm, group, grad_scale, clip_value, two_states=True)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay

    def kernel_args(self, t):
        f32 = np.float32
        beta1, beta2 = float(f32(self.betas[0])), float(f32(self.betas[1]))
        correction = f32(math.sqrt(1.0 - beta2 ** t) / (1.0 - beta1 ** t))
        lr = f32(self.lr)
        wd = f32(self.weight_decay) if self._kind == _C.UPDATE_ADAM else lr * f32(self.weight_decay)
        return _C.UpdateArgs(kind=self._kind, lr=float(lr * correction), momentum=0.0, beta1=beta1, beta2=beta2,
                             eps=float(f32(self.eps)), weight_decay=float(wd),
                             grad_scale=float(f32(self.grad_scale / self.comm.size)),
                             clip_value=float(f32(self.clip_value)))


class FusedAdamW(FusedAdam):
    """AdamW, decoupled weight decay (torch/core/optim/adam.py:89-130)."""

    _kind = _C.UPDATE_ADAMW

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, **kwargs):
        super(FusedAdamW, self).__init__(params, lr, betas, eps, weight_decay, **kwargs)
