"""dragon.distributed collective functions on torch CUDA tensors.

Signatures, defaults and error behaviour of
dragon/python/core/ops/distributed_ops.py:24-147: exactly one input tensor,
``reduction`` is a case-insensitive string, a missing group (argument and
default both None) raises ``ValueError("<group> is required.")``, and in eager
mode the result is a new tensor.  Each call becomes one `Collective` operator
run in the C++ operator layer.
"""

import torch

from dragon_b200 import op_lib
from dragon_b200.distributed import backend as dist_backend


def _resolve(group):
    if group is None:
        group = dist_backend.get_group()
    if group is None:
        raise ValueError("<group> is required.")
    return group


def _single(inputs):
    if isinstance(inputs, torch.Tensor):
        return inputs
    if isinstance(inputs, (list, tuple)) and len(inputs) == 1:
        return inputs[0]
    raise ValueError("Excepted 1 input(s), got {}.".format(len(inputs) if hasattr(inputs, "__len__") else inputs))


def _execute(group, inputs, outputs=None, **coll_args):
    args = group.arguments.copy()
    args.update(coll_args)
    args["comm"] = dist_backend.comm_argument(group)
    if args["comm"] == 0:
        # This rank is not a member: the operator sees "no group" and leaves
        # the tensors alone (collective_op.cc:89).
        args["group"] = 0
    return op_lib.run_collective(inputs, outputs, group_size=group.size, **args)


def all_gather(inputs, group=None, **kwargs):
    """Gather input across all nodes; the output has shape ``[n, *inputs.shape]``."""
    x = _single(inputs)
    group = _resolve(group)
    return _execute(group, [x], operation="ALLGATHER")[0]


def all_reduce(inputs, reduction="sum", group=None, **kwargs):
    """Reduce input across all nodes."""
    x = _single(inputs)
    group = _resolve(group)
    return _execute(group, [x], operation="ALLREDUCE", reduction=reduction.upper())[0]


def broadcast(inputs, root=0, group=None, **kwargs):
    """Broadcast input from the root node; ``root`` is the node index in the group."""
    x = _single(inputs)
    group = _resolve(group)
    return _execute(group, [x], operation="BROADCAST", root=root)[0]


def reduce_scatter(inputs, reduction="sum", group=None, **kwargs):
    """Reduce and scatter input across all nodes along the first dimension."""
    x = _single(inputs)
    group = _resolve(group)
    return _execute(group, [x], operation="REDUCESCATTER", reduction=reduction.upper())[0]


def all_reduce_coalesced(tensors, reduction="sum", group=None, bucket_size=512 * 1024 * 1024):
    """In-place all-reduce of a gradient list, bucketed: the call the
    optimizers make (torch/core/optim/optimizer.py:149-159 with SUM and
    bucket_size, dragon/python/core/training/optimizer.py:70-81 with MEAN)."""
    group = _resolve(group)
    tensors = list(tensors)
    _execute(group, tensors, outputs=tensors, operation="ALLREDUCE", reduction=reduction.upper(),
             bucket_size=bucket_size)
    return tensors


def sync_batch_norm_statistics(stats, batch_size, group=None, count_on_device=False):
    """The exchange of statistics of synchronized batch normalization
    (normalization/batch_norm_op.cc:29-43 and :168-170): ``stats`` holds this
    rank's ``2C`` partial sums (float32) and is all-reduced in place.

    With ``count_on_device=False`` the batch count goes through the blocking
    host all-reduce, as in the reference, and the global count is returned.
    With ``count_on_device=True`` ``stats`` holds ``2C + 1`` values, the last one
    receives ``float(batch_size)`` and travels with the statistics: one device
    kernel, nothing blocks, and the global count is ``stats[-1]``."""
    group = _resolve(group)
    args = group.arguments.copy()
    args["comm"] = dist_backend.comm_argument(group)
    if args["comm"] == 0:
        args["group"] = 0  # not a member: the operator leaves the tensor alone
    return op_lib.run_sync_bn_stats(stats, batch_size, count_on_device=count_on_device, **args)
