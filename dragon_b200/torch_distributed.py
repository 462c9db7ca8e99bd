"""The torch frontend's ``distributed`` functions on torch CUDA tensors.

Behaviour of torch/core/ops/distributed_ops.py:22-223 (installed as
``dragon.vm.torch.distributed``): ``op`` is a string, all_reduce and broadcast
work in place and return the tensor, and with no group (argument and default
both None) every function returns its input untouched.
"""

from dragon_b200.distributed import backend as dist_backend
from dragon_b200.distributed.backend import get_backend  # noqa: F401
from dragon_b200.distributed.backend import get_rank  # noqa: F401
from dragon_b200.distributed.backend import get_world_size  # noqa: F401
from dragon_b200.distributed.backend import is_initialized  # noqa: F401
from dragon_b200.distributed.backend import new_group  # noqa: F401
from dragon_b200.distributed.ops import _execute


def all_gather(tensor_list, tensor, group=None):
    """Gather tensor across all nodes.  As in the reference, the gathered
    tensor is split into ``len(tensor_list)`` new tensors which are returned
    (the passed list is not filled); an empty list returns ``[gathered]``.
    The parts are views of one gathered buffer rather than copies."""
    group = group or dist_backend.get_group()
    if group is None:
        return tensor
    gathered = _execute(group, [tensor], operation="ALLGATHER")[0]
    if len(tensor_list) > 0:
        return list(gathered.chunk(len(tensor_list), dim=0))
    return [gathered]


def all_gather_into_tensor(output_tensor, input_tensor, group=None):
    """Gather tensor across all nodes into ``output_tensor`` (``n * numel`` elements)."""
    group = group or dist_backend.get_group()
    if group is None:
        return input_tensor
    view = output_tensor.view((group.size,) + tuple(input_tensor.shape))
    _execute(group, [input_tensor], outputs=[view], operation="ALLGATHER")
    return output_tensor


def all_reduce(tensor, op="sum", group=None):
    """Reduce tensor across all nodes, in place."""
    group = group or dist_backend.get_group()
    if group is None:
        return tensor
    return _execute(group, [tensor], outputs=[tensor], operation="ALLREDUCE", reduction=op.upper())[0]


def broadcast(tensor, src=0, group=None):
    """Broadcast tensor from the source node, in place."""
    group = group or dist_backend.get_group()
    if group is None:
        return tensor
    return _execute(group, [tensor], outputs=[tensor], operation="BROADCAST", root=src)[0]


def reduce_scatter(output, input_list, op="sum", group=None):
    """Reduce and scatter the tensor list across all nodes."""
    import torch
    group = group or dist_backend.get_group()
    if group is None:
        return input_list
    flat = torch.cat([t.reshape(-1) for t in input_list]) if len(input_list) > 1 else input_list[0].reshape(-1)
    view = output.view(-1)
    _execute(group, [flat], outputs=[view], operation="REDUCESCATTER", reduction=op.upper())
    return output


def reduce_scatter_tensor(output, input, op="sum", group=None):
    """Reduce and scatter the tensor across all nodes."""
    group = group or dist_backend.get_group()
    if group is None:
        return input
    flat_out = output.view(-1)
    _execute(group, [input.reshape(-1)], outputs=[flat_out], operation="REDUCESCATTER", reduction=op.upper())
    return output
