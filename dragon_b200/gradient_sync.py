"""The two data-parallel gradient-sync call sites of the reference, as
functions over torch CUDA tensors.

* torch frontend, ``Optimizer.step`` (torch/core/optim/optimizer.py:134-164,
  261-262): gradients are grouped by dtype, each group is all-reduced in place
  with ``reduction="SUM"`` and ``bucket_size`` (512 MiB by default), and the
  division by the group size is folded into the update's ``grad_scale``.
* native optimizers, ``apply_gradients``
  (dragon/python/core/training/optimizer.py:70-81): all gradients go through
  one ``Collective`` with ``reduction="MEAN"`` and no bucketing (one collective
  per tensor in the reference; still one operator run here).

Both return without synchronising; the gradients are reduced in place.
"""

import collections

from dragon_b200.distributed import backend as dist_backend
from dragon_b200.distributed.ops import _execute


def sync_gradients_torch_style(grads, bucket_size=512 * 1024 * 1024, group=None):
    """SUM all-reduce per dtype, bucketed.  Returns the factor the caller folds
    into ``grad_scale`` (1 / group size, or 1.0 without a group)."""
    group = group or dist_backend.get_group()
    if group is None:
        return 1.0
    by_dtype = collections.defaultdict(list)
    for g in grads:
        if g is not None:
            by_dtype[g.dtype].append(g)
    for same in by_dtype.values():
        _execute(group, same, outputs=same, operation="ALLREDUCE", reduction="SUM", bucket_size=bucket_size)
    return 1.0 / group.size


def sync_gradients_native_style(grads, group=None):
    """MEAN all-reduce of every gradient, in place, unbucketed."""
    group = group or dist_backend.get_group()
    if group is None:
        return
    grads = [g for g in grads if g is not None]
    if grads:
        _execute(group, grads, outputs=grads, operation="ALLREDUCE", reduction="MEAN")
