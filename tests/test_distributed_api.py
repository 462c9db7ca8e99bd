"""Host-side behaviour of the distributed Python APIs (no GPU needed)."""

import pytest

from dragon_b200 import distributed
from dragon_b200 import op_lib
from dragon_b200 import torch_distributed
from dragon_b200 import workloads


def test_empty_group():
    """The reference's own test, test/dragon/test_distributed.py:28-40."""
    for backend in (None, "AUTO", "NCCL", "CNCL", "MPI", "UNKNOWN", 0):
        try:
            group = distributed.new_group(backend=backend)
            assert group.ranks is None
            assert group.size == 0
            assert group.arguments["backend"] == group.backend
            assert repr(group) == "%s:None" % group.backend
            with group.as_default():
                assert distributed.get_group() is None
                assert distributed.get_backend(group) == group.backend
        except ValueError:
            pass


def test_backend_names():
    assert distributed.Backend("mpi") == "MPI"
    with pytest.raises(ValueError, match="Invalid backend"):
        distributed.Backend("gloo")
    with pytest.raises(ValueError, match="must be a string"):
        distributed.Backend(3)
    with pytest.raises(ValueError):
        distributed.Backend("CNCL")


def test_single_process_world():
    """test/dragon/test_distributed.py:42-48 without MPI: rank 0 of 1."""
    distributed.finalize()
    assert distributed.get_rank() == 0
    assert distributed.get_world_size() == 1
    assert distributed.is_initialized()
    distributed.finalize()
    assert not distributed.is_initialized()


def test_group_is_required():
    import torch
    x = torch.zeros(4)
    for fn in (distributed.all_reduce, distributed.all_gather, distributed.broadcast, distributed.reduce_scatter):
        with pytest.raises(ValueError, match="<group> is required."):
            fn(x)
    with pytest.raises(ValueError):
        distributed.all_reduce([x, x], group=distributed.new_group(backend="MPI"))


def test_torch_frontend_without_group_returns_input():
    import torch
    x = torch.arange(4.0)
    assert torch_distributed.all_reduce(x) is x
    assert torch_distributed.broadcast(x, src=1) is x
    assert torch_distributed.all_gather([], x) is x
    assert torch_distributed.all_gather_into_tensor(torch.empty(8), x) is x
    assert torch_distributed.reduce_scatter_tensor(torch.empty(2), x) is x


def test_collective_argument_defaults():
    """Names and defaults of the operator's arguments (collective_op.h:24-37)."""
    args = op_lib.collective_args()
    assert args == {"operation": "", "reduction": "SUM", "root": 0, "bucket_size": 0, "comm": 0,
                    "group": 0, "backend": "MPI", "ranks": None}
    text = op_lib._def_text("Collective", ["a"], ["a"], 3, op_lib.collective_args(
        operation="ALLREDUCE", reduction="MEAN", comm=7, group=7, ranks=[0, 2], backend="NCCL")).decode()
    assert "type Collective" in text and "device 1 3" in text
    assert "arg_s reduction MEAN" in text and "arg_ints ranks 0 2" in text and "arg_i comm 7" in text


def test_workload_shapes():
    r = workloads.resnet50_shapes()
    assert len(r) == 161 and sum(map(workloads.numel, r)) == 25557032
    b = workloads.bert_base_shapes()
    assert len(b) == 199 and sum(map(workloads.numel, b)) == 109482240
    buckets = workloads.greedy_buckets(b, 2, 25 * workloads.MiB)
    assert len(buckets) == 8 and buckets[0] == [0]  # the embedding is a bucket of its own
    assert sorted(i for k in buckets for i in k) == list(range(199))
    sizes = workloads.sweep_sizes()
    assert sizes[0] == 1024 and sizes[-1] == 1 << 30 and len(sizes) == 21
    assert (workloads.uniform_message(3, 16) == workloads.uniform_message(3, 16)).all()
