"""The Python APIs and the C++ operator layer on a GPU: dragon.distributed and
the torch frontend's distributed functions, run as 4 virtual ranks on one
device and compared with the oracle."""

import numpy as np
import pytest
import torch

from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu
N = 4
DEV = "cuda:0"


@pytest.fixture(scope="module")
def world(dgn_lib):
    from dragon_b200 import distributed
    w = distributed.init_emulated_world(N, 0)
    yield w
    torch.cuda.synchronize()
    distributed.finalize()


@pytest.fixture(scope="module")
def group(world):
    from dragon_b200 import distributed
    return distributed.new_group(list(range(N)), backend="NCCL")


def per_rank(fn):
    from dragon_b200 import distributed
    out = []
    for r in range(N):
        with distributed.as_rank(r):
            out.append(fn(r))
    torch.cuda.synchronize()
    return out


def test_ranks_and_group(world, group):
    from dragon_b200 import distributed
    assert distributed.get_world_size() == N and group.size == N and group.backend == "NCCL"
    assert per_rank(lambda r: distributed.get_rank(group)) == list(range(N))
    sub = distributed.new_group([3, 1])
    assert per_rank(lambda r: distributed.get_rank(sub)) == [0, 1, 2, 0]  # world rank unless a member


def test_dragon_all_reduce_returns_new_tensor(group):
    from dragon_b200 import distributed
    arrays = [H.make_input(r, 4099, oracle.F32) for r in range(N)]
    xs = [H.to_torch(a, oracle.F32, DEV) for a in arrays]
    for reduction in ("sum", "MEAN", "max"):
        ys = per_rank(lambda r: distributed.all_reduce(xs[r], reduction, group))
        want = oracle.allreduce(arrays, oracle.F32, reduction)
        for r in range(N):
            assert ys[r].data_ptr() != xs[r].data_ptr()
            H.assert_bits_equal(H.to_numpy(ys[r], oracle.F32), want)
            H.assert_bits_equal(H.to_numpy(xs[r], oracle.F32), arrays[r])  # inputs untouched


def test_default_group_stack(group):
    from dragon_b200 import distributed
    xs = [torch.full((8,), float(r + 1), device=DEV) for r in range(N)]
    with group.as_default():
        ys = per_rank(lambda r: distributed.all_reduce(xs[r]))
    assert all(torch.equal(y, torch.full((8,), 10.0, device=DEV)) for y in ys)


def test_dragon_all_gather_broadcast_reduce_scatter(group):
    from dragon_b200 import distributed
    arrays = [H.make_input(r, 6 * N * 5, oracle.BF16) for r in range(N)]
    xs = [H.to_torch(a, oracle.BF16, DEV).view(N * 5, 6) for a in arrays]
    gs = per_rank(lambda r: distributed.all_gather(xs[r], group))
    want = oracle.allgather(arrays, oracle.BF16)
    for g in gs:
        assert tuple(g.shape) == (N, N * 5, 6)
        H.assert_bits_equal(H.to_numpy(g, oracle.BF16), want)
    bs = per_rank(lambda r: distributed.broadcast(xs[r], root=2, group=group))
    for b in bs:
        H.assert_bits_equal(H.to_numpy(b, oracle.BF16), arrays[2])
    H.assert_bits_equal(H.to_numpy(xs[0], oracle.BF16), arrays[0])
    rs = per_rank(lambda r: distributed.reduce_scatter(xs[r], "sum", group))
    want = oracle.reducescatter(arrays, oracle.BF16, "SUM")
    for r in range(N):
        assert tuple(rs[r].shape) == (5, 6)
        H.assert_bits_equal(H.to_numpy(rs[r], oracle.BF16), want[r])


def test_torch_frontend_in_place(group):
    from dragon_b200 import torch_distributed as tdist
    arrays = [H.make_input(r, 1000, oracle.F16) for r in range(N)]
    xs = [H.to_torch(a, oracle.F16, DEV) for a in arrays]
    rets = per_rank(lambda r: tdist.all_reduce(xs[r], op="sum", group=group))
    want = oracle.allreduce(arrays, oracle.F16, "SUM")
    for r in range(N):
        assert rets[r] is xs[r]
        H.assert_bits_equal(H.to_numpy(xs[r], oracle.F16), want)
    ys = [H.to_torch(a, oracle.F16, DEV) for a in arrays]
    per_rank(lambda r: tdist.broadcast(ys[r], src=1, group=group))
    for y in ys:
        H.assert_bits_equal(H.to_numpy(y, oracle.F16), arrays[1])


def test_torch_frontend_gathers(group):
    from dragon_b200 import torch_distributed as tdist
    arrays = [H.make_input(r, 77, oracle.I64) for r in range(N)]
    xs = [H.to_torch(a, oracle.I64, DEV) for a in arrays]
    lists = per_rank(lambda r: tdist.all_gather([None] * N, xs[r], group=group))
    for parts in lists:
        assert len(parts) == N
        for s in range(N):
            assert np.array_equal(parts[s].reshape(-1).cpu().numpy(), arrays[s])
    singles = per_rank(lambda r: tdist.all_gather([], xs[r], group=group))
    assert all(len(s) == 1 and tuple(s[0].shape) == (N, 77) for s in singles)
    outs = [torch.empty(N * 77, dtype=torch.int64, device=DEV) for _ in range(N)]
    per_rank(lambda r: tdist.all_gather_into_tensor(outs[r], xs[r], group=group))
    for o in outs:
        assert np.array_equal(o.cpu().numpy(), oracle.allgather(arrays, oracle.I64))
    ins = [H.to_torch(H.make_input(r, N * 33, oracle.F32), oracle.F32, DEV) for r in range(N)]
    routs = [torch.empty(33, device=DEV) for _ in range(N)]
    per_rank(lambda r: tdist.reduce_scatter_tensor(routs[r], ins[r], op="sum", group=group))
    want = oracle.reducescatter([H.to_numpy(t, oracle.F32) for t in ins], oracle.F32, "SUM")
    for r in range(N):
        H.assert_bits_equal(H.to_numpy(routs[r], oracle.F32), want[r])


def test_subgroup_and_non_members(world):
    from dragon_b200 import distributed
    from dragon_b200 import torch_distributed as tdist
    sub = distributed.new_group([3, 1])
    xs = [torch.full((16,), float(r + 1), device=DEV) for r in range(N)]
    per_rank(lambda r: tdist.all_reduce(xs[r], group=sub))
    assert torch.equal(xs[1], torch.full((16,), 6.0, device=DEV))
    assert torch.equal(xs[3], torch.full((16,), 6.0, device=DEV))
    assert torch.equal(xs[0], torch.full((16,), 1.0, device=DEV))  # not a member: untouched
    assert torch.equal(xs[2], torch.full((16,), 3.0, device=DEV))
    ys = [torch.full((4,), float(r), device=DEV) for r in range(N)]
    per_rank(lambda r: tdist.broadcast(ys[r], src=0, group=sub))  # root index 0 of the group = world rank 3
    assert torch.equal(ys[1], torch.full((4,), 3.0, device=DEV))


def test_optimizer_style_bucketed_all_reduce(group):
    """The gradient-sync call: a list of tensors, in place, bucket_size in bytes."""
    from dragon_b200 import distributed
    counts = [100, 3000, 7, 50000, 64, 1, 20000]
    arrays = [[H.make_input(r, k, oracle.F32, seed=3 + i) for i, k in enumerate(counts)] for r in range(N)]
    for bucket in (0, 16 * 1024, 512 * 1024 * 1024):
        grads = [[H.to_torch(a, oracle.F32, DEV) for a in row] for row in arrays]
        per_rank(lambda r: distributed.all_reduce_coalesced(grads[r], "mean", group, bucket_size=bucket))
        for i in range(len(counts)):
            want = oracle.allreduce([arrays[r][i] for r in range(N)], oracle.F32, "MEAN")
            for r in range(N):
                H.assert_bits_equal(H.to_numpy(grads[r][i], oracle.F32), want, "bucket {} tensor {}".format(bucket, i))


def test_operator_errors_are_reported(group):
    from dragon_b200 import distributed, op_lib
    from dragon_b200.distributed import ops
    x = torch.zeros(8, dtype=torch.int32, device=DEV)
    with distributed.as_rank(0):
        with pytest.raises(op_lib.OperatorError, match="Unsupported operation"):
            ops._execute(group, [x], operation="ALLTOALL")
        with pytest.raises(op_lib.OperatorError, match="Unsupported reduction"):
            ops._execute(group, [x], operation="ALLREDUCE", reduction="AVG")
        with pytest.raises(op_lib.OperatorError, match="MEAN"):
            ops._execute(group, [x], operation="ALLREDUCE", reduction="MEAN")
        with pytest.raises(op_lib.OperatorError, match="root"):
            ops._execute(group, [x], outputs=[x], operation="BROADCAST", root=9)
        with pytest.raises(TypeError):
            distributed.all_reduce(torch.zeros(4, dtype=torch.bool, device=DEV), group=group)
    # The failed calls never reached the kernel: the team is still usable.
    xs = [torch.ones(4, device=DEV) for _ in range(N)]
    ys = per_rank(lambda r: distributed.all_reduce(xs[r], group=group))
    assert torch.equal(ys[0], torch.full((4,), float(N), device=DEV))


def test_cached_operator_is_repointed(group):
    """One cached operator instance serves different tensors on every run."""
    from dragon_b200 import distributed, op_lib
    from dragon_b200.distributed import backend
    for step in range(3):
        xs = [torch.full((100 + step,), float(r + step), device=DEV) for r in range(N)]

        def run(r):
            args = group.arguments.copy()
            args["comm"] = backend.comm_argument(group)
            return op_lib.run_collective([xs[r]], [xs[r]], group_size=N, cache_key="Collective/rank{}".format(r),
                                         operation="ALLREDUCE", reduction="SUM", **args)[0]

        per_rank(run)
        want = float(sum(r + step for r in range(N)))
        assert all(torch.equal(x, torch.full((100 + step,), want, device=DEV)) for x in xs)


@pytest.mark.parametrize("channels", [64, 256, 2048])
def test_sync_batch_norm_statistics_operator(group, channels):
    """The statistics exchange of synchronized batch normalization
    (normalization/batch_norm_op.cc:29-43) through the `SyncBNStats` operator,
    with the batch count riding on the device message: 2C + 1 floats, one
    low-latency all-reduce, no host round trip.  Bit-exact against the oracle."""
    from dragon_b200 import _C, op_lib
    from dragon_b200 import distributed
    from dragon_b200.distributed import ops
    rng = np.random.default_rng(channels)
    host = [np.concatenate([rng.normal(0, 1, 2 * channels).astype(np.float32) * 32, np.zeros(1, np.float32)])
            for _ in range(N)]
    batch = [32, 31, 32, 17]
    stats = [torch.from_numpy(h.copy()).to(DEV) for h in host]
    before = _C.lib().dgn_launch_count()
    per_rank(lambda r: ops.sync_batch_norm_statistics(stats[r], batch[r], group, count_on_device=True))
    assert _C.lib().dgn_launch_count() == before + 1          # one kernel for the whole exchange
    for r in range(N):
        host[r][-1] = float(batch[r])
    want = oracle.allreduce(host, oracle.F32, "SUM")
    for r in range(N):
        H.assert_bits_equal(H.to_numpy(stats[r], oracle.F32), want, "rank {}".format(r))
    assert float(stats[0][-1].item()) == float(sum(batch))
    with distributed.as_rank(0):
        with pytest.raises(op_lib.OperatorError, match="2C"):   # host-count form takes 2C floats
            ops.sync_batch_norm_statistics(stats[0], 32, group)


def test_single_rank_group_is_a_no_op(dgn_lib):
    """comm_size <= 1: the operator returns at once and touches nothing (collective_op.cc:89)."""
    from dragon_b200 import _C, distributed
    distributed.finalize()
    try:
        g = distributed.new_group([0])
        x = torch.arange(8.0, device=DEV)
        before = _C.lib().dgn_launch_count()
        y = distributed.all_reduce(x, "mean", g)
        from dragon_b200 import torch_distributed as tdist
        assert tdist.all_reduce(x, group=g) is x
        torch.cuda.synchronize()
        assert _C.lib().dgn_launch_count() == before and y.shape == x.shape
        assert torch.equal(x, torch.arange(8.0, device=DEV))
    finally:
        distributed.finalize()


def test_optimizer_call_sites(dgn_lib):
    """The two gradient-sync call sites of the reference's optimizers: SUM per
    dtype with buckets and a 1/n grad scale (torch frontend), MEAN unbucketed
    (native); mixed dtypes and a missing gradient."""
    from dragon_b200 import distributed, gradient_sync
    distributed.init_emulated_world(N, 0)
    try:
        group = distributed.new_group(list(range(N)))
        spec = [(oracle.F32, 1000), (oracle.F16, 4099), (oracle.F32, 7), (oracle.F16, 33), (oracle.F32, 70001)]
        host = [[H.make_input(r, k, dt, seed=11 + i) for i, (dt, k) in enumerate(spec)] for r in range(N)]
        grads = [[H.to_torch(a, dt, DEV) for a, (dt, _) in zip(row, spec)] for row in host]
        with group.as_default():
            scales = per_rank(lambda r: gradient_sync.sync_gradients_torch_style(
                grads[r][:2] + [None] + grads[r][2:], bucket_size=64 * 1024))
        assert scales == [1.0 / N] * N
        for i, (dt, _) in enumerate(spec):
            want = oracle.allreduce([host[r][i] for r in range(N)], dt, "SUM")
            for r in range(N):
                H.assert_bits_equal(H.to_numpy(grads[r][i], dt), want, "torch style tensor {}".format(i))
        f32 = [i for i, (dt, _) in enumerate(spec) if dt == oracle.F32]
        grads = [[H.to_torch(host[r][i], oracle.F32, DEV) for i in f32] for r in range(N)]
        per_rank(lambda r: gradient_sync.sync_gradients_native_style(grads[r], group))
        for j, i in enumerate(f32):
            want = oracle.allreduce([host[r][i] for r in range(N)], oracle.F32, "MEAN")
            for r in range(N):
                H.assert_bits_equal(H.to_numpy(grads[r][j], oracle.F32), want, "native style tensor {}".format(i))
        assert gradient_sync.sync_gradients_torch_style([torch.ones(3, device=DEV)]) == 1.0  # no group: untouched
    finally:
        torch.cuda.synchronize()
        distributed.finalize()
