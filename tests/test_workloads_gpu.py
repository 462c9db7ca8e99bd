"""The benchmark configurations as parity cases: ResNet-50 and BERT-base
gradient buckets, the int64 / bf16 gather and broadcast shapes, and full-size
messages checked through size-independent properties."""

import numpy as np
import pytest
import torch

from dragon_b200 import workloads
from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def team(dgn_lib):
    from dragon_b200.comm import Communicator
    made = {}

    def get(n):
        if n not in made:
            made[n] = Communicator.emulated(n, 0)
        return made[n]

    yield get
    torch.cuda.synchronize()
    for comms in made.values():
        for c in comms:
            c.destroy()


def test_resnet50_gradient_bucket_mean_8_ranks(team):
    """161 fp32 tensors, 25,557,032 elements, one bucket, MEAN at 8 ranks."""
    n = 8
    comms = team(n)
    shapes = workloads.resnet50_shapes()
    host = [workloads.normal_tensors(r, shapes, 1e-3) for r in range(n)]
    grads = [[torch.from_numpy(a).to(DEV) for a in row] for row in host]
    for r in range(n):
        comms[r].all_reduce(grads[r], None, "MEAN")
    torch.cuda.synchronize()
    assert comms[0].last_launch()["variant"] == 2
    worst = 0.0
    for i in range(len(shapes)):
        want = oracle.allreduce([host[r][i] for r in range(n)], oracle.F32, "MEAN")
        for r in (0, 3, 7):
            H.assert_bits_equal(grads[r][i].cpu().numpy(), want, "tensor {} rank {}".format(i, r))
        ref = oracle.fp64_sum([host[r][i] for r in range(n)], oracle.F32, mean=True)
        worst = max(worst, oracle.max_rel_err(want, ref, oracle.F32))
    assert worst <= 1e-6


def test_bert_base_fp16_buckets_mean(team):
    """199 fp16 tensors in 25 MiB buckets (the embedding is a bucket of its own), fp32 accumulation."""
    n = 2
    comms = team(n)
    shapes = workloads.bert_base_shapes()
    buckets = workloads.greedy_buckets(shapes, 2, 25 * workloads.MiB)
    host = [workloads.normal_tensors(r, shapes, 1e-2, np.float16) for r in range(n)]
    grads = [[torch.from_numpy(a).to(DEV) for a in row] for row in host]
    for bucket in buckets:
        for r in range(n):
            comms[r].all_reduce([grads[r][i] for i in bucket], None, "MEAN")
    torch.cuda.synchronize()
    for i in range(len(shapes)):
        want = oracle.allreduce([host[r][i] for r in range(n)], oracle.F16, "MEAN")
        H.assert_bits_equal(grads[1][i].cpu().numpy(), want, "tensor {}".format(i))
    big = 0  # the word embedding: tolerance against the fp64 sum
    ref = oracle.fp64_sum([host[r][big] for r in range(n)], oracle.F16, mean=True)
    assert oracle.max_rel_err(grads[0][big].cpu().numpy(), ref, oracle.F16) <= 2e-3


@pytest.mark.parametrize("n", [2, 8])
def test_gather_and_broadcast_config_shapes(team, n):
    """int64 [65536] in [0, 2^40) and bf16 [8192, 4096] N(0,1): bit-exact moves."""
    comms = team(n)
    idx = [workloads.index_message(r) for r in range(n)]
    xs = [torch.from_numpy(a).to(DEV) for a in idx]
    outs = [torch.empty(n * 65536, dtype=torch.int64, device=DEV) for _ in range(n)]
    for r in range(n):
        comms[r].all_gather(xs[r], outs[r])
    for r in range(n):
        comms[r].broadcast(xs[r], 0)
    torch.cuda.synchronize()
    want = np.concatenate(idx)
    for r in range(n):
        assert np.array_equal(outs[r].cpu().numpy(), want)
        assert np.array_equal(xs[r].cpu().numpy(), idx[0])
    # bf16 activations: generated on the device from a per-rank seed, compared on the device.
    acts = []
    for r in range(n):
        g = torch.Generator(device=DEV).manual_seed(1000 + r)
        acts.append(torch.randn(8192, 4096, generator=g, device=DEV).to(torch.bfloat16))
    # Ranks 0 and n-1 get outputs of their own; the ranks in between share one
    # scratch output (they all write the same bytes to it).
    gathered = [torch.empty(n, 8192, 4096, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    scratch = torch.empty(n, 8192, 4096, dtype=torch.bfloat16, device=DEV)
    members = list(range(n))
    for r in members:
        out = gathered[0] if r == 0 else (gathered[1] if r == n - 1 else scratch)
        comms[r].all_gather(acts[r], out)
    torch.cuda.synchronize()
    for g in gathered:
        for s in range(n):
            assert torch.equal(g[s].view(torch.int16), acts[s].view(torch.int16))
    copies = [a.clone() for a in acts]
    for r in members:
        comms[r].broadcast(copies[r], 0)
    torch.cuda.synchronize()
    for c in copies:
        assert torch.equal(c.view(torch.int16), acts[0].view(torch.int16))


def test_one_gib_message_properties(team):
    """Full-size message (1 GiB fp32 per rank, 2 ranks): fp32 a + b is unique, so
    torch's own add is the check; a second all-reduce shows linearity."""
    comms = team(2)
    count = (1 << 30) // 4
    g = torch.Generator(device=DEV).manual_seed(7)
    a = torch.rand(count, generator=g, device=DEV) * 2 - 1
    b = torch.rand(count, generator=g, device=DEV) * 2 - 1
    want = a + b
    x, y = a.clone(), b.clone()
    comms[0].all_reduce([x], None, "SUM")
    comms[1].all_reduce([y], None, "SUM")
    torch.cuda.synchronize()
    assert torch.equal(x, want) and torch.equal(y, want)
    del want
    comms[0].all_reduce([x], None, "MEAN")  # (s + s) / 2 == s exactly
    comms[1].all_reduce([y], None, "MEAN")
    torch.cuda.synchronize()
    assert torch.equal(x, a + b) and torch.equal(x, y)


def test_one_gib_fp16_sum_is_exact_on_representable_values(team):
    """512 Mi fp16 elements: values k/1024 with small k add exactly, so the
    expected result is known in closed form at any size."""
    comms = team(2)
    count = (1 << 30) // 2
    k = torch.arange(count, device=DEV, dtype=torch.int32) % 512
    a = (k.float() / 1024).half()
    b = ((511 - k).float() / 1024).half()
    del k
    comms[0].all_reduce([a], None, "SUM")
    comms[1].all_reduce([b], None, "SUM")
    torch.cuda.synchronize()
    expect = torch.tensor(511.0 / 1024).half().item()
    assert float(a.min()) == expect and float(a.max()) == expect and torch.equal(a, b)
