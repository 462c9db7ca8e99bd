"""Parity of the CUDA collectives with the CPU oracle, through the C-ABI.

All ranks are virtual ranks on one device (dgn_comm_create_emulated): one
cooperative kernel runs every rank's blocks, so the flag protocol, the peer
stores/loads and the reduction code are the ones a multi-GPU run executes.
Integer and byte work must match bit for bit; floating point must match the
oracle bit for bit too (same order, same single rounding) and stay within the
contract's tolerance of an fp64 host sum: 1e-6 fp32, 2e-3 fp16, 1e-2 bf16.
"""

import numpy as np
import pytest
import torch

from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu

SIZES = [1, 7, 8, 9, 15, 16, 17, 1000, 4099, 65536 + 3]


@pytest.fixture(scope="module")
def teams(dgn_lib):
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


def run_allreduce(comms, arrays, dtype, redop, inplace=False):
    dev = "cuda:0"
    ins = [H.to_torch(a, dtype, dev) for a in arrays]
    outs = ins if inplace else [torch.empty_like(t) for t in ins]
    for c, i, o in zip(comms, ins, outs):
        c.all_reduce([i], [o], redop)
    torch.cuda.synchronize()
    assert all(c.status() == 0 for c in comms)
    return [H.to_numpy(o, dtype) for o in outs]


def check_allreduce(comms, count, dtype, redop, inplace=False):
    n = len(comms)
    arrays = [H.make_input(r, count, dtype) for r in range(n)]
    want = oracle.allreduce(arrays, dtype, redop)
    got = run_allreduce(comms, arrays, dtype, redop, inplace)
    for r in range(n):
        H.assert_bits_equal(got[r], want, "allreduce n={} count={} dtype={} {} rank {}".format(
            n, count, H.NAMES[dtype], redop, r))
    if dtype in oracle.TOLERANCE and redop in ("SUM", "MEAN"):
        ref = oracle.fp64_sum(arrays, dtype, mean=(redop == "MEAN"))
        err = oracle.max_rel_err(got[0], ref, dtype)
        assert err <= oracle.TOLERANCE[dtype], "max rel err {} > {}".format(err, oracle.TOLERANCE[dtype])


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("dtype", H.ALL_DTYPES, ids=H.NAMES)
def test_allreduce_sum_all_sizes(teams, n, dtype):
    comms = teams(n)
    for variant in (1, 2, 4, 5, 7):
        for c in comms:
            c.set_tuning(variant=variant)
        for count in SIZES:
            check_allreduce(comms, count, dtype, "SUM")
    for c in comms:
        c.set_tuning()


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("dtype", H.FLOAT_DTYPES, ids=[H.NAMES[d] for d in H.FLOAT_DTYPES])
def test_allreduce_mean_inplace(teams, n, dtype):
    comms = teams(n)
    for variant in (1, 2, 4, 5, 7):
        for c in comms:
            c.set_tuning(variant=variant)
        for count in (5, 4099, 1 << 18):
            check_allreduce(comms, count, dtype, "MEAN", inplace=True)
    for c in comms:
        c.set_tuning()


@pytest.mark.parametrize("redop", ["PROD", "MIN", "MAX"])
@pytest.mark.parametrize("dtype", [oracle.I32, oracle.U8, oracle.F32, oracle.F16], ids=["i32", "u8", "f32", "f16"])
def test_allreduce_other_reductions(teams, redop, dtype):
    check_allreduce(teams(4), 4099, dtype, redop)


def test_mean_rejected_for_integers(teams):
    from dragon_b200 import _C
    comms = teams(2)
    t = torch.zeros(16, dtype=torch.int32, device="cuda:0")
    with pytest.raises(_C.DgnError) as e:
        comms[0].all_reduce([t], [t], "MEAN")
    assert e.value.status == _C.ERR_UNSUPPORTED


@pytest.mark.parametrize("n", [2, 8])
def test_allreduce_multi_round_small_chunks(teams, n):
    """Tiny chunks and few blocks force many rounds of the two-shot pipeline."""
    comms = teams(n)
    for c in comms:
        c.set_tuning(variant=2, blocks=3, threads=64, chunk_bytes=256)
    try:
        for dtype in (oracle.F32, oracle.BF16, oracle.I64):
            check_allreduce(comms, 20011, dtype, "SUM")
        info = comms[0].last_launch()
        assert info["rounds"] > 4 and info["blocks"] == 3
    finally:
        for c in comms:
            c.set_tuning()


@pytest.mark.parametrize("n", [2, 3, 8])
def test_allreduce_staged_ring_many_chunks(teams, n):
    """The staged dataflow kernel (copy-in, reducing and copy-out blocks around
    a ring of chunk buffers) with chunks so small that every ring slot is
    reused many times, for one tensor and for a bucket, with rings of one, two,
    four and eight slots and 4, 8 and 16 loads in flight per lane."""
    comms = teams(n)
    try:
        for unroll, depth, chunk in ((4, 1, 4096), (8, 2, 4096), (16, 4, 8192), (8, 8, 4096), (8, 0, 65536)):
            for c in comms:
                c.set_tuning(variant=7, chunk_bytes=chunk)
                c.set_knob("nvls_unroll", unroll)
                c.set_knob("flow_depth", depth)
            for dtype, redop in ((oracle.F32, "MEAN"), (oracle.BF16, "SUM"), (oracle.I64, "SUM")):
                check_allreduce(comms, 200011, dtype, redop, inplace=True)
            info = comms[0].last_launch()
            assert info["variant"] == 7 and info["rounds"] >= 8, info
            counts = [64, 1, 0, 40999, 7, 1 << 16, 33, 2048]
            arrays = [[H.make_input(r, k, oracle.F16, seed=7 + 13 * i) for i, k in enumerate(counts)] for r in range(n)]
            ins = [[H.to_torch(a, oracle.F16, "cuda:0") for a in row] for row in arrays]
            for r in range(n):
                comms[r].all_reduce(ins[r], None, "MEAN")
            torch.cuda.synchronize()
            assert all(c.status() == 0 for c in comms)
            for i in range(len(counts)):
                want = oracle.allreduce([arrays[r][i] for r in range(n)], oracle.F16, "MEAN")
                for r in range(n):
                    H.assert_bits_equal(H.to_numpy(ins[r][i], oracle.F16), want, "tensor {} rank {}".format(i, r))
    finally:
        for c in comms:
            c.set_tuning()
            c.set_knob("nvls_unroll", 0)
            c.set_knob("flow_depth", 0)


def test_config1_fp32_16mib_two_ranks(teams):
    """16 MiB fp32 SUM on 2 ranks (the reference's CPU-runnable case)."""
    from dragon_b200 import workloads
    comms = teams(2)
    arrays = [workloads.uniform_message(r, 4194304) for r in range(2)]
    got = run_allreduce(comms, arrays, oracle.F32, "SUM")
    want = oracle.allreduce(arrays, oracle.F32, "SUM")
    H.assert_bits_equal(got[0], want)
    H.assert_bits_equal(got[1], want)
    # n = 2 leaves no freedom in the order: a + b in fp32 is the fp64 sum rounded once.
    ref = (arrays[0].astype(np.float64) + arrays[1].astype(np.float64)).astype(np.float32)
    H.assert_bits_equal(got[0], ref)


def test_back_to_back_collectives_reuse_staging(teams):
    """Many collectives in a row without host syncs: staging reuse must be safe."""
    comms = teams(4)
    n = 4
    dev = "cuda:0"
    for variant in (1, 2, 4, 5, 7):
        for c in comms:
            c.set_tuning(variant=variant)
        steps = 24
        ins = [[H.to_torch(H.make_input(r, 3001, oracle.F32, seed=50 * s), oracle.F32, dev) for r in range(n)]
               for s in range(steps)]
        outs = [[torch.empty_like(t) for t in row] for row in ins]
        for s in range(steps):
            for r in range(n):
                comms[r].all_reduce([ins[s][r]], [outs[s][r]], "SUM")
        torch.cuda.synchronize()
        for s in range(steps):
            want = oracle.allreduce([H.to_numpy(t, oracle.F32) for t in ins[s]], oracle.F32, "SUM")
            for r in range(n):
                H.assert_bits_equal(H.to_numpy(outs[s][r], oracle.F32), want, "step {}".format(s))
    for c in comms:
        c.set_tuning()


@pytest.mark.parametrize("n", [2, 4])
def test_allreduce_bucket_of_tensors(teams, n):
    """A tensor list travels as one message; results are per tensor."""
    comms = teams(n)
    dev = "cuda:0"
    counts = [64, 1, 0, 4099, 7, 1 << 16, 33, 2048]
    for dtype, redop in ((oracle.F32, "MEAN"), (oracle.F16, "MEAN"), (oracle.I32, "SUM")):
        for variant in (1, 2, 4, 5, 7):
            for c in comms:
                c.set_tuning(variant=variant)
            arrays = [[H.make_input(r, k, dtype, seed=7 + 13 * i) for i, k in enumerate(counts)] for r in range(n)]
            ins = [[H.to_torch(a, dtype, dev) for a in row] for row in arrays]
            for r in range(n):
                comms[r].all_reduce(ins[r], None, redop)
            torch.cuda.synchronize()
            for i, k in enumerate(counts):
                want = oracle.allreduce([arrays[r][i] for r in range(n)], dtype, redop)
                for r in range(n):
                    H.assert_bits_equal(H.to_numpy(ins[r][i], dtype), want, "tensor {} rank {}".format(i, r))
    for c in comms:
        c.set_tuning()


def test_allreduce_unaligned_views(teams):
    """Tensors that start off a 16-byte boundary take the element path."""
    comms = teams(2)
    dev = "cuda:0"
    for dtype in (oracle.F32, oracle.F16, oracle.U8):
        arrays = [H.make_input(r, 5000, dtype) for r in range(2)]
        full = [H.to_torch(a, dtype, dev) for a in arrays]
        views = [t[1:4998] for t in full]
        outs = [torch.zeros(5001, dtype=t.dtype, device=dev)[3:5000] for t in full]
        for variant in (1, 2, 4, 5, 7):
            for c in comms:
                c.set_tuning(variant=variant)
            for r in range(2):
                comms[r].all_reduce([views[r]], [outs[r]], "SUM")
            torch.cuda.synchronize()
            want = oracle.allreduce([a[1:4998] for a in arrays], dtype, "SUM")
            for r in range(2):
                H.assert_bits_equal(H.to_numpy(outs[r], dtype), want)
    for c in comms:
        c.set_tuning()


@pytest.mark.parametrize("n", [2, 4, 8])
def test_allgather_bit_exact(teams, n):
    comms = teams(n)
    dev = "cuda:0"
    # variant 0: automatic (low-latency lines for small blocks, the pushing
    # kernel above, the pulling one for the largest); variant 2: always the
    # pushing kernel, variant 1: always the pulling one; the last shapes force
    # many rounds of them, so that both halves of the boxes are reused.
    for variant, dtype, count, shape in (
            (0, oracle.I64, 65536, {}), (0, oracle.BF16, 70001, {}), (0, oracle.U8, 13, {}), (0, oracle.F64, 1, {}),
            (0, oracle.F32, (1 << 20) + 3, {}), (2, oracle.I64, 65536, {}), (2, oracle.BF16, 70001, {}),
            (2, oracle.U8, 13, {}), (4, oracle.F32, 100003, {}),
            (1, oracle.I64, 65536, {}), (1, oracle.BF16, 70001, {}),
            (1, oracle.F32, 50021, dict(blocks=3, threads=64, chunk_bytes=512)),
            (2, oracle.F32, 50021, dict(blocks=3, threads=64, chunk_bytes=512)),
            # variant 7: the staged gather (pushing and copying blocks around a ring) with remote stores
            (7, oracle.I64, 65536, {}), (7, oracle.BF16, 70001, {}), (7, oracle.U8, 13, {}),
            (7, oracle.F32, 50021, dict(blocks=2, threads=64, chunk_bytes=4096)),
            (7, oracle.F32, (1 << 20) + 3, dict(blocks=3, threads=96, chunk_bytes=65536)),
            # variant 8: staged too, but the ranks load the chunks from the sources' rings
            (8, oracle.I64, 65536, {}), (8, oracle.U8, 13, {}),
            (8, oracle.BF16, 70001, dict(blocks=2, threads=64, chunk_bytes=4096)),
            (8, oracle.F32, (1 << 20) + 3, dict(blocks=3, threads=96, chunk_bytes=65536))):
        for c in comms:
            c.set_tuning(variant=variant, **shape)
        arrays = [H.make_input(r, count, dtype) for r in range(n)]
        if dtype == oracle.BF16:  # NaN payloads, infinities, signed zeros, subnormals travel untouched
            arrays[0][:6] = np.array([0x7FC1, 0xFFFF, 0x7F80, 0x8000, 0x0001, 0xFF80], dtype=np.uint16)
        ins = [H.to_torch(a, dtype, dev) for a in arrays]
        outs = [torch.empty(n * count, dtype=t.dtype, device=dev) for t in ins]
        for r in range(n):
            comms[r].all_gather(ins[r], outs[r])
        torch.cuda.synchronize()
        want = oracle.allgather(arrays, dtype)
        for r in range(n):
            H.assert_bits_equal(H.to_numpy(outs[r], dtype), want, "allgather variant {} rank {}".format(variant, r))
        if shape:
            assert comms[0].last_launch()["rounds"] > 4
    for c in comms:
        c.set_tuning()


@pytest.mark.parametrize("n", [2, 4, 8])
def test_broadcast_bit_exact(teams, n):
    comms = teams(n)
    dev = "cuda:0"
    # variant 1: peers pull from the root; variant 2: scatter + all-gather
    # (large messages); the third shape forces many rounds of the latter.
    # variant 7: the staged gather with the root as its only source.
    # The last two: the root scatters shards to the ranks' inboxes and every rank pushes its own.
    shapes = [dict(variant=1), dict(variant=2), dict(variant=2, blocks=3, threads=64, chunk_bytes=512),
              dict(variant=7), dict(variant=7, blocks=2, threads=64, chunk_bytes=4096),
              dict(variant=7, gather_mode=2), dict(variant=7, blocks=2, threads=64, chunk_bytes=4096, gather_mode=2)]
    most_rounds = 0
    try:
        for shape in shapes:
            shape = dict(shape)
            mode = shape.pop("gather_mode", 1)
            for c in comms:
                c.set_tuning(**shape)
                c.set_knob("gather_mode", mode)
            for root in (0, n - 1):
                for dtype, count in ((oracle.I64, 65536), (oracle.BF16, 100003), (oracle.U8, 1), (oracle.F32, 7)):
                    arrays = [H.make_input(r, count, dtype) for r in range(n)]
                    bufs = [H.to_torch(a, dtype, dev) for a in arrays]
                    for r in range(n):
                        comms[r].broadcast(bufs[r], root)
                    torch.cuda.synchronize()
                    assert all(c.status() == 0 for c in comms)
                    most_rounds = max(most_rounds, comms[0].last_launch()["rounds"])
                    want = oracle.broadcast(arrays, dtype, root)
                    for r in range(n):
                        H.assert_bits_equal(H.to_numpy(bufs[r], dtype), want[r],
                                            "broadcast {} mode {} root {} rank {}".format(shape, mode, root, r))
        assert most_rounds > 4
    finally:
        for c in comms:
            c.set_tuning()
            c.set_knob("gather_mode", 0)


@pytest.mark.parametrize("n", [2, 4, 8])
def test_staged_gather_launches_back_to_back(teams, n):
    """All-gathers (one of them in place) and broadcasts from changing roots,
    with changing chunk sizes, share one ring: a launch must not overwrite what
    a slower rank has not copied out of the launch before."""
    comms = teams(n)
    dev = "cuda:0"
    try:
        plan = [("gather", oracle.F32, 30011, 4096), ("bcast", oracle.BF16, 100003, 8192), ("gather", oracle.U8, 77777, 4096),
                ("bcast", oracle.I64, 9000, 4096), ("gather", oracle.F16, 4099, 0), ("bcast", oracle.F32, 50021, 16384)]
        for rep in range(2):
            for i, (op, dtype, count, chunk) in enumerate(plan):
                variant = 8 if op == "gather" and i == 4 else 7   # one all-gather pulls
                for c in comms:
                    c.set_tuning(variant=variant, chunk_bytes=chunk, threads=128 if i % 2 else 64, blocks=1 + i % 3)
                    c.set_knob("gather_mode", 2 if i in (1, 5) else 1)   # two broadcasts scatter shards
                    c.set_knob("gather_forward_blocks", 1 + rep)
                arrays = [H.make_input(10 * i + r, count, dtype) for r in range(n)]
                if op == "gather":
                    in_place = i == 2
                    outs = [torch.empty(n * count, dtype=H.to_torch(arrays[0], dtype, dev).dtype, device=dev)
                            for _ in range(n)]
                    ins = []
                    for r in range(n):
                        t = H.to_torch(arrays[r], dtype, dev)
                        if in_place:
                            outs[r][r * count:(r + 1) * count].copy_(t)
                            t = outs[r][r * count:(r + 1) * count]
                        ins.append(t)
                    for r in range(n):
                        comms[r].all_gather(ins[r], outs[r])
                    torch.cuda.synchronize()
                    want = oracle.allgather(arrays, dtype)
                    for r in range(n):
                        H.assert_bits_equal(H.to_numpy(outs[r], dtype), want, "staged gather {} rank {}".format(i, r))
                else:
                    root = (i + rep) % n
                    bufs = [H.to_torch(a, dtype, dev) for a in arrays]
                    for r in range(n):
                        comms[r].broadcast(bufs[r], root)
                    torch.cuda.synchronize()
                    want = oracle.broadcast(arrays, dtype, root)
                    for r in range(n):
                        H.assert_bits_equal(H.to_numpy(bufs[r], dtype), want[r], "staged broadcast {} rank {}".format(i, r))
                assert all(c.status() == 0 for c in comms)
                assert comms[0].last_launch()["variant"] == variant
    finally:
        for c in comms:
            c.set_tuning()
            c.set_knob("gather_mode", 0)
            c.set_knob("gather_forward_blocks", 0)


@pytest.mark.parametrize("n", [2, 4, 8])
def test_reducescatter(teams, n):
    comms = teams(n)
    dev = "cuda:0"
    for dtype, count, redop in ((oracle.F32, 4099, "SUM"), (oracle.F16, 1 << 15, "MEAN"), (oracle.I32, 5, "SUM")):
        arrays = [H.make_input(r, n * count, dtype) for r in range(n)]
        ins = [H.to_torch(a, dtype, dev) for a in arrays]
        outs = [torch.empty(count, dtype=t.dtype, device=dev) for t in ins]
        for r in range(n):
            comms[r].reduce_scatter(ins[r], outs[r], redop)
        torch.cuda.synchronize()
        want = oracle.reducescatter(arrays, dtype, redop)
        for r in range(n):
            H.assert_bits_equal(H.to_numpy(outs[r], dtype), want[r], "reducescatter rank {}".format(r))


def test_captured_launches_can_be_replayed(teams):
    """Protocol state (epochs, parity, low-latency counters) lives in device
    memory, so a CUDA graph that holds collectives can be replayed: every
    replay must give the all-reduce of whatever the buffers hold at that time."""
    n = 4
    comms = teams(n)
    dev = "cuda:0"
    small = [torch.zeros(3001, device=dev) for _ in range(n)]        # low-latency kernel
    large = [torch.zeros(1 << 20, device=dev) for _ in range(n)]     # two-shot kernel
    ops = [c.prepare_all_reduce([a], [a], "SUM") for c, a in zip(comms, small)]
    ops += [c.prepare_all_reduce([a], [a], "MEAN") for c, a in zip(comms, large)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for op in ops:  # first launches outside the capture (table / module set-up)
            op()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for op in ops:
            op()
    for rep in range(3):
        for r in range(n):
            small[r].fill_(float(rep + r + 1))
            large[r].copy_(torch.arange(1 << 20, device=dev, dtype=torch.float32) % 7 + r * rep)
        graph.replay()
        torch.cuda.synchronize()
        assert all(c.status() == 0 for c in comms)
        want_small = float(sum(rep + r + 1 for r in range(n)))
        want_large = torch.arange(1 << 20, device=dev, dtype=torch.float32) % 7 + rep * (n - 1) / 2.0
        for r in range(n):
            assert torch.equal(small[r], torch.full((3001,), want_small, device=dev)), "replay {}".format(rep)
            assert torch.equal(large[r], want_large), "replay {}".format(rep)


def test_results_are_deterministic(teams):
    comms = teams(8)
    arrays = [H.make_input(r, 100003, oracle.F16) for r in range(8)]
    a = run_allreduce(comms, arrays, oracle.F16, "MEAN")
    b = run_allreduce(comms, arrays, oracle.F16, "MEAN")
    for r in range(8):
        H.assert_bits_equal(a[r], a[0])
        H.assert_bits_equal(b[r], a[0])


def test_single_rank_paths(dgn_lib):
    """comm_size 1: in place is a no-op (collective_op.cc:89), out of place copies."""
    from dragon_b200 import _C
    from dragon_b200.comm import Communicator
    c = Communicator.init_local(0, 1, 0)
    try:
        x = torch.randn(100003, device="cuda:0")
        y = torch.zeros_like(x)
        before = _C.lib().dgn_launch_count()
        c.all_reduce([x], [x], "MEAN")
        assert _C.lib().dgn_launch_count() == before
        c.all_reduce([x], [y], "MEAN")
        torch.cuda.synchronize()
        assert _C.lib().dgn_launch_count() == before + 1
        assert torch.equal(x, y)
        parts = [torch.randn(k, device="cuda:0").half() for k in (5, 4096, 77)]
        outs = [torch.zeros_like(p) for p in parts]
        c.all_reduce(parts, outs, "SUM")
        g = torch.zeros(100003, device="cuda:0")
        c.all_gather(x, g)
        c.broadcast(x, 0)
        torch.cuda.synchronize()
        assert all(torch.equal(a, b) for a, b in zip(parts, outs))
        assert torch.equal(g, x)
    finally:
        c.destroy()


def test_wait_limit_reports_timeout_without_hanging(dgn_lib):
    """A peer that never launches: the kernel gives up after the limit, the
    status word says so and the communicator refuses further work."""
    from dragon_b200 import _C
    from dragon_b200.comm import Communicator
    a = Communicator.init_local(0, 2, 0)
    b = Communicator.init_local(1, 2, 0)
    try:
        handles = [a.handle_bytes(), b.handle_bytes()]
        a.connect(handles)
        b.connect(handles)
        a.set_wait_limit_ms(50)
        x = torch.ones(1024, device="cuda:0")
        a.all_reduce([x], [x], "SUM")  # rank 1 never joins
        torch.cuda.synchronize()
        assert a.status() == _C.ERR_TIMEOUT
        with pytest.raises(_C.DgnError) as e:
            a.all_reduce([x], [x], "SUM")
        assert e.value.status == _C.ERR_STATE
        assert b.status() == 0
    finally:
        a.destroy()
        b.destroy()


def test_empty_messages_launch_nothing(teams):
    """count == 0 is legal everywhere and enqueues no kernel."""
    from dragon_b200 import _C
    comms = teams(2)
    lib = _C.lib()
    before = lib.dgn_launch_count()
    e32 = [torch.empty(0, device="cuda:0") for _ in range(2)]
    for r in range(2):
        comms[r].all_reduce([e32[r]], None, "MEAN")
        comms[r].all_reduce([], None, "SUM")
        comms[r].all_gather(e32[r], torch.empty(0, device="cuda:0"))
        comms[r].broadcast(e32[r], 1)
        comms[r].reduce_scatter(e32[r], torch.empty(0, device="cuda:0"), "SUM")
    torch.cuda.synchronize()
    assert lib.dgn_launch_count() == before
    # A list whose only non-empty tensor is in the middle is the flat case.
    xs = [[torch.empty(0, device="cuda:0"), torch.full((33,), float(r + 1), device="cuda:0"),
           torch.empty(0, device="cuda:0")] for r in range(2)]
    for r in range(2):
        comms[r].all_reduce(xs[r], None, "SUM")
    torch.cuda.synchronize()
    assert torch.equal(xs[0][1], torch.full((33,), 3.0, device="cuda:0"))
    assert lib.dgn_launch_count() == before + 1


def test_more_tensors_than_one_launch_takes(teams):
    """A list longer than the per-launch table (1024 entries) is split into several launches."""
    from dragon_b200 import _C
    comms = teams(2)
    nt = 1500
    rng = np.random.default_rng(5)
    counts = rng.integers(1, 40, nt)
    host = [[rng.integers(-1000, 1000, int(k)).astype(np.int32) for k in counts] for _ in range(2)]
    dev = [[torch.from_numpy(a).to("cuda:0") for a in row] for row in host]
    before = _C.lib().dgn_launch_count()
    for r in range(2):
        comms[r].all_reduce(dev[r], None, "SUM")
    torch.cuda.synchronize()
    assert _C.lib().dgn_launch_count() == before + 2
    for i in (0, 1, 777, 1023, 1024, 1499):
        want = host[0][i] + host[1][i]
        assert np.array_equal(dev[0][i].cpu().numpy(), want) and np.array_equal(dev[1][i].cpu().numpy(), want)


def test_argument_errors(dgn_lib):
    """Bad arguments come back as status codes with a message; nothing is launched."""
    import ctypes
    from dragon_b200 import _C
    from dragon_b200.comm import Communicator
    a = Communicator.init_local(0, 2, 0)
    b = Communicator.init_local(1, 2, 0)
    try:
        x = torch.zeros(8, device="cuda:0")
        with pytest.raises(_C.DgnError) as e:  # not connected yet
            a.all_reduce([x], None, "SUM")
        assert e.value.status == _C.ERR_STATE
        ha, hb = a.handle_bytes(), b.handle_bytes()
        with pytest.raises(_C.DgnError) as e:  # handles in the wrong order
            a.connect([hb, ha])
        assert e.value.status == _C.ERR_ARG
        with pytest.raises(_C.DgnError) as e:  # not a handle
            a.connect([ha, b"\0" * _C.HANDLE_BYTES])
        assert e.value.status == _C.ERR_ARG
        a.connect([ha, hb])
        b.connect([ha, hb])
        with pytest.raises(_C.DgnError) as e:
            a.set_tuning(variant=99)
        assert e.value.status == _C.ERR_ARG
        with pytest.raises(_C.DgnError) as e:
            a.broadcast(x, root=2)
        assert e.value.status == _C.ERR_ARG and "root" in str(e.value)
        assert dgn_lib.dgn_allreduce(a._h, None, None, None, 1, _C.F32, _C.SUM, None) == _C.ERR_ARG
        one = (ctypes.c_void_p * 1)(x.data_ptr())
        cnt = (ctypes.c_int64 * 1)(8)
        assert dgn_lib.dgn_allreduce(a._h, one, one, cnt, 1, 42, _C.SUM, None) == _C.ERR_ARG
        assert dgn_lib.dgn_allreduce(a._h, one, one, cnt, 1, _C.F32, 9, None) == _C.ERR_ARG
        neg = (ctypes.c_int64 * 1)(-1)
        assert dgn_lib.dgn_allreduce(a._h, one, one, neg, 1, _C.F32, _C.SUM, None) == _C.ERR_ARG
        assert a.status() == 0 and b.status() == 0
    finally:
        a.destroy()
        b.destroy()


def test_host_allreduce_where_no_peer_is_needed(teams, dgn_lib):
    """The host-memory all-reduce: identity at comm_size 1, refused on emulated
    ranks (it blocks, and virtual ranks share one host thread)."""
    from dragon_b200 import _C
    from dragon_b200.comm import Communicator
    c = Communicator.init_local(0, 1, 0)
    try:
        assert c.all_reduce_host(np.array([3, 4], dtype=np.int64)).tolist() == [3, 4]
    finally:
        c.destroy()
    with pytest.raises(_C.DgnError) as e:
        teams(2)[0].all_reduce_host(np.array([1.0], dtype=np.float32))
    assert e.value.status == _C.ERR_UNSUPPORTED
