"""Real peer traffic: one rank per GPU.  Skipped where fewer than two GPUs are
visible.  Ranks of one process use peer access; the two-process case goes
through CUDA IPC and the file rendezvous (dgn_comm_create)."""

import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def gpu_count():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


needs_two = pytest.mark.skipif(gpu_count() < 2, reason="needs at least two GPUs")


@pytest.fixture(scope="module")
def comms(dgn_lib):
    from dragon_b200.comm import Communicator
    n = min(gpu_count(), 8)
    made = [Communicator.init_local(r, n, r, symm_bytes=64 << 20) for r in range(n)]
    handles = [c.handle_bytes() for c in made]
    for c in made:
        c.connect(handles)
    yield made
    for r in range(n):
        torch.cuda.synchronize(r)
    for c in made:
        c.destroy()


def sync_all(n):
    for r in range(n):
        torch.cuda.synchronize(r)


@needs_two
@pytest.mark.parametrize("variant", [4, 5, 1, 2, 7])
def test_allreduce_across_gpus(comms, variant):
    n = len(comms)
    for c in comms:
        c.set_tuning(variant=variant)
    try:
        for dtype, redop, count in ((oracle.F32, "MEAN", 100003), (oracle.F16, "MEAN", 1 << 20),
                                    (oracle.BF16, "SUM", 4099), (oracle.I64, "SUM", 70001),
                                    (oracle.F32, "SUM", 4194304)):
            arrays = [H.make_input(r, count, dtype) for r in range(n)]
            xs = [H.to_torch(a, dtype, "cuda:{}".format(r)) for r, a in enumerate(arrays)]
            for r in range(n):
                with torch.cuda.device(r):
                    comms[r].all_reduce([xs[r]], None, redop)
            sync_all(n)
            want = oracle.allreduce(arrays, dtype, redop)
            for r in range(n):
                assert comms[r].status() == 0
                H.assert_bits_equal(H.to_numpy(xs[r], dtype), want, "variant {} rank {}".format(variant, r))
    finally:
        for c in comms:
            c.set_tuning()


@needs_two
def test_nvls_allreduce_across_gpus(comms):
    """The staged ring reduced through NVSwitch multicast, where the box exposes
    it: one chunk, many chunks with every ring slot reused, ragged sizes, out of
    place and in place back to back, a bucket of tensors.  The switch chooses
    the order of the additions, so the check is the tolerance contract against
    an fp64 host sum plus identical bits on every rank (with two ranks a + b has
    one order, so float32 also equals the oracle bit for bit)."""
    n = len(comms)
    if not comms[0].has_nvls():
        pytest.skip("NVSwitch multicast is not available on this box")
    assert all(c.has_nvls() for c in comms)
    cases = ((oracle.F32, "MEAN", 5, 0, 8), (oracle.F32, "SUM", (1 << 20) + 3, 0, 4),
             (oracle.F16, "MEAN", 1 << 24, 1 << 20, 8), (oracle.BF16, "SUM", (1 << 22) + 1, 256 << 10, 16),
             (oracle.F32, "MEAN", 1 << 22, 1 << 20, 4), (oracle.F32, "SUM", 1 << 24, 0, 8))
    try:
        for dtype, redop, count, chunk, unroll in cases:
            for c in comms:
                c.set_tuning(variant=3, chunk_bytes=chunk)
                c.set_knob("nvls_unroll", unroll)
            arrays = [H.make_input(r, count, dtype) for r in range(n)]
            xs = [H.to_torch(a, dtype, "cuda:{}".format(r)) for r, a in enumerate(arrays)]
            outs = [torch.empty_like(x) for x in xs]
            for r in range(n):
                with torch.cuda.device(r):
                    comms[r].all_reduce([xs[r]], [outs[r]], redop)   # out of place
                    comms[r].all_reduce([xs[r]], None, redop)        # in place, back to back
            sync_all(n)
            launch = comms[0].last_launch()
            assert launch["variant"] == 3
            if chunk:
                assert launch["rounds"] >= 16   # more chunks than ring slots
            ref = oracle.fp64_sum(arrays, dtype, mean=(redop == "MEAN"))
            got0 = H.to_numpy(outs[0], dtype)
            assert oracle.max_rel_err(got0, ref, dtype) <= oracle.TOLERANCE[dtype]
            for r in range(n):
                assert comms[r].status() == 0
                H.assert_bits_equal(H.to_numpy(outs[r], dtype), got0, "out of place, rank {}".format(r))
                H.assert_bits_equal(H.to_numpy(xs[r], dtype), got0, "in place, rank {}".format(r))
            if n == 2 and dtype == oracle.F32:
                H.assert_bits_equal(got0, oracle.allreduce(arrays, dtype, redop), "two ranks: one order")
        # A bucket of ragged tensors as one message, several chunks.
        for c in comms:
            c.set_tuning(variant=3, chunk_bytes=1 << 20)
            c.set_knob("nvls_unroll", 8)
        sizes = [70001, 3, 1 << 19, 257, (1 << 20) + 1]
        host = [[H.make_input(r, k, oracle.F32, seed=77 + i) for i, k in enumerate(sizes)] for r in range(n)]
        dev = [[H.to_torch(a, oracle.F32, "cuda:{}".format(r)) for a in host[r]] for r in range(n)]
        for r in range(n):
            with torch.cuda.device(r):
                comms[r].all_reduce(dev[r], None, "MEAN")
        sync_all(n)
        assert comms[0].last_launch()["variant"] == 3
        for i in range(len(sizes)):
            ref = oracle.fp64_sum([host[r][i] for r in range(n)], oracle.F32, mean=True)
            for r in range(n):
                assert oracle.max_rel_err(H.to_numpy(dev[r][i], oracle.F32), ref, oracle.F32) <= 1e-6
                H.assert_bits_equal(H.to_numpy(dev[r][i], oracle.F32), H.to_numpy(dev[0][i], oracle.F32))
    finally:
        for c in comms:
            c.set_tuning()
            c.set_knob("nvls_unroll", 0)


@needs_two
def test_symmetric_memory_allreduce_in_place_across_gpus(comms):
    """Buffers from the symmetric arena are reduced in place by the switch.
    With two ranks a + b has one possible order, so float32 results equal the
    oracle bit for bit (for the 16-bit types the switch's final rounding is its
    own); otherwise the tolerance contract applies, and all ranks must always
    hold identical bits."""
    n = len(comms)
    if not comms[0].has_nvls() or comms[0].symm_capacity() == 0:
        pytest.skip("NVSwitch multicast is not available on this box")
    assert all(c.symm_capacity() == 64 << 20 for c in comms)
    torch_dtype = {oracle.F32: torch.float32, oracle.F16: torch.float16, oracle.BF16: torch.bfloat16}
    cases = ((oracle.F32, "MEAN", 1 << 20), (oracle.F16, "MEAN", (1 << 21) + 8), (oracle.BF16, "SUM", 1 << 19),
             (oracle.F32, "SUM", 4), (oracle.F32, "MEAN", (1 << 22) + 4))
    try:
        for dtype, redop, count in cases:
            for c in comms:
                c.symm_reset()
                c.set_tuning(variant=6)
            arrays = [H.make_input(r, count, dtype) for r in range(n)]
            xs = []
            for r in range(n):
                with torch.cuda.device(r):
                    pad = comms[r].symm_empty(100, torch.uint8)  # buffers need not start the arena
                    x = comms[r].symm_empty(count, torch_dtype[dtype])
                    x.copy_(H.to_torch(arrays[r], dtype, "cuda:{}".format(r)))
                    xs.append(x)
                    del pad
            for rep in range(2):
                for r in range(n):
                    with torch.cuda.device(r):
                        comms[r].all_reduce([xs[r]], None, redop)
                sync_all(n)
                assert comms[0].last_launch()["variant"] == 6
                got0 = H.to_numpy(xs[0], dtype)
                for r in range(n):
                    assert comms[r].status() == 0
                    H.assert_bits_equal(H.to_numpy(xs[r], dtype), got0, "rank {} differs from rank 0".format(r))
                if rep == 0:
                    ref = oracle.fp64_sum(arrays, dtype, mean=(redop == "MEAN"))
                    assert oracle.max_rel_err(got0, ref, dtype) <= oracle.TOLERANCE[dtype]
                    if n == 2 and dtype == oracle.F32:
                        H.assert_bits_equal(got0, oracle.allreduce(arrays, dtype, redop), "two ranks: one order")
        # Automatic choice: in place through the switch from 4 MiB on (the
        # default at three ranks and more; set here for any rank count), the
        # usual kernels below; a ragged tail (not a whole number of vectors)
        # and an out-of-place call never take the in-place path.
        for c in comms:
            c.symm_reset()
            c.set_tuning()
            c.set_knob("symm_min_bytes", 4 << 20)
        for count, want_symm in ((1 << 20, True), (1 << 10, False), ((1 << 20) + 1, False)):
            arrays = [H.make_input(r, count, oracle.F32) for r in range(n)]
            xs = []
            for r in range(n):
                with torch.cuda.device(r):
                    comms[r].symm_reset()
                    x = comms[r].symm_empty(count, torch.float32)
                    x.copy_(H.to_torch(arrays[r], oracle.F32, "cuda:{}".format(r)))
                    xs.append(x)
            for r in range(n):
                with torch.cuda.device(r):
                    comms[r].all_reduce([xs[r]], None, "SUM")
            sync_all(n)
            assert (comms[0].last_launch()["variant"] == 6) == want_symm
            ref = oracle.fp64_sum(arrays, oracle.F32)
            for r in range(n):
                assert oracle.max_rel_err(H.to_numpy(xs[r], oracle.F32), ref, oracle.F32) <= 1e-6
        outs = [torch.empty(1 << 20, device="cuda:{}".format(r)) for r in range(n)]
        for r in range(n):
            with torch.cuda.device(r):
                comms[r].all_reduce([xs[r][:1 << 20]], [outs[r]], "SUM")
        sync_all(n)
        assert comms[0].last_launch()["variant"] != 6
        with pytest.raises(Exception, match="exhausted"):
            comms[0].symm_empty(65 << 20, torch.uint8)
    finally:
        for c in comms:
            c.set_tuning()
            c.symm_reset()
            c.set_knob("symm_min_bytes", 0)


@needs_two
def test_back_to_back_mixed_collectives_across_gpus(comms):
    n = len(comms)
    steps = 12
    sizes = [257, 70000, 3, 1 << 19, 5000, 1 << 21]
    arrays = [[H.make_input(r, sizes[s % len(sizes)], oracle.F32, seed=31 * s) for r in range(n)] for s in range(steps)]
    xs = [[H.to_torch(a, oracle.F32, "cuda:{}".format(r)) for r, a in enumerate(row)] for row in arrays]
    gathered = [torch.empty(n * 257, device="cuda:{}".format(r)) for r in range(n)]
    for s in range(steps):
        for r in range(n):
            with torch.cuda.device(r):
                comms[r].all_reduce([xs[s][r]], None, "SUM")
                if s == 6:
                    comms[r].all_gather(xs[0][r], gathered[r])
                    comms[r].broadcast(xs[2][r], n - 1)
    sync_all(n)
    for s in range(steps):
        if s in (0, 2):
            continue
        want = oracle.allreduce(arrays[s], oracle.F32, "SUM")
        for r in range(n):
            H.assert_bits_equal(H.to_numpy(xs[s][r], oracle.F32), want, "step {} rank {}".format(s, r))
    first = oracle.allreduce(arrays[0], oracle.F32, "SUM")
    for r in range(n):
        H.assert_bits_equal(H.to_numpy(gathered[r], oracle.F32), np.tile(first, n))


@needs_two
def test_gather_broadcast_reducescatter_across_gpus(comms):
    n = len(comms)
    arrays = [H.make_input(r, n * 65536, oracle.I64) for r in range(n)]
    xs = [H.to_torch(a, oracle.I64, "cuda:{}".format(r)) for r, a in enumerate(arrays)]
    outs = [torch.empty(n * n * 65536, dtype=torch.int64, device="cuda:{}".format(r)) for r in range(n)]
    rs = [torch.empty(65536, dtype=torch.int64, device="cuda:{}".format(r)) for r in range(n)]
    for r in range(n):
        with torch.cuda.device(r):
            comms[r].all_gather(xs[r], outs[r])
            comms[r].reduce_scatter(xs[r], rs[r], "SUM")
    sync_all(n)
    want = oracle.allgather(arrays, oracle.I64)
    parts = oracle.reducescatter(arrays, oracle.I64, "SUM")
    for r in range(n):
        assert np.array_equal(outs[r].cpu().numpy(), want)
        assert np.array_equal(rs[r].cpu().numpy(), parts[r])
    for r in range(n):
        with torch.cuda.device(r):
            comms[r].broadcast(xs[r], 1)
    sync_all(n)
    for r in range(n):
        assert np.array_equal(xs[r].cpu().numpy(), arrays[1])
    # Large broadcast (scatter + all-gather from three ranks up), odd size, last rank as root.
    big = [H.make_input(r, (1 << 22) + 3, oracle.F32) for r in range(n)]
    bs = [H.to_torch(a, oracle.F32, "cuda:{}".format(r)) for r, a in enumerate(big)]
    for rep in range(2):
        for r in range(n):
            with torch.cuda.device(r):
                comms[r].broadcast(bs[r], n - 1)
    sync_all(n)
    for r in range(n):
        assert comms[r].status() == 0
        H.assert_bits_equal(H.to_numpy(bs[r], oracle.F32), big[n - 1], "large broadcast rank {}".format(r))


@needs_two
def test_sharded_adamw_step_across_gpus(comms):
    """The sharded optimizer step with one rank per GPU: shard slices and the
    updated parameters travel over NVLink; same bit-exact bar as on virtual ranks."""
    from tests.test_zero_gpu import RAGGED, Harness, _grads
    n = len(comms)
    devices = ["cuda:{}".format(r) for r in range(n)]
    for dtype in (oracle.F16, oracle.F32):
        h = Harness(comms, RAGGED, dtype, devices=devices)
        found = [torch.zeros(1, dtype=torch.float32, device=d) for d in devices]
        for step in range(3):
            assert h.step([_grads(r, step, RAGGED, dtype) for r in range(n)], found_inf=found) == 0.0
            h.check(what="multi-GPU step {}".format(step))
        assert all(f.item() == 0.0 for f in found)
    # A bucket of several staging rounds: 8 Mi + 3 elements in one tensor.
    counts = [(1 << 23) + 3]
    h = Harness(comms, counts, oracle.BF16, devices=devices)
    h.step([_grads(r, 0, counts, oracle.BF16) for r in range(n)])
    h.check(what="multi-GPU large bucket")


@needs_two
def test_multicast_broadcast_across_gpus(comms):
    """BROADCAST through the switch (the root alone, or every rank its shard):
    byte-exact for every root, ragged sizes, several rounds, back to back."""
    n = len(comms)
    if not comms[0].has_nvls():
        pytest.skip("NVSwitch multicast is not available on this box")
    try:
        for dtype, count in ((oracle.I64, 65536), (oracle.U8, 13), (oracle.BF16, (1 << 20) + 5),
                             (oracle.I64, (5 << 20) + 3), (oracle.F32, 1)):
            # The large case in 128 KiB pieces, so that it takes several rounds at any rank count.
            for c in comms:
                c.set_tuning(variant=3, chunk_bytes=(128 << 10) if count > (4 << 20) else 0)
            # mode 1: the root multicasts alone; mode 2: it scatters shards and every rank multicasts its own
            for root, mode in ((0, 1), (n - 1, 2), (0, 2), (n - 1, 1)):
                for c in comms:
                    c.set_knob("gather_mode", mode)
                arrays = [H.make_input(r, count, dtype, seed=500 + root) for r in range(n)]
                if dtype == oracle.BF16:
                    arrays[root][:4] = [0x7FC1, 0xFFFF, 0x8000, 0x0001]  # NaN payloads, -0, a subnormal
                xs = [H.to_torch(a, dtype, "cuda:{}".format(r)) for r, a in enumerate(arrays)]
                for rep in range(2):
                    for r in range(n):
                        with torch.cuda.device(r):
                            comms[r].broadcast(xs[r], root)
                sync_all(n)
                assert comms[0].last_launch()["variant"] == 3
                if count > (4 << 20):
                    assert comms[0].last_launch()["rounds"] >= 2
                for r in range(n):
                    assert comms[r].status() == 0
                    H.assert_bits_equal(H.to_numpy(xs[r], dtype), arrays[root], "root {} rank {}".format(root, r))
    finally:
        for c in comms:
            c.set_tuning()
            c.set_knob("gather_mode", 0)


@needs_two
def test_multicast_allgather_across_gpus(comms):
    """ALLGATHER through the switch (every rank stores its block once, the switch
    replicates it): byte-exact, ragged sizes, more chunks than ring slots, in
    place and out of place, alternating with broadcasts on the same ring."""
    n = len(comms)
    if not comms[0].has_nvls():
        pytest.skip("NVSwitch multicast is not available on this box")
    try:
        for i, (dtype, count, chunk) in enumerate(((oracle.I64, 65536, 0), (oracle.U8, 13, 0), (oracle.BF16, (1 << 20) + 5, 65536),
                                                   (oracle.F32, (3 << 20) + 1, 256 << 10), (oracle.F16, 70001, 4096))):
            for c in comms:
                c.set_tuning(variant=3, chunk_bytes=chunk, blocks=1 + i % 4)
                c.set_knob("gather_mode", 2 if i % 2 else 1)  # the broadcasts in between: scattering / root alone
            arrays = [H.make_input(r, count, dtype, seed=700 + i) for r in range(n)]
            want = oracle.allgather(arrays, dtype)
            ins = [H.to_torch(a, dtype, "cuda:{}".format(r)) for r, a in enumerate(arrays)]
            outs = [torch.empty(n * count, dtype=ins[r].dtype, device="cuda:{}".format(r)) for r in range(n)]
            if i == 3:  # in place: the own block already sits in the output
                for r in range(n):
                    outs[r][r * count:(r + 1) * count].copy_(ins[r])
                    ins[r] = outs[r][r * count:(r + 1) * count]
            bs = [H.to_torch(a, dtype, "cuda:{}".format(r)) for r, a in enumerate(arrays)]
            for rep in range(2):
                for r in range(n):
                    with torch.cuda.device(r):
                        comms[r].all_gather(ins[r], outs[r])
                        comms[r].broadcast(bs[r], (i + rep) % n)
            sync_all(n)
            assert comms[0].last_launch()["variant"] == 3
            for r in range(n):
                assert comms[r].status() == 0
                H.assert_bits_equal(H.to_numpy(outs[r], dtype), want, "multicast all-gather case {} rank {}".format(i, r))
                H.assert_bits_equal(H.to_numpy(bs[r], dtype), arrays[i % n], "broadcast between gathers, rank {}".format(r))
        # All-gather where every rank loads from the sources' rings (no switch involved).
        for c in comms:
            c.set_tuning(variant=8, chunk_bytes=64 << 10)
        arrays = [H.make_input(r, (1 << 20) + 7, oracle.BF16, seed=900) for r in range(n)]
        ins = [H.to_torch(a, oracle.BF16, "cuda:{}".format(r)) for r, a in enumerate(arrays)]
        outs = [torch.empty(n * ins[r].numel(), dtype=ins[r].dtype, device="cuda:{}".format(r)) for r in range(n)]
        for rep in range(2):
            for r in range(n):
                with torch.cuda.device(r):
                    comms[r].all_gather(ins[r], outs[r])
        sync_all(n)
        assert comms[0].last_launch()["variant"] == 8 and comms[0].last_launch()["rounds"] > 8
        want = oracle.allgather(arrays, oracle.BF16)
        for r in range(n):
            assert comms[r].status() == 0
            H.assert_bits_equal(H.to_numpy(outs[r], oracle.BF16), want, "pulling staged all-gather rank {}".format(r))
    finally:
        for c in comms:
            c.set_tuning()
            c.set_knob("gather_mode", 0)


@needs_two
def test_two_processes_over_ipc_and_file_rendezvous():
    with tempfile.TemporaryDirectory() as rdv:
        env = dict(os.environ, DGN_NVLS="0", PYTHONFAULTHANDLER="1")  # workers may leave early: keep them off the multicast object
        procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "mp_gpu_worker.py"), str(r), "2", rdv],
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env) for r in range(2)]
        # Every wait in a worker is bounded (rendezvous, device-side waits), so the
        # workers leave on their own, with a closing barrier, also when a check fails.
        outs = [p.communicate()[0] for p in procs]
        for r, p in enumerate(procs):
            assert p.returncode == 0 and "WORKER_OK {}".format(r) in outs[r], outs[r][-3000:]


def test_rendezvous_gives_up_on_a_rank_that_never_arrives(dgn_lib):
    """Failure made on the host: the second rank never shows up; creation
    returns DGN_ERR_TIMEOUT after the limit and no GPU work was started."""
    from dragon_b200 import _C
    from dragon_b200.comm import Communicator
    with tempfile.TemporaryDirectory() as rdv:
        with pytest.raises(_C.DgnError) as e:
            Communicator.create(0, 2, 0, rdv, "lonely", timeout_ms=300)
        assert e.value.status == _C.ERR_TIMEOUT and "never arrived" in str(e.value)
        assert os.listdir(rdv) == []


def test_rendezvous_ignores_files_of_a_run_that_died(dgn_lib):
    """Leftovers under the same tag -- this rank's own stale files, a peer's
    handle whose writer no longer exists, a stale ".ok" -- must not be taken for
    the peer: creation still ends with "never arrived", and removes its own files."""
    import struct
    from dragon_b200 import _C
    from dragon_b200.comm import Communicator
    donor = Communicator.init_local(1, 2, 0)
    try:
        stale = bytearray(donor.handle_bytes())
    finally:
        donor.destroy()
    struct.pack_into("<i", stale, 8, 4190000)  # pid field: a process that does not exist
    with tempfile.TemporaryDirectory() as rdv:
        for name, data in (("again.1.h", bytes(stale)), ("again.1.ok", b"\1" * 8), ("again.0.h", b"junk"),
                           ("again.0.ok", b"\1" * 8)):
            with open(os.path.join(rdv, name), "wb") as f:
                f.write(data)
        with pytest.raises(_C.DgnError) as e:
            Communicator.create(0, 2, 0, rdv, "again", timeout_ms=300)
        assert e.value.status == _C.ERR_TIMEOUT and "rank 1 never arrived" in str(e.value)
        assert sorted(os.listdir(rdv)) == ["again.1.h", "again.1.ok"]
