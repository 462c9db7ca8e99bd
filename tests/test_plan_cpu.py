"""Which kernel serves which message: the thresholds of the planner, queried
without a GPU (dgn_plan_query).  The expectations are the measured crossovers
the library documents: low-latency one-shot up to 2 MiB / 512 KiB / 128 KiB at
2 / 4 / 8 ranks, low-latency two-shot up to 2 MiB from 3 ranks, the store-only
two-shot kernel above, the staged ring through NVSwitch multicast from 16 MiB at
8 ranks, in place on symmetric memory from 4 MiB (never by default at 2 ranks)."""

import ctypes

import pytest

from dragon_b200 import _C

AR, RS, AG, BC = range(4)
KiB, MiB = 1 << 10, 1 << 20


def plan(lib, n, op, nbytes, dtype=_C.F32, redop=_C.MEAN, nvls=True, symm=0, in_symm=False, ntensors=1, sms=148):
    es = lib.dgn_dtype_size(dtype)
    v, b, t, r = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    cb = ctypes.c_int64()
    rc = lib.dgn_plan_query(n, sms, int(nvls), symm, int(in_symm), op, dtype, redop, nbytes // es, ntensors,
                            ctypes.byref(v), ctypes.byref(b), ctypes.byref(t), ctypes.byref(cb), ctypes.byref(r))
    assert rc == _C.OK, lib.dgn_last_error_string()
    return {"variant": v.value, "blocks": b.value, "threads": t.value, "chunk_bytes": cb.value, "rounds": r.value}


@pytest.fixture(autouse=True)
def clean_env(monkeypatch):
    for name in ("DGN_FORCE_VARIANT", "DGN_LL_MAX_BYTES", "DGN_LL2_MAX_BYTES", "DGN_ONESHOT_MAX_BYTES",
                 "DGN_NVLS_MIN_BYTES", "DGN_SYMM_MIN_BYTES", "DGN_NVLS_BCAST_MIN_BYTES", "DGN_FLOW_CHUNK_BYTES", "DGN_ALLGATHER_PULL_MIN_BYTES",
                 "DGN_FLOW_SWITCH_BLOCKS", "DGN_FLOW_DEPTH", "DGN_NVLS_RING_BYTES", "DGN_RING_BYTES",
                 "DGN_MAX_BLOCKS", "DGN_SLOT_BYTES", "DGN_LL_ALLGATHER_MAX_BYTES", "DGN_BCAST_SCATTER_MIN_BYTES",
                 "DGN_NVLS_ALLGATHER_MIN_BYTES", "DGN_ALLGATHER_RING_MIN_BYTES", "DGN_GATHER_CHUNK_BYTES",
                 "DGN_GATHER_PUSH_BLOCKS", "DGN_GATHER_FORWARD_BLOCKS", "DGN_GATHER_MODE", "DGN_BCAST_SHARD_MIN_BYTES",
                 "DGN_NVLS_GATHER_RING_BYTES"):
        monkeypatch.delenv(name, raising=False)


def test_allreduce_variant_by_size_and_rank_count(dgn_lib):
    expect = {
        2: [(1 * KiB, _C.VARIANT_LL), (1 * MiB, _C.VARIANT_LL), (2 * MiB, _C.VARIANT_LL), (3 * MiB, _C.VARIANT_TWOSHOT),
            (1024 * MiB, _C.VARIANT_TWOSHOT)],
        4: [(64 * KiB, _C.VARIANT_LL), (512 * KiB, _C.VARIANT_LL), (1 * MiB, _C.VARIANT_LL2),
            (2 * MiB, _C.VARIANT_LL2), (4 * MiB, _C.VARIANT_TWOSHOT), (1024 * MiB, _C.VARIANT_TWOSHOT)],
        8: [(1 * KiB, _C.VARIANT_LL), (128 * KiB, _C.VARIANT_LL), (256 * KiB, _C.VARIANT_LL2),
            (2 * MiB, _C.VARIANT_LL2), (4 * MiB, _C.VARIANT_TWOSHOT), (8 * MiB, _C.VARIANT_TWOSHOT),
            (16 * MiB, _C.VARIANT_NVLS), (32 * MiB, _C.VARIANT_NVLS), (256 * MiB, _C.VARIANT_NVLS), (1024 * MiB, _C.VARIANT_NVLS)],
    }
    for n, rows in expect.items():
        for nbytes, variant in rows:
            for dtype in (_C.F32, _C.F16):
                got = plan(dgn_lib, n, AR, nbytes, dtype)
                assert got["variant"] == variant, (n, nbytes, dtype, got)
    # Without the switch, integers and other reductions stay on the peer-store kernels.
    assert plan(dgn_lib, 8, AR, 512 * MiB, nvls=False)["variant"] == _C.VARIANT_TWOSHOT
    assert plan(dgn_lib, 8, AR, 512 * MiB, dtype=_C.I32, redop=_C.SUM)["variant"] == _C.VARIANT_TWOSHOT
    assert plan(dgn_lib, 8, AR, 512 * MiB, redop=_C.MAX)["variant"] == _C.VARIANT_TWOSHOT


def test_launch_shapes_stay_inside_the_workspace(dgn_lib):
    for n in (2, 4, 8):
        for nbytes in (4 * MiB, 64 * MiB, 1024 * MiB):
            p = plan(dgn_lib, n, AR, nbytes, nvls=False)
            assert 1 <= p["blocks"] <= 148 and p["chunk_bytes"] <= 128 * KiB  # one block per SM, one staging slot
            per_rank = -(-nbytes // n)
            assert p["blocks"] * p["chunk_bytes"] * p["rounds"] >= per_rank   # the rounds cover every shard
        p = plan(dgn_lib, n, AR, 64 * KiB)
        assert p["rounds"] == 1 and p["blocks"] <= 64 and p["chunk_bytes"] * 2 <= 64 * KiB  # lines are half flags
    # The staged ring: all blocks resident (they wait for one another), chunks
    # half of the message between 1 and 16 MiB, the ring never overrun.
    for nbytes, chunk, chunks in ((16 * MiB, 8 * MiB, 2), (32 * MiB, 16 * MiB, 2), (512 * MiB, 16 * MiB, 32),
                                  (100 * MiB + 16, None, 7)):
        p = plan(dgn_lib, 8, AR, nbytes)
        assert p["variant"] == _C.VARIANT_NVLS and 3 <= p["blocks"] <= 148 and p["rounds"] == chunks, p
        assert chunk is None or p["chunk_bytes"] == chunk
        assert p["chunk_bytes"] * p["rounds"] >= nbytes and p["chunk_bytes"] * 2 <= 256 * MiB
    p = plan(dgn_lib, 8, AR, 512 * MiB, ntensors=161)
    assert p["variant"] == _C.VARIANT_NVLS                            # buckets go the same way


def test_symmetric_memory_and_opt_in_variants(dgn_lib, monkeypatch):
    arena = 256 * MiB
    assert plan(dgn_lib, 8, AR, 64 * MiB, symm=arena, in_symm=True)["variant"] == _C.VARIANT_SYMM
    assert plan(dgn_lib, 4, AR, 4 * MiB, symm=arena, in_symm=True)["variant"] == _C.VARIANT_SYMM
    # Two ranks: the switch moves 1.5 S per direction where two-shot moves 1.0 S; off unless asked for.
    assert plan(dgn_lib, 2, AR, 256 * MiB, symm=arena, in_symm=True)["variant"] == _C.VARIANT_TWOSHOT
    monkeypatch.setenv("DGN_SYMM_MIN_BYTES", str(4 * MiB))
    assert plan(dgn_lib, 2, AR, 4 * MiB, symm=arena, in_symm=True)["variant"] == _C.VARIANT_SYMM
    monkeypatch.delenv("DGN_SYMM_MIN_BYTES")
    small = plan(dgn_lib, 8, AR, 1 * MiB, symm=arena, in_symm=True)
    assert small["variant"] == _C.VARIANT_LL2                       # below 4 MiB the low-latency kernels win
    assert plan(dgn_lib, 8, AR, 8 * MiB, symm=arena, in_symm=False)["variant"] == _C.VARIANT_TWOSHOT
    assert plan(dgn_lib, 8, AR, 64 * MiB, symm=arena, in_symm=False)["variant"] == _C.VARIANT_NVLS   # staged
    assert plan(dgn_lib, 8, AR, 64 * MiB + 4, symm=arena, in_symm=True)["variant"] == _C.VARIANT_NVLS  # ragged: staged
    assert plan(dgn_lib, 8, AR, 64 * MiB, symm=arena, in_symm=True, nvls=False)["variant"] == _C.VARIANT_TWOSHOT
    shape = plan(dgn_lib, 8, AR, 256 * MiB, symm=arena, in_symm=True)
    assert shape["blocks"] <= 16 and shape["threads"] == 256 and shape["rounds"] == 1
    # The broadcast through the switch: from 2 MiB at 5 ranks and more, opt-in
    # below; chunk size and block split of the staged ring can be set.
    assert plan(dgn_lib, 8, BC, 64 * MiB)["variant"] == _C.VARIANT_NVLS
    assert plan(dgn_lib, 8, BC, 64 * MiB, nvls=False)["variant"] == _C.VARIANT_TWOSHOT
    assert plan(dgn_lib, 4, BC, 64 * MiB)["variant"] == _C.VARIANT_TWOSHOT      # scatter + all-gather by stores
    assert plan(dgn_lib, 4, BC, 16 * MiB)["variant"] == _C.VARIANT_NVLS         # 4 ranks: the middle sizes only
    assert plan(dgn_lib, 4, BC, 16 * MiB)["rounds"] == 2
    assert plan(dgn_lib, 4, BC, 2 * MiB)["variant"] == _C.VARIANT_TWOSHOT
    assert plan(dgn_lib, 2, BC, 16 * MiB)["variant"] == _C.VARIANT_ONESHOT
    monkeypatch.setenv("DGN_NVLS_BCAST_MIN_BYTES", str(1 * MiB))
    monkeypatch.setenv("DGN_FLOW_CHUNK_BYTES", str(2 * MiB))
    monkeypatch.setenv("DGN_FLOW_SWITCH_BLOCKS", "32")
    ring = plan(dgn_lib, 8, AR, 64 * MiB)
    assert ring["variant"] == _C.VARIANT_NVLS and ring["rounds"] == 32 and ring["chunk_bytes"] == 2 * MiB
    assert plan(dgn_lib, 8, BC, 64 * MiB)["variant"] == _C.VARIANT_NVLS
    assert plan(dgn_lib, 8, BC, 64 * KiB)["variant"] == _C.VARIANT_ONESHOT


def test_allgather_and_broadcast_variants(dgn_lib):
    for n, limit in ((2, 512 * KiB), (4, 256 * KiB), (8, 64 * KiB)):
        assert plan(dgn_lib, n, AG, limit)["variant"] == _C.VARIANT_LL
        assert plan(dgn_lib, n, AG, limit * 2)["variant"] == _C.VARIANT_TWOSHOT
    assert plan(dgn_lib, 2, BC, 64 * MiB)["variant"] == _C.VARIANT_ONESHOT      # two ranks: peers pull
    assert plan(dgn_lib, 8, BC, 128 * KiB)["variant"] == _C.VARIANT_ONESHOT
    assert plan(dgn_lib, 8, BC, 1 * MiB)["variant"] == _C.VARIANT_ONESHOT
    assert plan(dgn_lib, 8, BC, 2 * MiB)["variant"] == _C.VARIANT_NVLS          # staged through the switch
    root_alone, shards = plan(dgn_lib, 8, BC, 16 * MiB), plan(dgn_lib, 8, BC, 64 * MiB)
    assert root_alone["rounds"] == 2 and root_alone["chunk_bytes"] == 8 * MiB   # the root multicasts halves
    assert shards["rounds"] == 8 and shards["chunk_bytes"] == 1 * MiB           # 8 MiB chunks, a shard per rank
    assert plan(dgn_lib, 8, BC, 2 * MiB, nvls=False)["variant"] == _C.VARIANT_TWOSHOT   # scatter + all-gather
    assert plan(dgn_lib, 8, AG, 4 * MiB)["variant"] == _C.VARIANT_TWOSHOT       # push
    assert plan(dgn_lib, 8, AG, 16 * MiB)["variant"] == _C.VARIANT_ONESHOT      # pull
    assert plan(dgn_lib, 4, AG, 64 * MiB)["variant"] == _C.VARIANT_TWOSHOT
    assert plan(dgn_lib, 4, BC, 1 * MiB)["variant"] == _C.VARIANT_TWOSHOT
    assert plan(dgn_lib, 4, RS, 16 * MiB)["variant"] == _C.VARIANT_TWOSHOT


def test_staged_gather_shapes_cover_the_message(dgn_lib, monkeypatch):
    """All-gather and broadcast as staged kernels (through the switch, with remote
    stores, pulling): the chunks cover every source's bytes, the grid fits the
    device, and a ring that is too small makes the planner fall back."""
    for forced, nvls in ((3, True), (7, False), (8, False)):
        monkeypatch.setenv("DGN_FORCE_VARIANT", str(forced))
        for n in (2, 3, 4, 8):
            for nbytes in (16, 1 * KiB, 100 * KiB + 16, 4 * MiB, 64 * MiB + 48, 1024 * MiB):
                ag = plan(dgn_lib, n, AG, nbytes, dtype=_C.U8, redop=_C.SUM, nvls=nvls)
                assert ag["variant"] == forced and 2 <= ag["blocks"] <= 148, (forced, n, nbytes, ag)
                assert ag["chunk_bytes"] * ag["rounds"] >= nbytes and ag["chunk_bytes"] <= 4 * MiB
                bc = plan(dgn_lib, n, BC, nbytes, dtype=_C.U8, redop=_C.SUM, nvls=nvls)
                if forced == 8:
                    assert bc["variant"] in (_C.VARIANT_ONESHOT, _C.VARIANT_TWOSHOT)   # pulling is an all-gather mode
                    continue
                assert bc["variant"] == forced and 2 <= bc["blocks"] <= 148, (forced, n, nbytes, bc)
                # chunk_bytes is per source: the root alone, or one shard per rank
                sources = n if (n >= 5 and nbytes >= 32 * MiB) else 1
                assert bc["chunk_bytes"] * sources * bc["rounds"] >= nbytes, (forced, n, nbytes, bc)
    # Without the ring in the workspace the remote-store form is not offered.
    monkeypatch.setenv("DGN_RING_BYTES", "0")
    monkeypatch.setenv("DGN_FORCE_VARIANT", "7")
    assert plan(dgn_lib, 8, AG, 4 * MiB, nvls=False)["variant"] == _C.VARIANT_TWOSHOT
    assert plan(dgn_lib, 8, BC, 4 * MiB, nvls=False)["variant"] in (_C.VARIANT_ONESHOT, _C.VARIANT_TWOSHOT)
    # ... and the broadcast through the switch goes back to the root alone (the inboxes of the scattered form lie there).
    monkeypatch.delenv("DGN_FORCE_VARIANT")
    alone = plan(dgn_lib, 8, BC, 64 * MiB)
    assert alone["variant"] == _C.VARIANT_NVLS and alone["chunk_bytes"] == 8 * MiB and alone["rounds"] == 8


def staged(lib, n, op, nbytes, nvls=True, sms=148):
    out = _C.StagedPlan()
    assert lib.dgn_plan_query_staged(n, sms, int(nvls), op, nbytes, ctypes.byref(out)) == _C.OK, lib.dgn_last_error_string()
    return out


@pytest.mark.parametrize("ring_bytes", [None, 64 * MiB, 1 * MiB, 64 * KiB])
def test_staged_plans_stay_inside_their_rings(dgn_lib, monkeypatch, ring_bytes):
    """Memory safety of the staged kernels' plans, for every staged variant,
    rank count, grid size and ring size: the ring slots in use fit the ring,
    the inboxes of the scattered broadcast fit what is left for them, every
    role keeps at least one block, the chunks cover the message."""
    if ring_bytes is not None:
        monkeypatch.setenv("DGN_RING_BYTES", str(ring_bytes))
        monkeypatch.setenv("DGN_NVLS_RING_BYTES", str(4 * ring_bytes))
        monkeypatch.setenv("DGN_NVLS_GATHER_RING_BYTES", str(2 * ring_bytes))
    seen = set()
    for forced, nvls in ((0, True), (3, True), (7, False), (8, False)):
        monkeypatch.setenv("DGN_FORCE_VARIANT", str(forced))
        for mode in (0, 1, 2):
            monkeypatch.setenv("DGN_GATHER_MODE", str(mode))
            for n in (2, 3, 4, 5, 8):
                for sms in (148, 18, 4):
                    for op in (AR, AG, BC):
                        for nbytes in (16, 48, 4 * KiB, 100 * KiB + 16, 3 * MiB, 16 * MiB, 64 * MiB + 48, 1024 * MiB):
                            p = staged(dgn_lib, n, op, nbytes, nvls=nvls, sms=sms)
                            if not p.staged:
                                continue
                            what = (forced, mode, n, sms, op, nbytes, p.variant, p.mode, p.depth, p.chunk_vectors, p.chunks)
                            seen.add((op, p.variant, p.mode))
                            assert p.variant in (_C.VARIANT_NVLS, _C.VARIANT_RING, _C.VARIANT_RING_PULL), what
                            assert 1 <= p.depth <= 8 and p.chunk_vectors >= 1 and p.chunks >= 1, what
                            assert p.ring_bytes_needed <= p.ring_bytes_available, what
                            assert p.inbox_bytes_needed <= p.inbox_bytes_available, what
                            assert p.blocks <= min(sms, 160), what
                            vectors = -(-nbytes // 16)
                            if op == AR:
                                assert p.chunk_vectors % n == 0, what                       # equal shards
                                assert p.first_role_blocks >= 1 and p.second_role_blocks >= 1, what
                                assert p.blocks - p.first_role_blocks - p.second_role_blocks >= 1, what
                                assert p.chunk_vectors * p.chunks >= vectors, what
                            else:
                                sources = n if (op == AG or p.mode & 1) else 1
                                assert p.first_role_blocks >= 1 and p.blocks - p.first_role_blocks >= 1, what
                                if p.mode & 1:
                                    assert p.second_role_blocks >= 1 and p.blocks - p.second_role_blocks >= 1, what
                                    assert p.inbox_bytes_needed == p.depth * p.chunk_vectors * 16, what
                                per_chunk = p.chunk_vectors * (1 if op == AG else sources)
                                assert per_chunk * p.chunks >= vectors, what
                                assert p.threads >= 64, what
    if ring_bytes is None:
        # every staged form was met: all-reduce ring (switch, peer), gather (switch, stores, loads), broadcast alone and scattered
        assert {(AR, 3, 0), (AR, 7, 0), (AG, 3, 0), (AG, 7, 0), (AG, 8, 2), (BC, 3, 0), (BC, 3, 1), (BC, 7, 0), (BC, 7, 1)} <= seen, seen


def test_environment_overrides(dgn_lib, monkeypatch):
    monkeypatch.setenv("DGN_FORCE_VARIANT", "2")
    assert plan(dgn_lib, 8, AR, 1 * KiB)["variant"] == _C.VARIANT_TWOSHOT
    monkeypatch.delenv("DGN_FORCE_VARIANT")
    monkeypatch.setenv("DGN_LL_MAX_BYTES", "0")
    monkeypatch.setenv("DGN_LL2_MAX_BYTES", "0")
    assert plan(dgn_lib, 8, AR, 64 * KiB)["variant"] == _C.VARIANT_ONESHOT
    assert plan(dgn_lib, 8, AR, 512 * KiB)["variant"] == _C.VARIANT_TWOSHOT
    monkeypatch.setenv("DGN_NVLS_MIN_BYTES", str(64 * MiB))
    assert plan(dgn_lib, 4, AR, 64 * MiB)["variant"] == _C.VARIANT_NVLS


def test_bad_queries_are_rejected(dgn_lib):
    z = ctypes.c_int()
    cb = ctypes.c_int64()
    args = (ctypes.byref(z), ctypes.byref(z), ctypes.byref(z), ctypes.byref(cb), ctypes.byref(z))
    assert dgn_lib.dgn_plan_query(1, 148, 1, 0, 0, AR, _C.F32, _C.SUM, 1024, 1, *args) == _C.ERR_ARG
    assert dgn_lib.dgn_plan_query(8, 148, 1, 0, 0, 7, _C.F32, _C.SUM, 1024, 1, *args) == _C.ERR_ARG
    assert dgn_lib.dgn_plan_query(8, 148, 1, 0, 0, AR, 99, _C.SUM, 1024, 1, *args) == _C.ERR_ARG
    assert dgn_lib.dgn_plan_query(8, 148, 1, 0, 0, AR, _C.F32, _C.SUM, 0, 1, *args) == _C.ERR_ARG
