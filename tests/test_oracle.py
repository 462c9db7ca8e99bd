"""The CPU oracle against the committed golden vectors (numpy arithmetic that
is independent of the oracle's C code) and against its own invariants."""

import os

import numpy as np
import pytest

from oracle import oracle

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "collective_golden.npz"))
KINDS = {"u8": oracle.U8, "i8": oracle.I8, "i32": oracle.I32, "i64": oracle.I64, "f16": oracle.F16,
         "bf16": oracle.BF16, "f32": oracle.F32, "f64": oracle.F64}


def bits(a):
    return np.ascontiguousarray(a).view(np.uint8)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("kind", list(KINDS))
def test_allreduce_matches_golden(n, kind):
    key = "n{}_{}".format(n, kind)
    bufs = list(GOLDEN[key + "_in"])
    got = oracle.allreduce(bufs, KINDS[kind], "SUM")
    assert np.array_equal(bits(got), bits(GOLDEN[key + "_sum"]))
    if key + "_mean" in GOLDEN:
        got = oracle.allreduce(bufs, KINDS[kind], "MEAN")
        assert np.array_equal(bits(got), bits(GOLDEN[key + "_mean"]))


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("kind", ["i64", "bf16", "u8"])
def test_allgather_broadcast_match_golden(n, kind):
    key = "n{}_{}".format(n, kind)
    bufs = list(GOLDEN[key + "_in"])
    assert np.array_equal(bits(oracle.allgather(bufs, KINDS[kind])), bits(GOLDEN[key + "_gather"]))
    for root in (0, n - 1):
        out = oracle.broadcast(bufs, KINDS[kind], root)
        assert all(np.array_equal(bits(o), bits(bufs[root])) for o in out)


def test_tolerance_contract_against_fp64_sum():
    for kind, tol in ((oracle.F32, 1e-6), (oracle.F16, 2e-3), (oracle.BF16, 1e-2)):
        for n in (2, 4, 8):
            bufs = list(GOLDEN["n{}_{}_in".format(n, {oracle.F32: "f32", oracle.F16: "f16", oracle.BF16: "bf16"}[kind])])
            for mean in (False, True):
                got = oracle.allreduce(bufs, kind, "MEAN" if mean else "SUM")
                assert oracle.max_rel_err(got, oracle.fp64_sum(bufs, kind, mean), kind) <= tol


def test_mean_rejected_for_integers():
    with pytest.raises(ValueError):
        oracle.allreduce([np.zeros(4, np.int32)] * 2, oracle.I32, "MEAN")


def test_float16_converters_over_all_bit_patterns():
    lib = oracle.lib()
    want = GOLDEN["f16_all_bits_as_f32"]
    for b in range(0, 65536):
        got = np.float32(lib.orc_f16_to_f32(b))
        if np.isnan(want[b]):
            assert np.isnan(got)
        else:
            assert got.view(np.uint32) == want[b].view(np.uint32), hex(b)
        if not np.isnan(want[b]):  # every half value converts back to itself
            assert lib.orc_f32_to_f16(float(want[b])) == b, hex(b)


def test_rounding_edges():
    lib = oracle.lib()
    for x, b in zip(GOLDEN["f16_edge_in"], GOLDEN["f16_edge_bits"]):
        assert lib.orc_f32_to_f16(float(x)) == int(b), float(x)
    for x, b in zip(GOLDEN["bf16_edge_in"], GOLDEN["bf16_edge_bits"]):
        assert lib.orc_f32_to_bf16(float(x)) == int(b), float(x)
    assert lib.orc_f32_to_f16(float("nan")) == 0x7FFF
    assert lib.orc_f32_to_bf16(float("nan")) == 0x7FFF


def test_reducescatter_is_a_slice_of_allreduce():
    n, count = 4, 37
    bufs = [np.random.default_rng(r).uniform(-1, 1, n * count).astype(np.float32) for r in range(n)]
    full = oracle.allreduce(bufs, oracle.F32, "SUM")
    parts = oracle.reducescatter(bufs, oracle.F32, "SUM")
    for r in range(n):
        assert np.array_equal(parts[r], full[r * count:(r + 1) * count])


def test_multi_process_runner_matches_single_process():
    """The MPI-shaped runner (2 and 3 forked rank processes) gives the oracle's bits."""
    for n in (2, 3):
        bufs = [np.random.default_rng(10 + r).uniform(-1, 1, 10007).astype(np.float32) for r in range(n)]
        secs, out = oracle.mp_allreduce(bufs, oracle.F32, "MEAN", iters=2)
        assert len(secs) == 2 and all(s > 0 for s in secs)
        assert np.array_equal(out, oracle.allreduce(bufs, oracle.F32, "MEAN"))


def test_empty_message():
    out = oracle.allreduce([np.zeros(0, np.float32)] * 2, oracle.F32, "SUM")
    assert out.size == 0
