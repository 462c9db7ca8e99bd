"""Shared helpers of the parity tests: seeded per-rank inputs in every dtype,
numpy <-> torch conversion that keeps bit patterns, oracle comparison."""

import numpy as np
import torch

from oracle import oracle

TORCH_DTYPE = {
    oracle.U8: torch.uint8, oracle.I8: torch.int8, oracle.I32: torch.int32, oracle.I64: torch.int64,
    oracle.F16: torch.float16, oracle.BF16: torch.bfloat16, oracle.F32: torch.float32,
    oracle.F64: torch.float64,
}
ALL_DTYPES = list(range(8))
FLOAT_DTYPES = [oracle.F16, oracle.BF16, oracle.F32, oracle.F64]
NAMES = ["u8", "i8", "i32", "i64", "f16", "bf16", "f32", "f64"]


def make_input(rank, count, dtype, seed=1000, lo=-1.0, hi=1.0):
    """Per-rank message as a numpy array in oracle storage (bf16 = uint16 bits)."""
    rng = np.random.default_rng(seed + rank)
    if dtype in (oracle.U8, oracle.I8, oracle.I32, oracle.I64):
        st = oracle.NP_STORAGE[dtype]
        info = np.iinfo(st)
        return rng.integers(info.min, info.max, count, dtype=st, endpoint=True)
    x = rng.uniform(lo, hi, count).astype(np.float32)
    if dtype == oracle.F32:
        return x
    if dtype == oracle.F64:
        return rng.uniform(lo, hi, count)
    if dtype == oracle.F16:
        return x.astype(np.float16)
    return oracle.f32_to_bf16_bits(x)


def to_torch(arr, dtype, device):
    """numpy storage -> torch tensor of the real dtype, same bits."""
    t = torch.from_numpy(np.ascontiguousarray(arr).copy())
    if dtype == oracle.BF16:
        t = t.view(torch.int16).view(torch.bfloat16) if t.dtype != torch.uint16 else t.view(torch.bfloat16)
    return t.to(device)


def to_numpy(t, dtype):
    """torch tensor -> numpy storage array, same bits."""
    t = t.detach().cpu().contiguous()
    if dtype == oracle.BF16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def assert_bits_equal(got, want, what=""):
    got = np.ascontiguousarray(got).reshape(-1).view(np.uint8)
    want = np.ascontiguousarray(want).reshape(-1).view(np.uint8)
    assert got.size == want.size, "{}: size {} != {}".format(what, got.size, want.size)
    if not np.array_equal(got, want):
        bad = np.flatnonzero(got != want)
        raise AssertionError("{}: {} of {} bytes differ, first at byte {}".format(
            what, bad.size, got.size, int(bad[0])))
