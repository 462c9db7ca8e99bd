"""The CPU oracle against REFERENCE code: the 16-bit float converters of
dragon/utils/conversions.h:42-149 and the CPU optimizer loops of
dragon/kernels/training/cpu/adam_kernel.cc:11-57 and sgd_kernel.cc:10-45.

Two routes.  The committed vectors (tests/golden/reference_vectors.npz, written
by tests/golden/make_reference_vectors.py from the compiled reference files)
always apply.  Where the reference tree is present the same functions are also
compiled and called directly (oracle.ref_lib())."""

import os
import sys

import numpy as np
import pytest

from oracle import oracle

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_reference_vectors as gen  # noqa: E402

VEC = np.load(os.path.join(HERE, "golden", "reference_vectors.npz"))


def oracle_f32_to_16(bits, name):
    fn = getattr(oracle.lib(), name)
    f = bits.view(np.float32)
    return np.fromiter((fn(float(x)) if x == x else fn(float("nan")) for x in f), dtype=np.uint16, count=f.size)


def oracle_convert_array(bits, dtype):
    """fp32 bit patterns -> 16-bit storage through the oracle's vector path
    (what the collectives and the sharded step use)."""
    return np.ascontiguousarray(oracle.from_f32(bits.view(np.float32), dtype)).view(np.uint16)


def test_all_half_patterns_widen_like_the_reference():
    lib = oracle.lib()
    want = VEC["f16_to_f32_bits"]
    got = np.array([np.float32(lib.orc_f16_to_f32(b)).view(np.uint32) for b in range(65536)], dtype=np.uint32)
    nan = (np.arange(65536) & 0x7FFF) > 0x7C00
    # Not-a-number inputs: the reference widens every NaN to 0x7fffffff
    # (conversions.h:120-124 drops the sign and fills the mantissa); the oracle
    # keeps sign and payload, as the hardware conversion does.  Both are NaNs.
    assert np.array_equal(got[~nan], want[~nan])
    assert np.all((want[nan] & 0x7FFFFFFF) > 0x7F800000) and np.all((got[nan] & 0x7FFFFFFF) > 0x7F800000)
    want = VEC["bf16_to_f32_bits"]
    got = np.array([np.float32(lib.orc_bf16_to_f32(b)).view(np.uint32) for b in range(65536)], dtype=np.uint32)
    # Signalling NaNs are quieted on their way back through the C float return
    # of the scalar entry point; the bit pattern itself is a 16-bit shift in both.
    nan = (np.arange(65536) & 0x7FFF) > 0x7F80
    assert np.array_equal(got[~nan], want[~nan])
    assert np.all((got[nan] & 0x7FFFFFFF) > 0x7F800000) and np.all((want[nan] & 0x7FFFFFFF) > 0x7F800000)
    assert np.array_equal(oracle.bf16_bits_to_f32(np.arange(65536, dtype=np.uint16)).view(np.uint32), want)


@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_narrowing_matches_the_reference(kind):
    bits = gen.f32_samples()
    want = VEC["f32_to_" + kind]
    dtype = oracle.F16 if kind == "f16" else oracle.BF16
    got = oracle_convert_array(bits, dtype)
    a = bits & 0x7FFFFFFF
    nan = a > 0x7F800000
    # NaN: the reference returns 0x7fff whatever the input's sign and payload
    # (conversions.h:51, :91); the oracle's vector path keeps numpy's quiet NaN
    # for float16.  Everything that is not a NaN must agree bit for bit --
    # including float32 values above the float16 range: conversions.h:52-54
    # clamps them to 0x7bff with a remainder of exactly one half, which the
    # round-to-nearest-even step at :73-76 then bumps to 0x7c00, infinity, the
    # same answer IEEE rounding gives.
    assert np.array_equal(got[~nan], want[~nan])
    assert np.all((want[nan] & 0x7FFF) > (0x7C00 if kind == "f16" else 0x7F80))
    assert np.all((got[nan] & 0x7FFF) > (0x7C00 if kind == "f16" else 0x7F80))
    # The scalar entry points of the C oracle agree with its vector path.
    sample = bits[::37]
    scalar = oracle_f32_to_16(sample, "orc_f32_to_" + kind)
    keep = ~nan[::37]
    assert np.array_equal(scalar[keep], want[::37][keep])


def test_float16_overflow_rounds_to_infinity_in_both():
    big = np.array([0x477FF000, 0x47800000, 0x7F7FFFFF, 0xC77FF000], dtype=np.uint32)
    got = oracle_convert_array(big, oracle.F16)
    assert list(got) == [0x7C00, 0x7C00, 0x7C00, 0xFC00]
    ref = oracle.ref_lib()
    if ref is not None:
        out = np.empty(4, np.uint16)
        ref.ref_f32_to_f16(big.view(np.float32).ctypes.data, out.ctypes.data, 4)
        assert list(out) == [0x7C00, 0x7C00, 0x7C00, 0xFC00]


def _run_oracle(name, wd, nesterov=False):
    y0, grads = gen.optimizer_inputs()
    n = y0.size
    y, m, v = y0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    h = gen.HYPER
    for g in grads:
        if name == "adamw":
            oracle.adamw(g, m, v, y, h["lr"], h["beta1"], h["beta2"], h["eps"], wd)
        elif name == "adam":
            oracle.adam(g, m, v, y, h["lr"], h["beta1"], h["beta2"], h["eps"], wd)
        else:
            oracle.momentum_sgd(g, m, y, h["lr"], h["momentum"], wd, nesterov)
    return y, m, v


@pytest.mark.parametrize("wd", [0.0, 0.01])
@pytest.mark.parametrize("name", ["adamw", "adam"])
def test_adam_loops_match_the_reference_over_three_steps(name, wd):
    tag = "wd" if wd > 0 else "nowd"
    y, m, v = _run_oracle(name, wd)
    for arr, key in ((y, "y"), (m, "m"), (v, "v")):
        assert np.array_equal(arr.view(np.uint32), VEC["{}_{}_{}".format(name, tag, key)].view(np.uint32)), key
    # The low-precision copy the loop writes (y_copy) is convert::To of y.
    assert np.array_equal(np.ascontiguousarray(oracle.from_f32(y, oracle.F16)).view(np.uint16),
                          VEC["{}_{}_y_f16".format(name, tag)])


@pytest.mark.parametrize("wd", [0.0, 0.01])
@pytest.mark.parametrize("nesterov", [False, True])
def test_sgd_loops_match_the_reference_over_three_steps(nesterov, wd):
    tag = "wd" if wd > 0 else "nowd"
    y, m, _ = _run_oracle("sgd", wd, nesterov)
    key = "{}_{}".format("nesterov" if nesterov else "momentum", tag)
    assert np.array_equal(y.view(np.uint32), VEC[key + "_y"].view(np.uint32))
    assert np.array_equal(m.view(np.uint32), VEC[key + "_m"].view(np.uint32))
    assert np.array_equal(oracle.from_f32(y, oracle.BF16), VEC[key + "_y_bf16"])


def test_committed_vectors_are_what_the_reference_code_gives():
    """Where the reference tree is present, recompute every vector from the
    compiled reference files and compare with the committed file."""
    if oracle.ref_lib() is None:
        pytest.skip("the reference tree is not on this machine; the committed vectors were used above")
    fresh = gen.run_reference()
    assert sorted(fresh) == sorted(VEC.files)
    for key, val in fresh.items():
        assert np.array_equal(np.ascontiguousarray(val).view(np.uint8), np.ascontiguousarray(VEC[key]).view(np.uint8)), key
