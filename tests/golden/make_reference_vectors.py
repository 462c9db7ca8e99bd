"""Writes tests/golden/reference_vectors.npz: outputs of REFERENCE code.

Run where the Dragon source tree is present (its location: the environment
variable DRAGON_REFERENCE, else the recipe's default): `make -C oracle ref` compiles dragon/utils/conversions.h and
dragon/kernels/training/cpu/{adam,sgd}_kernel.cc where they lie, and this script
runs them on seeded inputs.  The committed file lets a machine without the
reference tree still check the oracle against the reference's own arithmetic
(tests/test_oracle_ref.py regenerates the inputs from the same seeds).

    python tests/golden/make_reference_vectors.py
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle  # noqa: E402

OUT = os.path.join(HERE, "reference_vectors.npz")


def f32_samples():
    """fp32 bit patterns that stress the converters: random patterns over the
    whole encoding, every float16 value, its neighbours and the exact ties
    between neighbouring float16 / bfloat16 values."""
    rng = np.random.default_rng(2024)
    rand = rng.integers(0, 1 << 32, 30000, dtype=np.uint64).astype(np.uint32)
    halves = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32).view(np.uint32)
    finite = halves[np.isfinite(halves.view(np.float32))]
    some = finite[::5]
    near = np.concatenate([some + 1, some - 1, some + 0x1000, some + 0x0FFF, some + 0x1001])
    bf_ties = (rng.integers(0, 1 << 16, 4096, dtype=np.uint32) << 16) | 0x8000
    edge = np.array([0x477FEFFF, 0x477FF000, 0x477FF001, 0x47800000, 0x7F7FFFFF, 0xC77FF000, 0x33000000,
                     0x33000001, 0x387FFFFF, 0x38800000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00001,
                     0x7F800001, 0x00000000, 0x80000000, 0x00000001, 0x7F7F8000, 0x7F7F7FFF], dtype=np.uint32)
    return np.concatenate([rand, halves, near.astype(np.uint32), bf_ties.astype(np.uint32), edge])


def optimizer_inputs(n=4099, seed=77):
    rng = np.random.default_rng(seed)
    y0 = rng.normal(0, 1, n).astype(np.float32)
    grads = [rng.normal(0, 1e-2, n).astype(np.float32) for _ in range(3)]
    return y0, grads


HYPER = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, momentum=0.9)


def run_reference():
    ref = oracle.ref_lib()
    if ref is None:
        raise SystemExit("the reference tree is not available; nothing written")
    out = {}
    bits = f32_samples()
    f = bits.view(np.float32)
    h = np.empty(f.size, np.uint16)
    ref.ref_f32_to_f16(f.ctypes.data, h.ctypes.data, f.size)
    out["f32_to_f16"] = h.copy()
    ref.ref_f32_to_bf16(f.ctypes.data, h.ctypes.data, f.size)
    out["f32_to_bf16"] = h.copy()
    allh = np.arange(65536, dtype=np.uint16)
    w = np.empty(65536, np.float32)
    ref.ref_f16_to_f32(allh.ctypes.data, w.ctypes.data, 65536)
    out["f16_to_f32_bits"] = w.view(np.uint32).copy()
    ref.ref_bf16_to_f32(allh.ctypes.data, w.ctypes.data, 65536)
    out["bf16_to_f32_bits"] = w.view(np.uint32).copy()

    y0, grads = optimizer_inputs()
    n = y0.size
    for wd in (0.0, 0.01):
        tag = "wd" if wd > 0 else "nowd"
        for name in ("adamw", "adam"):
            y, m, v = y0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
            c16 = np.zeros(n, np.uint16)
            for g in grads:
                fn = getattr(ref, "ref_" + name)
                # x and y are the same array, as in the update operators.
                fn(n, HYPER["lr"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"], wd, y.ctypes.data, g.ctypes.data,
                   m.ctypes.data, v.ctypes.data, y.ctypes.data, c16.ctypes.data, 1)
            out["{}_{}_y".format(name, tag)] = y.copy()
            out["{}_{}_m".format(name, tag)] = m.copy()
            out["{}_{}_v".format(name, tag)] = v.copy()
            out["{}_{}_y_f16".format(name, tag)] = c16.copy()
        for nesterov in (0, 1):
            y, m = y0.copy(), np.zeros(n, np.float32)
            cb16 = np.zeros(n, np.uint16)
            for g in grads:
                ref.ref_momentum_sgd(n, HYPER["lr"], HYPER["momentum"], wd, y.ctypes.data, g.ctypes.data,
                                     m.ctypes.data, y.ctypes.data, cb16.ctypes.data, 2, nesterov)
            key = "{}_{}".format("nesterov" if nesterov else "momentum", tag)
            out[key + "_y"] = y.copy()
            out[key + "_m"] = m.copy()
            out[key + "_y_bf16"] = cb16.copy()
    return out


if __name__ == "__main__":
    np.savez_compressed(OUT, **run_reference())
    print("wrote", OUT, os.path.getsize(OUT), "bytes")
