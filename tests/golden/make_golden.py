"""Generates tests/golden/collective_golden.npz.

The reference has no golden vectors for the Collective path and cannot be
imported on this machine, so these vectors are produced by plain numpy
arithmetic that is independent of the C oracle: sequential np.float32 adds in
ascending rank order, numpy's own float16 rounding, integer adds that wrap,
and concatenation / copies for ALLGATHER / BROADCAST.  The C oracle (and,
through it, the CUDA kernels) must reproduce them bit for bit.

    python tests/golden/make_golden.py
"""

import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
COUNT = 53
RANKS = (2, 4, 8)


def bf16_round(x32):
    """fp32 -> bf16 bits, round to nearest even, written with integer ops only."""
    u = x32.astype(np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def make_inputs(n, kind, seed):
    rng = np.random.default_rng(seed)
    out = []
    for r in range(n):
        if kind in ("u8", "i8", "i32", "i64"):
            dt = {"u8": np.uint8, "i8": np.int8, "i32": np.int32, "i64": np.int64}[kind]
            info = np.iinfo(dt)
            out.append(rng.integers(info.min, info.max, COUNT, dtype=dt, endpoint=True))
        else:
            x = rng.uniform(-1, 1, COUNT).astype(np.float32)
            if kind == "f32":
                out.append(x)
            elif kind == "f64":
                out.append(rng.uniform(-1, 1, COUNT))
            elif kind == "f16":
                out.append(x.astype(np.float16))
            else:
                out.append(bf16_round(x))
    return out


def reduce_numpy(bufs, kind, mean):
    n = len(bufs)
    if kind in ("u8", "i8", "i32", "i64"):
        acc = bufs[0].copy()
        with np.errstate(over="ignore"):
            for b in bufs[1:]:
                acc = (acc + b).astype(acc.dtype)  # wraps modulo 2^k
        return acc
    if kind == "f64":
        acc = bufs[0].copy()
        for b in bufs[1:]:
            acc = acc + b
        return acc * np.float64(np.float32(1.0) / np.float32(n)) if mean else acc
    if kind == "f32":
        acc = bufs[0].copy()
        for b in bufs[1:]:
            acc = (acc + b).astype(np.float32)
        return (acc * (np.float32(1.0) / np.float32(n))).astype(np.float32) if mean else acc
    wide = [b.astype(np.float32) if kind == "f16" else bf16_to_f32(b) for b in bufs]
    acc = wide[0].copy()
    for b in wide[1:]:
        acc = (acc + b).astype(np.float32)
    if mean:
        acc = (acc * (np.float32(1.0) / np.float32(n))).astype(np.float32)
    return acc.astype(np.float16) if kind == "f16" else bf16_round(acc)


def main():
    data = {}
    seed = 4242
    for n in RANKS:
        for kind in ("u8", "i8", "i32", "i64", "f16", "bf16", "f32", "f64"):
            seed += 1
            bufs = make_inputs(n, kind, seed)
            key = "n{}_{}".format(n, kind)
            data[key + "_in"] = np.stack(bufs)
            data[key + "_sum"] = reduce_numpy(bufs, kind, False)
            if kind in ("f16", "bf16", "f32", "f64"):
                data[key + "_mean"] = reduce_numpy(bufs, kind, True)
            data[key + "_gather"] = np.concatenate(bufs)
    # Special values that must travel untouched / round as IEEE says.
    data["f16_all_bits_as_f32"] = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    edge = np.array([65504.0, 65519.99, 65520.0, 70000.0, -70000.0, 5.9604645e-08, 2.9802322e-08,
                     2.9802326e-08, 6.1035156e-05, 6.0975552e-05, 0.0, -0.0, np.inf, -np.inf, 1.0009766,
                     1.0004883, 1.0014648], dtype=np.float32)
    data["f16_edge_in"] = edge
    with np.errstate(over="ignore"):
        data["f16_edge_bits"] = edge.astype(np.float16).view(np.uint16)
    data["bf16_edge_in"] = np.array([1.0, 1.00390625, 1.01171875, 3.3895314e38, -1.1754944e-38, 1e-40, 0.1, -0.3],
                                    dtype=np.float32)
    data["bf16_edge_bits"] = bf16_round(data["bf16_edge_in"])
    np.savez_compressed(os.path.join(HERE, "collective_golden.npz"), **data)
    print("wrote", os.path.join(HERE, "collective_golden.npz"), len(data), "arrays")


if __name__ == "__main__":
    main()
