"""Python face of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Two checkers live here:

* the C restatement of the `Collective` operator (collective_oracle.c, built
  into liboracle.so by the Makefile beside it), bit-exact target for the CUDA
  path -- ascending-rank order, fp32 accumulation for fp16/bf16, one rounding;
* the fp64 host sum the tolerance contract is written against
  (max relative error 1e-6 fp32 / 2e-3 fp16 / 1e-2 bf16).

PARITY: the 16-bit converters and the optimizer loops are pinned to reference
code (`ref_lib()`: oracle/_ref/libdragon_ref.so, compiled by `make -C oracle ref`
from dragon/utils/conversions.h and dragon/kernels/training/cpu/*.cc where they
lie; tests/test_oracle_ref.py).  The reduction order of the collectives stays
unpinned: the reference has no golden vectors for them and its MPI library is
absent; see the header of collective_oracle.c.  Only tests, the smoke check and
the benchmark's CPU baseline may import this module.
"""

import ctypes
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_DIR, "liboracle.so")

U8, I8, I32, I64, F16, BF16, F32, F64 = range(8)
SUM, MEAN, PROD, MIN, MAX = range(5)
REDOPS = {"SUM": SUM, "MEAN": MEAN, "PROD": PROD, "MIN": MIN, "MAX": MAX}

# numpy storage type per dtype code (bf16 travels as its uint16 bit pattern).
NP_STORAGE = {U8: np.uint8, I8: np.int8, I32: np.int32, I64: np.int64, F16: np.float16,
              BF16: np.uint16, F32: np.float32, F64: np.float64}
TOLERANCE = {F32: 1e-6, F16: 2e-3, BF16: 1e-2, F64: 1e-12}

_lib = None


def build():
    """Compile liboracle.so if it is missing or older than its source."""
    src = os.path.join(_DIR, "collective_oracle.c")
    if not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _DIR, "liboracle.so"], check=True, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT)
    return _LIB


_REF_LIB = os.path.join(_DIR, "_ref", "libdragon_ref.so")
_REFERENCE = os.environ.get("DRAGON_REFERENCE", "/root/reference")
_ref = None


def build_ref():
    """Compile the reference's converters and CPU optimizer loops (Makefile
    target `ref`) when the reference tree is present; returns the library path
    or None.  A prebuilt library is used as it is where the tree is absent."""
    if os.path.isdir(os.path.join(_REFERENCE, "dragon", "utils")):
        subprocess.run(["make", "-C", _DIR, "ref", "REFERENCE=" + _REFERENCE], check=True, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT)
    return _REF_LIB if os.path.exists(_REF_LIB) else None


def ref_lib():
    """ctypes handle of the compiled reference pieces, or None if unavailable."""
    global _ref
    if _ref is None:
        path = build_ref()
        if path is None:
            return None
        h = ctypes.CDLL(path)
        for name in ("ref_f32_to_f16", "ref_f16_to_f32", "ref_f32_to_bf16", "ref_bf16_to_f32"):
            getattr(h, name).restype = None
            getattr(h, name).argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
        for name in ("ref_adamw", "ref_adam"):
            getattr(h, name).restype = None
            getattr(h, name).argtypes = [ctypes.c_int] + [ctypes.c_float] * 5 + [ctypes.c_void_p] * 6 + [ctypes.c_int]
        h.ref_momentum_sgd.restype = None
        h.ref_momentum_sgd.argtypes = [ctypes.c_int] + [ctypes.c_float] * 3 + [ctypes.c_void_p] * 5 + [ctypes.c_int] * 2
        _ref = h
    return _ref


def lib():
    global _lib
    if _lib is None:
        build()
        h = ctypes.CDLL(_LIB)
        vpp = ctypes.POINTER(ctypes.c_void_p)
        h.orc_allreduce.restype = ctypes.c_int
        h.orc_allreduce.argtypes = [vpp, ctypes.c_int, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        h.orc_reducescatter.restype = ctypes.c_int
        h.orc_reducescatter.argtypes = [vpp, ctypes.c_int, ctypes.c_int64, ctypes.c_int, ctypes.c_int, vpp]
        h.orc_allgather.restype = ctypes.c_int
        h.orc_allgather.argtypes = [vpp, ctypes.c_int, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
        h.orc_broadcast.restype = ctypes.c_int
        h.orc_broadcast.argtypes = [vpp, ctypes.c_int, ctypes.c_int64, ctypes.c_int, ctypes.c_int]
        h.orc_mp_allreduce.restype = ctypes.c_int
        h.orc_mp_allreduce.argtypes = [vpp, ctypes.c_int, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_int, ctypes.POINTER(ctypes.c_double), ctypes.c_void_p]
        h.orc_f32_to_f16.restype = ctypes.c_uint16
        h.orc_f32_to_f16.argtypes = [ctypes.c_float]
        h.orc_f16_to_f32.restype = ctypes.c_float
        h.orc_f16_to_f32.argtypes = [ctypes.c_uint16]
        h.orc_f32_to_bf16.restype = ctypes.c_uint16
        h.orc_f32_to_bf16.argtypes = [ctypes.c_float]
        h.orc_bf16_to_f32.restype = ctypes.c_float
        h.orc_bf16_to_f32.argtypes = [ctypes.c_uint16]
        h.orc_adamw.restype = None
        h.orc_adamw.argtypes = [ctypes.c_int64] + [ctypes.c_float] * 5 + [ctypes.c_void_p] * 5
        h.orc_adam.restype = None
        h.orc_adam.argtypes = [ctypes.c_int64] + [ctypes.c_float] * 5 + [ctypes.c_void_p] * 4
        h.orc_momentum_sgd.restype = None
        h.orc_momentum_sgd.argtypes = [ctypes.c_int64] + [ctypes.c_float] * 3 + [ctypes.c_int] + [ctypes.c_void_p] * 3
        _lib = h
    return _lib


def _ptrs(arrays):
    return (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])


def _prep(bufs, dtype):
    st = NP_STORAGE[dtype]
    out = [np.ascontiguousarray(b).view(st).reshape(-1) for b in bufs]
    n = out[0].size
    assert all(b.size == n for b in out), "ragged rank buffers"
    return out


def allreduce(bufs, dtype, redop="SUM", out=None):
    """Result every rank must hold after ALLREDUCE of the per-rank arrays."""
    op = REDOPS[redop.upper()] if isinstance(redop, str) else redop
    bufs = _prep(bufs, dtype)
    if out is None:
        out = np.empty_like(bufs[0])
    rc = lib().orc_allreduce(_ptrs(bufs), len(bufs), bufs[0].size, dtype, op, out.ctypes.data)
    if rc != 0:
        raise ValueError("oracle rejected allreduce(dtype={}, redop={})".format(dtype, redop))
    return out


def reducescatter(bufs, dtype, redop="SUM"):
    """List of per-rank results of REDUCESCATTER (each input holds n equal blocks)."""
    op = REDOPS[redop.upper()] if isinstance(redop, str) else redop
    bufs = _prep(bufs, dtype)
    n = len(bufs)
    assert bufs[0].size % n == 0
    count = bufs[0].size // n
    outs = [np.empty(count, dtype=bufs[0].dtype) for _ in range(n)]
    rc = lib().orc_reducescatter(_ptrs(bufs), n, count, dtype, op, _ptrs(outs))
    if rc != 0:
        raise ValueError("oracle rejected reducescatter")
    return outs


def allgather(bufs, dtype):
    bufs = _prep(bufs, dtype)
    out = np.empty(bufs[0].size * len(bufs), dtype=bufs[0].dtype)
    rc = lib().orc_allgather(_ptrs(bufs), len(bufs), bufs[0].size, dtype, out.ctypes.data)
    if rc != 0:
        raise ValueError("oracle rejected allgather")
    return out


def broadcast(bufs, dtype, root=0):
    """Per-rank buffers after an in-place BROADCAST from `root`."""
    bufs = [b.copy() for b in _prep(bufs, dtype)]
    rc = lib().orc_broadcast(_ptrs(bufs), len(bufs), bufs[0].size, dtype, root)
    if rc != 0:
        raise ValueError("oracle rejected broadcast")
    return bufs


def mp_allreduce(bufs, dtype, redop="SUM", iters=5):
    """Runs the MPI-shaped multi-process all-reduce; returns (seconds per
    iteration as a list, rank 0's result)."""
    op = REDOPS[redop.upper()] if isinstance(redop, str) else redop
    bufs = _prep(bufs, dtype)
    secs = (ctypes.c_double * iters)()
    out = np.empty_like(bufs[0])
    rc = lib().orc_mp_allreduce(_ptrs(bufs), len(bufs), bufs[0].size, dtype, op, iters, secs, out.ctypes.data)
    if rc != 0:
        raise RuntimeError("orc_mp_allreduce failed with {}".format(rc))
    return list(secs), out


# ---- the fp64 side of the contract ---------------------------------------------

def bf16_bits_to_f32(bits):
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (NaN -> 0x7fff)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = 0x7FFF
    return r


def to_f64(buf, dtype):
    st = NP_STORAGE[dtype]
    a = np.ascontiguousarray(buf).view(st).reshape(-1)
    if dtype == BF16:
        return bf16_bits_to_f32(a).astype(np.float64)
    return a.astype(np.float64)


def fp64_sum(bufs, dtype, mean=False):
    acc = np.zeros(np.ascontiguousarray(bufs[0]).view(NP_STORAGE[dtype]).size, dtype=np.float64)
    for b in bufs:
        acc += to_f64(b, dtype)
    return acc / len(bufs) if mean else acc


def max_rel_err(result, ref64, dtype):
    """max |y - ref| / max(|ref|_inf, tiny): the contract's error measure,
    relative to the largest reference magnitude of the message."""
    y = to_f64(result, dtype)
    scale = max(float(np.max(np.abs(ref64))) if ref64.size else 0.0, 1e-30)
    return float(np.max(np.abs(y - ref64))) / scale if ref64.size else 0.0


# ---- sharded (ZeRO-style) AdamW step -----------------------------------------

def from_f32(x, dtype):
    """fp32 -> storage of `dtype`, round to nearest even (convert::To of the reference)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == F16:
        with np.errstate(over="ignore"):
            return x.astype(np.float16)
    if dtype == BF16:
        return f32_to_bf16_bits(x)
    return x.copy()


def to_f32(buf, dtype):
    a = np.ascontiguousarray(buf).view(NP_STORAGE[dtype]).reshape(-1)
    return bf16_bits_to_f32(a) if dtype == BF16 else a.astype(np.float32)


def adamw(g, m, v, y, lr, beta1, beta2, eps, wd, lrs=None):
    """In-place AdamW on fp32 arrays through the C restatement (orc_adamw)."""
    for a in (g, m, v, y):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    if lrs is not None:
        lrs = np.ascontiguousarray(lrs, dtype=np.float32)
    lib().orc_adamw(g.size, lr, beta1, beta2, eps, wd, lrs.ctypes.data if lrs is not None else None,
                    g.ctypes.data, m.ctypes.data, v.ctypes.data, y.ctypes.data)


def adam(g, m, v, y, lr, beta1, beta2, eps, wd):
    """In-place Adam (coupled weight decay) on fp32 arrays (orc_adam)."""
    for a in (g, m, v, y):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    lib().orc_adam(g.size, lr, beta1, beta2, eps, wd, g.ctypes.data, m.ctypes.data, v.ctypes.data, y.ctypes.data)


def momentum_sgd(g, m, y, lr, momentum, wd, nesterov=False):
    """In-place SGD with momentum, plain or Nesterov (orc_momentum_sgd)."""
    for a in (g, m, y):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    lib().orc_momentum_sgd(g.size, lr, momentum, wd, 1 if nesterov else 0, g.ctypes.data, m.ctypes.data, y.ctypes.data)


def allreduce_update(grads, param, m, v, kind, hyper):
    """The reference's data-parallel step for one float32 tensor, all ranks at
    once: ALLREDUCE SUM of the per-rank gradients (ascending rank order), then
    the update operator -- TransformGrad (scale by grad_scale, clamp to
    +-clip_value; operators/training/update_op_base.cc:21-38) and the kernel
    loop (kernels/training/cpu/sgd_kernel.cc, adam_kernel.cc).  `param`, `m`
    and `v` (None for the SGD kinds) are updated in place; every rank ends up
    with these values.  kind: "momentum_sgd", "nesterov_sgd", "adam", "adamw";
    hyper: dict(lr, momentum | beta1, beta2, eps, weight_decay, grad_scale,
    clip_value) with lr / weight_decay as the kernel receives them."""
    g = allreduce(grads, F32, "SUM").copy()
    f32 = np.float32
    if hyper.get("grad_scale", 1.0) != 1.0:
        g *= f32(hyper["grad_scale"])
    if hyper.get("clip_value", 0.0) > 0:
        cv = f32(hyper["clip_value"])
        g = np.ascontiguousarray(np.maximum(-cv, np.minimum(g, cv)))
    if kind in ("momentum_sgd", "nesterov_sgd"):
        momentum_sgd(g, m, param, hyper["lr"], hyper["momentum"], hyper["weight_decay"], kind == "nesterov_sgd")
    elif kind == "adam":
        adam(g, m, v, param, hyper["lr"], hyper["beta1"], hyper["beta2"], hyper["eps"], hyper["weight_decay"])
    elif kind == "adamw":
        adamw(g, m, v, param, hyper["lr"], hyper["beta1"], hyper["beta2"], hyper["eps"], hyper["weight_decay"])
    else:
        raise ValueError("unknown update kind {}".format(kind))


def zero_shard_count(total, n):
    return (total + n - 1) // n


def zero_init_master(params_flat, n, dtype):
    """Per-rank fp32 master shards of the flat parameters (InitMaster,
    dragon/operators/training/zero_update_op_base.cc:21-44); entries past the
    end of the bucket are zero."""
    total = params_flat.size
    rc = zero_shard_count(total, n)
    full = np.zeros(n * rc, dtype=np.float32)
    full[:total] = to_f32(params_flat, dtype)
    return [full[r * rc:(r + 1) * rc].copy() for r in range(n)]


def zero_adamw_step(grads, params, states, counts, dtype, hyper, lr_scales=None, check_finite=False):
    """One step of the reference's ZeroAdamW operator for one bucket
    (zero_update_op_base.cc:103-143, adam_op.cc:48-81), all ranks at once.

    grads   per rank: flat gradient bucket (storage of `dtype`)
    params  per rank: flat parameter bucket, updated in place
    states  per rank: dict(master=, m=, v=) of rc fp32 values, updated in place
    counts  element counts of the tensors in the bucket (for lr_scales)
    hyper   dict(lr, beta1, beta2, eps, weight_decay, grad_scale, clip_norm, clip_value)
            with lr / weight_decay as the kernel receives them
    Returns 1.0 if the step was skipped because of an overflow, else 0.0.
    The reduce-scatter sums in ascending rank order in fp32 and rounds once to
    `dtype`, like the all-reduce of this oracle."""
    n = len(grads)
    total = int(sum(counts))
    rc = zero_shard_count(total, n)
    st = NP_STORAGE[dtype]
    padded = []
    for gr in grads:  # the send buffer, zero beyond the bucket (:118)
        buf = np.zeros(n * rc, dtype=st)
        buf[:total] = np.ascontiguousarray(gr).view(st).reshape(-1)
        padded.append(buf)
    recv = reducescatter(padded, dtype, "SUM")
    if check_finite:  # CheckFinite per rank, then the host all-reduce and min(., 1) (:121-131)
        if any(not np.all(np.isfinite(to_f32(x, dtype))) for x in recv):
            return 1.0
    f32 = np.float32
    new_shards = []
    for r in range(n):
        lo = min(r * rc, total)
        valid = min((r + 1) * rc, total) - lo
        dx = to_f32(recv[r], dtype)[:valid].copy()
        if hyper["grad_scale"] != 1.0:  # TransformGrad (:85-101)
            dx *= f32(hyper["grad_scale"])
        if hyper["clip_norm"] > 0:
            norm = f32(np.sqrt(f32(np.dot(dx.astype(np.float64), dx.astype(np.float64)))))
            if norm > f32(hyper["clip_norm"]):
                dx *= f32(hyper["clip_norm"]) / norm
        elif hyper["clip_value"] > 0:
            cv = f32(hyper["clip_value"])
            dx = np.maximum(-cv, np.minimum(dx, cv))
        lrs = None
        if lr_scales is not None and any(x != 1 for x in lr_scales):  # SetDenseHyper (:47-60)
            dense = np.repeat(np.asarray(lr_scales, dtype=np.float32), np.asarray(counts, dtype=np.int64))
            lrs = np.ascontiguousarray(dense[lo:lo + valid])
        s = states[r]
        m, v, y = (np.ascontiguousarray(s[k][:valid]) for k in ("m", "v", "master"))
        adamw(np.ascontiguousarray(dx), m, v, y, hyper["lr"], hyper["beta1"], hyper["beta2"], hyper["eps"],
              hyper["weight_decay"], lrs)
        s["m"][:valid], s["v"][:valid], s["master"][:valid] = m, v, y
        new_shards.append(from_f32(y, dtype))
    flat = np.concatenate(new_shards)  # the all-gather (:141) and the split copies (:142)
    for p in params:
        np.ascontiguousarray(p).view(st).reshape(-1)[:total] = flat[:total]
    return 0.0
