"""CPU side of the sharded AdamW step: the oracle's restatement against
independent float64 arithmetic, the shard geometry exported by the C-ABI, and
the bucketing rule of the host layer.  No GPU is touched."""

import numpy as np
import pytest

from oracle import oracle


def _adamw_f64(g, m, v, y, lr, b1, b2, eps, wd, lrs=None):
    g, m, v, y = (a.astype(np.float64) for a in (g, m, v, y))
    s = np.ones_like(g) if lrs is None else lrs.astype(np.float64)
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    y = y - (wd * s * y + lr * s * m / (np.sqrt(v) + eps)) if wd > 0 else y - lr * s * m / (np.sqrt(v) + eps)
    return m, v, y


@pytest.mark.parametrize("wd", [0.0, 1e-5])
@pytest.mark.parametrize("scaled", [False, True])
def test_oracle_adamw_against_float64(wd, scaled):
    rng = np.random.default_rng(11)
    n = 10000
    g = rng.normal(0, 1e-2, n).astype(np.float32)
    m = rng.normal(0, 1e-3, n).astype(np.float32)
    v = (rng.normal(0, 1e-3, n) ** 2).astype(np.float32)
    y = rng.normal(0, 1, n).astype(np.float32)
    lrs = rng.uniform(0.1, 2.0, n).astype(np.float32) if scaled else None
    f32 = np.float32
    lr, b1, b2, eps = float(f32(3e-4)), float(f32(0.9)), float(f32(0.999)), float(f32(1e-8))
    wm, wv, wy = _adamw_f64(g, m, v, y, lr, b1, b2, eps, float(f32(wd)), lrs)
    oracle.adamw(g, m, v, y, lr, b1, b2, eps, float(f32(wd)), lrs)
    np.testing.assert_allclose(m, wm, rtol=3e-7, atol=1e-9)
    np.testing.assert_allclose(v, wv, rtol=3e-7, atol=1e-12)
    np.testing.assert_allclose(y, wy, rtol=3e-7, atol=1e-7)


# ---- exact rational arithmetic: an independent model of every IEEE operation ----

def _rn32(x):
    """Fraction -> nearest float32 (ties to even), as a Fraction; exact integer arithmetic."""
    from fractions import Fraction
    if x == 0:
        return Fraction(0)
    sign = -1 if x < 0 else 1
    a = abs(x)
    e = a.numerator.bit_length() - a.denominator.bit_length()  # 2^(e-1) <= a < 2^(e+1)
    if Fraction(2) ** e > a:
        e -= 1
    e = max(e, -126)                      # below 2^-126 the spacing stays 2^-149
    ulp = Fraction(2) ** (e - 23)
    q = a / ulp
    m = q.numerator // q.denominator
    rest = q - m
    if rest > Fraction(1, 2) or (rest == Fraction(1, 2) and m % 2 == 1):
        m += 1
    r = m * ulp
    assert r < Fraction(2) ** 128, "overflow is not part of this test"
    return sign * r


def _sqrt32(x):
    """Correctly rounded float32 square root of a non-negative Fraction."""
    from fractions import Fraction
    from math import isqrt
    if x == 0:
        return Fraction(0)
    k = 200
    s = isqrt(x.numerator * x.denominator << (2 * k))  # floor(sqrt(p q) 2^k)
    approx = Fraction(s, x.denominator << k)            # within 2^-k of sqrt(p/q) from below
    lo, hi = _rn32(approx), _rn32(approx + Fraction(1, 1 << (k - 8)))
    assert lo == hi, "rounding boundary within the approximation error"
    return lo


def _adamw_exact(g, m, v, y, lr, b1, b2, eps, wd, ls=None):
    """The reference's AdamW kernel, one element, every operation rounded to float32 once."""
    from fractions import Fraction
    F = lambda t: Fraction(float(np.float32(t)))  # noqa: E731
    g, m, v, y, lr, b1, b2, eps, wd = map(F, (g, m, v, y, lr, b1, b2, eps, wd))
    one = Fraction(1)
    mi = _rn32(b1 * m + _rn32(_rn32(one - b1) * g))                       # fma(b1, m, (1-b1)*g)
    vi = _rn32(b2 * v + _rn32(_rn32(_rn32(one - b2) * g) * g))            # fma(b2, v, ((1-b2)*g)*g)
    den = _rn32(_sqrt32(vi) + eps)
    if ls is None:
        step = _rn32(_rn32(lr * mi) / den)
        dec = _rn32(wd * y + step) if wd > 0 else step                  # fma(wd, y, step)
    else:
        ls = F(ls)
        step = _rn32(_rn32(_rn32(lr * ls) * mi) / den)
        dec = _rn32(_rn32(wd * ls) * y + step) if wd > 0 else step
    return float(mi), float(vi), float(_rn32(y - dec))


@pytest.mark.parametrize("wd", [0.0, 0.003])
@pytest.mark.parametrize("scaled", [False, True])
def test_oracle_adamw_bit_exact_against_exact_rational_arithmetic(wd, scaled):
    """Pins the C restatement bit for bit: every multiply, add, fused
    multiply-add, square root and divide must be the correctly rounded float32
    operation, in the order of the reference's kernel (no contraction, no fast
    math).  The model uses integers and fractions only."""
    rng = np.random.default_rng(2024)
    n = 96
    g = rng.normal(0, 1e-2, n).astype(np.float32)
    m = rng.normal(0, 1e-3, n).astype(np.float32)
    v = (rng.normal(0, 1e-3, n) ** 2).astype(np.float32)
    y = rng.normal(0, 1, n).astype(np.float32)
    g[:4] = [0.0, 1e-30, -3.0, 1e-20]  # zero and tiny gradients: subnormal products, eps-dominated denominators
    v[:2] = 0.0
    lrs = rng.uniform(0.1, 2.0, n).astype(np.float32) if scaled else None
    f32 = np.float32
    lr, b1, b2, eps = float(f32(3e-4)), float(f32(0.9)), float(f32(0.999)), float(f32(1e-8))
    want = [_adamw_exact(g[i], m[i], v[i], y[i], lr, b1, b2, eps, wd, None if lrs is None else lrs[i])
            for i in range(n)]
    oracle.adamw(g, m, v, y, lr, b1, b2, eps, float(f32(wd)), lrs)
    wm, wv, wy = (np.array(col, dtype=np.float32) for col in zip(*want))
    assert np.array_equal(m.view(np.uint32), wm.view(np.uint32))
    assert np.array_equal(v.view(np.uint32), wv.view(np.uint32))
    assert np.array_equal(y.view(np.uint32), wy.view(np.uint32))


def test_oracle_adamw_known_answer():
    """First step from zero moments: m = (1-b1) g, v = (1-b2) g^2 and the step
    is lr * m / (sqrt(v) + eps); values chosen so that every product is exact."""
    g = np.array([0.5, -0.25], dtype=np.float32)
    m = np.zeros(2, np.float32)
    v = np.zeros(2, np.float32)
    y = np.array([1.0, 2.0], dtype=np.float32)
    oracle.adamw(g, m, v, y, 0.5, 0.5, 0.75, 0.0, 0.0)
    assert m.tolist() == [0.25, -0.125]
    assert v.tolist() == [0.0625, 0.015625]
    assert y.tolist() == [1.0 - 0.5 * 0.25 / 0.25, 2.0 + 0.5 * 0.125 / 0.125]
    # decoupled decay: y -= wd * y + step
    y2 = np.array([1.0], dtype=np.float32)
    oracle.adamw(np.array([0.5], np.float32), np.zeros(1, np.float32), np.zeros(1, np.float32), y2,
                 0.5, 0.5, 0.75, 0.0, 0.25)
    assert y2.tolist() == [1.0 - (0.25 * 1.0 + 0.5)]


@pytest.mark.parametrize("dtype", [oracle.F16, oracle.BF16, oracle.F32])
def test_oracle_zero_step_against_unsharded_float64(dtype):
    """Sharding must not change the result: the step over n ranks equals AdamW
    on the whole bucket with the fp64 mean gradient, within the element type's
    rounding."""
    rng = np.random.default_rng(3)
    n, counts = 3, [50, 7, 130]
    total = sum(counts)
    grads = [oracle.from_f32(rng.normal(0, 1e-2, total).astype(np.float32), dtype) for _ in range(n)]
    p0 = oracle.from_f32(rng.normal(0, 1, total).astype(np.float32), dtype)
    params = [p0.copy() for _ in range(n)]
    rc = oracle.zero_shard_count(total, n)
    masters = oracle.zero_init_master(p0, n, dtype)
    states = [dict(master=masters[r], m=np.zeros(rc, np.float32), v=np.zeros(rc, np.float32)) for r in range(n)]
    hyper = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-5, grad_scale=1.0 / n,
                 clip_norm=0.0, clip_value=0.0)
    assert oracle.zero_adamw_step(grads, params, states, counts, dtype, hyper) == 0.0
    gmean = oracle.fp64_sum(grads, dtype, mean=True)
    _, _, want = _adamw_f64(gmean, np.zeros(total), np.zeros(total), oracle.to_f32(p0, dtype),
                            1e-3, 0.9, 0.999, 1e-8, 1e-5)
    got = oracle.to_f32(params[0], dtype).astype(np.float64)
    tol = {oracle.F32: 5e-6, oracle.F16: 1.5e-3, oracle.BF16: 1e-2}[dtype]
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-2)) <= tol
    for r in range(1, n):
        assert np.array_equal(params[r], params[0])
    # overflow: one non-finite gradient anywhere skips the step everywhere
    grads[1][3] = np.inf if dtype != oracle.BF16 else 0x7F80
    before = params[0].copy()
    assert oracle.zero_adamw_step(grads, params, states, counts, dtype, hyper, check_finite=True) == 1.0
    assert np.array_equal(params[0], before)


@pytest.mark.parametrize("dtype", [oracle.F16, oracle.F32])
def test_oracle_zero_step_does_not_depend_on_the_number_of_shards(dtype):
    """Without clipping by norm (the one place where the shard shows: the norm
    is taken over the local shard) the update is elementwise, so cutting the
    same summed gradient into 1, 2, 3 or 8 shards must give identical bits."""
    rng = np.random.default_rng(21)
    counts = [33, 1, 400, 7]
    total = sum(counts)
    g = oracle.from_f32(rng.normal(0, 1e-2, total).astype(np.float32), dtype)
    zero = np.zeros(total, dtype=oracle.NP_STORAGE[dtype])
    p0 = oracle.from_f32(rng.normal(0, 1, total).astype(np.float32), dtype)
    hyper = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-5, grad_scale=0.5,
                 clip_norm=0.0, clip_value=0.004)
    results = []
    for n in (1, 2, 3, 8):
        grads = [g.copy()] + [zero.copy() for _ in range(n - 1)]  # x + 0 is exact: every n sees the same sum
        params = [p0.copy() for _ in range(n)]
        rc = oracle.zero_shard_count(total, n)
        masters = oracle.zero_init_master(p0, n, dtype)
        states = [dict(master=masters[r], m=np.zeros(rc, np.float32), v=np.zeros(rc, np.float32)) for r in range(n)]
        for _ in range(2):
            oracle.zero_adamw_step(grads, params, states, counts, dtype, hyper, lr_scales=[1, 0.5, 1, 2])
        results.append(params[0])
        flat_master = np.concatenate([s["master"] for s in states])[:total]
        results.append(flat_master)
    for k in range(2, len(results), 2):
        assert np.array_equal(results[k], results[0]) and np.array_equal(results[k + 1], results[1])


@pytest.mark.parametrize("dtype,E", [(4, 8), (5, 8), (6, 4)])
def test_shard_geometry_covers_the_bucket_once(dgn_lib, dtype, E):
    """Every flat element belongs to exactly one rank's shard, and its slot in
    that rank's state arrays (offset + index in shard) lies inside the arrays
    and shares the vector alignment of the flat bucket."""
    for n in (1, 2, 3, 5, 8):
        for total in (1, 2, 7, 8, 9, 15, 64, 1000, 4099, 25557032):
            rc = dgn_lib.dgn_zero_shard_count(n, total)
            assert rc == (total + n - 1) // n
            count = dgn_lib.dgn_zero_state_count(n, total, dtype)
            assert count % E == 0
            covered = 0
            for r in range(n):
                lo, hi = min(r * rc, total), min((r + 1) * rc, total)
                off = dgn_lib.dgn_zero_state_offset(r, n, total, dtype)
                assert 0 <= off < E
                if hi > lo:
                    assert off == lo % E              # element lo sits in lane lo % E of its vector
                    assert off + (hi - lo) <= count
                covered += hi - lo
            assert covered == total
    assert dgn_lib.dgn_zero_shard_count(0, 5) == -1
    assert dgn_lib.dgn_zero_state_count(2, 5, 99) == -1
    assert dgn_lib.dgn_zero_state_offset(2, 2, 5, dtype) == -1


def test_bucketing_rule_of_the_host_layer():
    """One dtype per bucket, float16 before bfloat16 before float32, parameters
    walked in inverse order, a bucket closed before the parameter that would
    overflow it, an oversize parameter alone in its bucket."""
    import torch
    from dragon_b200.zero import ZeroReduceBucket
    h = [torch.zeros(10, dtype=torch.float16) for _ in range(5)]  # 20 bytes each
    f = [torch.zeros(7), torch.zeros(100), torch.zeros(2)]        # 28, 400, 8 bytes
    buckets = ZeroReduceBucket.new(h[:2] + f + h[2:], bucket_size=45)
    assert [b.dtype for b in buckets] == [torch.float16] * 3 + [torch.float32] * 3
    assert [len(b.params) for b in buckets] == [2, 2, 1, 1, 1, 1]
    assert buckets[0].params[0] is h[4] and buckets[2].params[0] is h[0]
    assert buckets[3].params[0] is f[2] and buckets[4].params[0] is f[1] and buckets[4].size == 400
    assert ZeroReduceBucket.new([]) == []


def test_zero_adamw_needs_a_group_and_supported_dtypes():
    import torch
    from dragon_b200.zero import ZeroAdamW
    with pytest.raises(ValueError, match="<group> is required"):
        ZeroAdamW([torch.zeros(4)])
    with pytest.raises(ValueError, match="empty sequence"):
        ZeroAdamW([], comm=object())
    with pytest.raises(TypeError, match="Unsupported data type"):
        ZeroAdamW([torch.zeros(4, dtype=torch.float64)], comm=object())
