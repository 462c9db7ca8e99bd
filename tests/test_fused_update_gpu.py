"""The gradient all-reduce fused with the optimizer update (dgn_allreduce_update)
against the CPU oracle: ALLREDUCE SUM in ascending rank order, the update
operator's gradient transform, and the reference's SGD / Adam loops
(kernels/training/cpu/sgd_kernel.cc, adam_kernel.cc, which the oracle is pinned
to).  Parameters and optimizer state must match bit for bit on every rank, over
several steps; gradients are left untouched."""

import numpy as np
import pytest
import torch

from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
COUNTS = [64, 1, 0, 4099, 7, 1 << 16, 33, 2048, 300001]


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


def make_optimizer(kind, params, comm, hyper):
    from dragon_b200 import fused_optim
    if kind in ("momentum_sgd", "nesterov_sgd"):
        return fused_optim.FusedSGD(params, hyper["lr"], hyper["momentum"], hyper["weight_decay"],
                                    nesterov=(kind == "nesterov_sgd"), comm=comm, grad_scale=hyper["grad_scale"],
                                    clip_value=hyper["clip_value"])
    cls = fused_optim.FusedAdam if kind == "adam" else fused_optim.FusedAdamW
    return cls(params, hyper["lr"], (hyper["beta1"], hyper["beta2"]), hyper["eps"], hyper["weight_decay"], comm=comm,
               grad_scale=hyper["grad_scale"], clip_value=hyper["clip_value"])


def oracle_hyper(opt, t):
    a = opt.kernel_args(t)
    return dict(lr=a.lr, momentum=a.momentum, beta1=a.beta1, beta2=a.beta2, eps=a.eps, weight_decay=a.weight_decay,
                grad_scale=a.grad_scale, clip_value=a.clip_value)


@pytest.mark.parametrize("n", [1, 2, 4, 8])
@pytest.mark.parametrize("kind,hyper", [
    ("momentum_sgd", dict(lr=0.1, momentum=0.9, weight_decay=1e-4, grad_scale=1.0, clip_value=0.0)),
    ("nesterov_sgd", dict(lr=0.05, momentum=0.8, weight_decay=0.0, grad_scale=0.5, clip_value=0.0)),
    ("adam", dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-2, grad_scale=1.0, clip_value=0.0)),
    ("adamw", dict(lr=2e-3, beta1=0.9, beta2=0.99, eps=1e-6, weight_decay=0.01, grad_scale=128.0, clip_value=0.05)),
])
def test_fused_update_matches_the_reference_sequence(teams, n, kind, hyper):
    comms = teams(n)
    rng = np.random.default_rng(11)
    p0 = [rng.normal(0, 1, k).astype(np.float32) for k in COUNTS]
    params = [[torch.from_numpy(a.copy()).to(DEV) for a in p0] for _ in range(n)]
    opts = [make_optimizer(kind, params[r], comms[r], hyper) for r in range(n)]
    want_p = [a.copy() for a in p0]
    want_m = [np.zeros_like(a) for a in p0]
    want_v = [np.zeros_like(a) for a in p0] if kind in ("adam", "adamw") else [None] * len(p0)
    for step in range(3):
        grads = [[np.random.default_rng(1000 + r + 50 * step + 7 * i).normal(0, 1e-2, k).astype(np.float32)
                  for i, k in enumerate(COUNTS)] for r in range(n)]
        dev_grads = [[torch.from_numpy(g.copy()).to(DEV) for g in grads[r]] for r in range(n)]
        for r in range(n):
            for p, g in zip(params[r], dev_grads[r]):
                p.grad = g
        for r in range(n):
            opts[r].step()
        torch.cuda.synchronize()
        assert all(c.status() == 0 for c in comms)
        h = oracle_hyper(opts[0], step + 1)
        for i, k in enumerate(COUNTS):
            if k == 0:
                continue
            oracle.allreduce_update([grads[r][i] for r in range(n)], want_p[i], want_m[i], want_v[i], kind, h)
        for r in range(n):
            for i, k in enumerate(COUNTS):
                what = "{} step {} rank {} tensor {}".format(kind, step, r, i)
                H.assert_bits_equal(params[r][i].cpu().numpy(), want_p[i], what + " param")
                H.assert_bits_equal(opts[r].m[i].cpu().numpy(), want_m[i], what + " m")
                if want_v[i] is not None:
                    H.assert_bits_equal(opts[r].v[i].cpu().numpy(), want_v[i], what + " v")
                H.assert_bits_equal(dev_grads[r][i].cpu().numpy(), grads[r][i], what + " gradient untouched")


def test_fused_update_is_one_launch_and_spans_rounds(teams, dgn_lib):
    """One kernel per step whatever the number of tensors; small chunks force
    many rounds of the staging pipeline; unaligned views take the element path."""
    n = 4
    comms = teams(n)
    for c in comms:
        c.set_tuning(variant=2, blocks=3, threads=64, chunk_bytes=256)
    try:
        rng = np.random.default_rng(3)
        base = [rng.normal(0, 1, 20011).astype(np.float32) for _ in range(2)]
        full = [[torch.from_numpy(a.copy()).to(DEV) for a in base] for _ in range(n)]
        params = [[t[1:] for t in row] for row in full]           # 4 bytes off the vector boundary
        from dragon_b200.fused_optim import FusedSGD
        opts = [FusedSGD(params[r], 0.1, momentum=0.9, comm=comms[r]) for r in range(n)]
        grads = [[np.random.default_rng(90 + r + i).normal(0, 1, 20010).astype(np.float32) for i in range(2)]
                 for r in range(n)]
        for r in range(n):
            for p, g in zip(params[r], grads[r]):
                p.grad = torch.from_numpy(g.copy()).to(DEV)
        before = dgn_lib.dgn_launch_count()
        for r in range(n):
            opts[r].step()
        torch.cuda.synchronize()
        assert dgn_lib.dgn_launch_count() == before + 1
        assert comms[0].last_launch()["rounds"] > 4
        h = oracle_hyper(opts[0], 1)
        for i in range(2):
            want_p, want_m = base[i][1:].copy(), np.zeros(20010, np.float32)
            oracle.allreduce_update([grads[r][i] for r in range(n)], want_p, want_m, None, "momentum_sgd", h)
            for r in range(n):
                H.assert_bits_equal(params[r][i].cpu().numpy(), want_p)
                H.assert_bits_equal(opts[r].m[i].cpu().numpy(), want_m)
                assert float(full[r][i][0].item()) == float(base[i][0])   # the element before the view is untouched
    finally:
        for c in comms:
            c.set_tuning()


def test_fused_update_argument_errors(teams):
    import ctypes
    from dragon_b200 import _C
    from dragon_b200.fused_optim import FusedAdam, FusedSGD
    comm = teams(2)[0]
    with pytest.raises(TypeError):
        FusedSGD([torch.zeros(4, dtype=torch.float16, device=DEV)], 0.1, comm=comm)
    with pytest.raises(ValueError):
        FusedSGD([], 0.1, comm=comm)
    with pytest.raises(ValueError):
        FusedAdam([torch.zeros(4, device=DEV)], betas=(1.0, 0.9), comm=comm)
    x = torch.zeros(8, device=DEV)
    one = (ctypes.c_void_p * 1)(x.data_ptr())
    cnt = (ctypes.c_int64 * 1)(8)
    args = _C.UpdateArgs(kind=7)
    lib = _C.lib()
    assert lib.dgn_allreduce_update(comm._h, one, one, one, None, cnt, 1, _C.F32, ctypes.byref(args), None) == _C.ERR_ARG
    args = _C.UpdateArgs(kind=_C.UPDATE_ADAM)
    assert lib.dgn_allreduce_update(comm._h, one, one, one, None, cnt, 1, _C.F32, ctypes.byref(args), None) == _C.ERR_ARG
    args = _C.UpdateArgs(kind=_C.UPDATE_MOMENTUM_SGD)
    assert lib.dgn_allreduce_update(comm._h, one, one, one, None, cnt, 1, _C.F16, ctypes.byref(args),
                                    None) == _C.ERR_UNSUPPORTED
