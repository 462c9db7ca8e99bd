"""The `ZeroAdamW` operator of the C++ operator layer (arguments, hyper
tensors, state tensors and cached step count as in the reference) against the
oracle, on four virtual ranks of one device."""

import numpy as np
import pytest
import torch

from oracle import oracle
from tests import helpers as H
from tests.test_zero_gpu import RAGGED, _flat, _grads, _split

pytestmark = pytest.mark.gpu
N = 4
DEV = "cuda:0"


@pytest.fixture(scope="module")
def comms(dgn_lib):
    from dragon_b200.comm import Communicator
    made = Communicator.emulated(N, 0)
    yield made
    torch.cuda.synchronize()
    for c in made:
        c.destroy()


def _kernel_hyper(h, t, n):
    """What the operator hands its kernel at step t (zero_update_op.h:108-116, adam_op.cc:52,56)."""
    f32 = np.float32
    b1, b2 = float(f32(h["beta1"])), float(f32(h["beta2"]))
    corr = f32(np.sqrt(1.0 - b2 ** t) / (1.0 - b1 ** t))
    return dict(lr=float(f32(h["lr"]) * corr), beta1=b1, beta2=b2, eps=float(f32(h["eps"])),
                weight_decay=float(f32(h["lr"]) * f32(h["weight_decay"])), grad_scale=float(f32(h["grad_scale"])),
                clip_norm=float(f32(h["clip_norm"])), clip_value=float(f32(h["clip_value"])))


@pytest.mark.parametrize("dtype", [oracle.F16, oracle.F32], ids=["f16", "f32"])
def test_zero_adamw_operator_matches_the_oracle(comms, dgn_lib, dtype):
    from dragon_b200 import _C, op_lib
    counts = RAGGED
    total = int(sum(counts))
    hyper = dict(lr=2e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, grad_scale=1.0 / N,
                 clip_norm=0.0, clip_value=0.01)
    scales = [1.0, 0.5, 1.0, 1.0, 2.0, 1.0, 1.0]
    p0 = oracle.from_f32(np.random.default_rng(9).normal(0, 1, total).astype(np.float32), dtype)
    params = [_split(p0, counts, dtype, DEV) for _ in range(N)]
    found = [torch.zeros(1, dtype=torch.float32, device=DEV) for _ in range(N)]
    o_params = [p0.copy() for _ in range(N)]
    rc = oracle.zero_shard_count(total, N)
    masters = oracle.zero_init_master(p0, N, dtype)
    o_states = [dict(master=masters[r], m=np.zeros(rc, np.float32), v=np.zeros(rc, np.float32)) for r in range(N)]
    names = ["ZeroAdamW_{}/rank{}".format(oracle.NP_STORAGE[dtype].__name__, r) for r in range(N)]
    dgn_dtype = {oracle.F16: _C.F16, oracle.F32: _C.F32}[dtype]
    for step in range(1, 4):
        grads = [_grads(r, step, counts, dtype) for r in range(N)]
        if step == 2:
            grads[1][17] = np.inf  # this run is skipped everywhere, but still counts as a step
        # Virtual ranks queue their calls until the last rank has issued its own:
        # the gradient tensors must stay alive until the launch has run.
        g_dev = [_split(grads[r], counts, dtype, DEV) for r in range(N)]
        for r in range(N):
            op_lib.run_zero_adamw(g_dev[r], params[r], hyper, name=names[r],
                                  bucket_name="Bucket_1", lr_scales=scales, found_inf=found[r],
                                  comm=int(comms[r]._h.value), group=1, backend="NCCL", ranks=list(range(N)))
        torch.cuda.synchronize()
        assert all(c.status() == 0 for c in comms)
        skipped = oracle.zero_adamw_step(grads, o_params, o_states, counts, dtype, _kernel_hyper(hyper, step, N),
                                         lr_scales=scales, check_finite=True)
        assert skipped == (1.0 if step == 2 else 0.0)
        for r in range(N):
            H.assert_bits_equal(_flat(params[r], dtype), o_params[r], "parameters step {} rank {}".format(step, r))
            off = dgn_lib.dgn_zero_state_offset(r, N, total, dgn_dtype)
            valid = min((r + 1) * rc, total) - min(r * rc, total)
            for key in ("master", "m", "v"):
                got = op_lib.zero_state(names[r], "Bucket_1", key, DEV)[off:off + valid].cpu().numpy()
                H.assert_bits_equal(got, o_states[r][key][:valid], "{} step {} rank {}".format(key, step, r))
    assert all(f.item() == 1.0 for f in found)


def test_zero_adamw_operator_is_registered_and_checks_its_arguments(comms, dgn_lib):
    from dragon_b200 import op_lib
    assert op_lib.lib().dragon_operator_is_registered(b"ZeroAdamW") == 1
    assert op_lib.lib().dragon_schema_allows_inplace(b"ZeroAdamW", 0, 0) == 0
    hyper = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, grad_scale=1.0, clip_norm=0.0,
                 clip_value=0.0)
    g = torch.zeros(8, dtype=torch.float64, device=DEV)
    with pytest.raises(op_lib.OperatorError, match="float16, bfloat16 or float32"):
        op_lib.run_zero_adamw([g], [g.clone()], hyper, name="ZeroAdamW/f64", comm=int(comms[0]._h.value), group=1)
    x = torch.zeros(8, device=DEV)
    with pytest.raises(op_lib.OperatorError, match="lr_scales"):
        op_lib.run_zero_adamw([x, x.clone()], [x.clone(), x.clone()], hyper, name="ZeroAdamW/bad",
                              lr_scales=[0.5], comm=int(comms[0]._h.value), group=1)
