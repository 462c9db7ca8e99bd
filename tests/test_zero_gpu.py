"""Sharded AdamW step (dgn_zero_adamw) against the oracle's restatement of the
reference's ZeroAdamW operator, through the C-ABI, on virtual ranks of one
device.

Bit-exact bar: the reduce-scatter sums in ascending rank order in fp32 and
rounds once; the update spells out every rounding of the reference's AdamW
kernel; so parameters, master copies and both moments must equal the oracle's
bit for bit on every rank.  Only clipping by norm is compared with a tolerance
(1e-6 relative on the fp32 state): the order in which the squares are summed
is the kernel's own, as it is cuBLAS's own in the reference.
"""

import os

import numpy as np
import pytest
import torch

from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
HYPER = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)


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


def _grads(rank, step, counts, dtype, scale=1e-2):
    rng = np.random.default_rng(7000 + 100 * step + rank)
    flat = rng.normal(0, scale, int(sum(counts))).astype(np.float32)
    return oracle.from_f32(flat, dtype)


def _split(flat, counts, dtype, device, offset_elems=0):
    """Flat numpy storage -> list of torch tensors; with offset_elems every
    tensor is a view that starts that many elements into its own allocation,
    which takes it off the 16-byte boundary."""
    out, pos = [], 0
    for c in counts:
        piece = flat[pos:pos + c]
        pos += c
        if offset_elems:
            base = H.to_torch(np.concatenate([np.zeros(offset_elems, dtype=flat.dtype), piece]), dtype, device)
            out.append(base[offset_elems:])
        else:
            out.append(H.to_torch(piece, dtype, device))
    return out


def _flat(tensors, dtype):
    return np.concatenate([H.to_numpy(t, dtype).reshape(-1) for t in tensors])


class Harness(object):
    """n virtual ranks with their own parameters, optimizer and oracle state."""

    def __init__(self, comms, counts, dtype, offset_elems=0, lr_scales=None, devices=None, **opt_kwargs):
        from dragon_b200.zero import ZeroAdamW
        self.comms, self.counts, self.dtype, self.n = comms, counts, dtype, len(comms)
        self.devices = devices or [DEV] * self.n  # one device per rank; virtual ranks share one
        self.offset_elems = offset_elems
        self.lr_scales = lr_scales
        total = int(sum(counts))
        p0 = oracle.from_f32(np.random.default_rng(5).normal(0, 1, total).astype(np.float32), dtype)
        self.params = [_split(p0, counts, dtype, self.devices[r], offset_elems) for r in range(self.n)]
        if lr_scales is not None:
            for plist in self.params:
                for p, s in zip(plist, lr_scales):
                    p.lr_scale = s
        kw = dict(HYPER)
        kw.update(opt_kwargs)
        # One bucket holding the tensors in the given order (the optimizer walks
        # parameters in inverse order, so hand them over reversed).
        self.opts = [ZeroAdamW(self.params[r][::-1], comms[r], **kw) for r in range(self.n)]
        self.o_params = [p0.copy() for _ in range(self.n)]
        masters = oracle.zero_init_master(p0, self.n, dtype)
        rc = oracle.zero_shard_count(total, self.n)
        self.o_states = [dict(master=masters[r], m=np.zeros(rc, np.float32), v=np.zeros(rc, np.float32))
                         for r in range(self.n)]
        self.t = 0

    def step(self, grads, found_inf=None):
        """grads: per-rank flat numpy storage.  Returns the oracle's verdict."""
        self.t += 1
        for r in range(self.n):
            pieces = _split(grads[r], self.counts, self.dtype, self.devices[r], self.offset_elems)
            for p, g in zip(self.params[r], pieces):
                p.grad = g
        for r in range(self.n):
            with torch.cuda.device(self.devices[r]):
                self.opts[r].step(found_inf=None if found_inf is None else found_inf[r])
        for d in set(self.devices):
            torch.cuda.synchronize(d)
        assert all(c.status() == 0 for c in self.comms)
        a = self.opts[0].kernel_args(self.t)
        hyper = dict(lr=a.lr, beta1=a.beta1, beta2=a.beta2, eps=a.eps, weight_decay=a.weight_decay,
                     grad_scale=a.grad_scale, clip_norm=a.clip_norm, clip_value=a.clip_value)
        return oracle.zero_adamw_step(grads, self.o_params, self.o_states, self.counts, self.dtype, hyper,
                                      lr_scales=self.lr_scales, check_finite=found_inf is not None)

    def check(self, exact=True, what=""):
        total = int(sum(self.counts))
        for r in range(self.n):
            got = _flat(self.params[r], self.dtype)
            st = self.opts[r].state(0)
            lo = min(r * st.shard, total)
            valid = min((r + 1) * st.shard, total) - lo
            for name in ("master", "m", "v"):
                g = st.view(name)[:valid].cpu().numpy()
                w = self.o_states[r][name][:valid]
                if exact:
                    H.assert_bits_equal(g, w, "{} {} rank {}".format(what, name, r))
                else:
                    np.testing.assert_allclose(g, w, rtol=1e-6, atol=1e-12, err_msg="{} {} rank {}".format(what, name, r))
            if exact:
                H.assert_bits_equal(got, self.o_params[r], "{} parameters rank {}".format(what, r))
            else:
                a = oracle.to_f32(got, self.dtype).astype(np.float64)
                b = oracle.to_f32(self.o_params[r], self.dtype).astype(np.float64)
                ulp = {oracle.F32: 2e-6, oracle.F16: 2e-3, oracle.BF16: 1.6e-2}[self.dtype]
                assert np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-3)) <= ulp, what


# Tensor sizes that are not multiples of a vector, so that vectors straddle
# tensors and shards; 15 elements in total for the tiny case (fewer than 8 ranks x 2).
RAGGED = [1000, 37, 4096, 3, 513, 1, 70001]
TINY = [5, 7, 3]
ALIGNED = [4096, 1024, 64, 8192, 512]


@pytest.mark.parametrize("n", [1, 2, 3, 8])
@pytest.mark.parametrize("dtype", [oracle.F16, oracle.BF16, oracle.F32], ids=["f16", "bf16", "f32"])
@pytest.mark.parametrize("counts", [RAGGED, TINY, ALIGNED], ids=["ragged", "tiny", "aligned"])
def test_three_steps_match_the_oracle(teams, n, dtype, counts):
    h = Harness(teams(n), counts, dtype)
    for step in range(3):
        assert h.step([_grads(r, step, counts, dtype) for r in range(n)]) == 0.0
        h.check(what="step {}".format(step))


@pytest.mark.parametrize("dtype", [oracle.F16, oracle.F32], ids=["f16", "f32"])
def test_tensors_off_the_vector_boundary(teams, dtype):
    """Every tensor starts one element into its allocation: vectors inside a
    tensor take the two-load path, borders go element by element."""
    n = 4
    h = Harness(teams(n), RAGGED, dtype, offset_elems=1)
    for step in range(2):
        h.step([_grads(r, step, RAGGED, dtype) for r in range(n)])
        h.check(what="offset step {}".format(step))


def test_learning_rate_scales_and_no_decay(teams):
    n, dtype = 4, oracle.BF16
    scales = [1.0, 0.1, 1.0, 2.0, 1.0, 0.0, 0.5]
    h = Harness(teams(n), RAGGED, dtype, lr_scales=scales, weight_decay=0.0)
    h.step([_grads(r, 0, RAGGED, dtype) for r in range(n)])
    h.check(what="lr scales, no decay")
    h2 = Harness(teams(n), RAGGED, dtype, lr_scales=scales)
    h2.step([_grads(r, 1, RAGGED, dtype) for r in range(n)])
    h2.check(what="lr scales with decay")


def test_clip_by_value_is_exact_and_clip_by_norm_is_close(teams):
    n, dtype = 4, oracle.F32
    h = Harness(teams(n), RAGGED, dtype, clip_value=5e-3, grad_scale=0.5)
    h.step([_grads(r, 0, RAGGED, dtype) for r in range(n)])
    h.check(what="clip by value")
    h = Harness(teams(n), RAGGED, dtype, clip_norm=0.05)
    h.step([_grads(r, 0, RAGGED, dtype) for r in range(n)])
    h.check(exact=False, what="clip by norm")


def test_overflow_skips_the_step_on_every_rank(teams):
    n, dtype = 4, oracle.F16
    h = Harness(teams(n), RAGGED, dtype)
    found = [torch.zeros(1, dtype=torch.float32, device=DEV) for _ in range(n)]
    good = [_grads(r, 0, RAGGED, dtype) for r in range(n)]
    assert h.step(good, found_inf=found) == 0.0
    h.check(what="checked step without overflow")
    assert all(f.item() == 0.0 for f in found)
    bad = [_grads(r, 1, RAGGED, dtype) for r in range(n)]
    bad[2][-5] = np.float16(np.inf)  # lands in the last rank's shard; everyone must skip
    before = [_flat(h.params[r], dtype) for r in range(n)]
    assert h.step(bad, found_inf=found) == 1.0
    assert all(f.item() == 1.0 for f in found)
    for r in range(n):
        H.assert_bits_equal(_flat(h.params[r], dtype), before[r], "parameters after a skipped step")
    h.check(what="state after a skipped step")
    # fp16 sums that overflow only after the reduction count too
    big = [np.full(int(sum(RAGGED)), 40000.0, dtype=np.float16) for _ in range(n)]
    assert h.step(big, found_inf=found) == 1.0
    assert all(f.item() == 2.0 for f in found)
    # The step count advanced on the skipped runs, as the reference's does.
    assert h.step([_grads(r, 3, RAGGED, dtype) for r in range(n)], found_inf=found) == 0.0
    h.check(what="step after skipped steps")


def test_resnet50_shaped_bucket_eight_ranks(teams):
    """The ResNet-50 parameter list as one fp32 bucket: 25,557,032 elements whose
    shard size (3,194,629) is odd, so shards begin inside vectors."""
    from dragon_b200 import workloads
    counts = [int(np.prod(s)) for s in workloads.resnet50_shapes()]
    n, dtype = 8, oracle.F32
    h = Harness(teams(n), counts, dtype)
    h.step([_grads(r, 0, counts, dtype, scale=1e-3) for r in range(n)])
    h.check(what="resnet50 bucket")


def test_bert_base_shaped_fp16_bucket_eight_ranks(teams):
    """The BERT-base parameter list (199 fp16 tensors, 109,482,240 elements) as
    one bucket on eight ranks, overflow check on: bit for bit against the
    oracle, and every rank ends with the same parameters."""
    from dragon_b200 import workloads
    counts = [int(np.prod(s)) for s in workloads.bert_base_shapes()]
    n, dtype = 8, oracle.F16
    h = Harness(teams(n), counts, dtype)
    found = [torch.zeros(1, dtype=torch.float32, device=DEV) for _ in range(n)]
    assert h.step([_grads(r, 0, counts, dtype) for r in range(n)], found_inf=found) == 0.0
    h.check(what="bert-base bucket")
    first = _flat(h.params[0], dtype)
    assert all(np.array_equal(_flat(h.params[r], dtype), first) for r in range(1, n))
    assert all(f.item() == 0.0 for f in found)


def test_argument_errors(teams, dgn_lib):
    import ctypes
    from dragon_b200 import _C
    comms = teams(2)
    x = torch.zeros(16, dtype=torch.int32, device=DEV)
    ptrs = (ctypes.c_void_p * 1)(x.data_ptr())
    counts = (ctypes.c_int64 * 1)(16)
    args = _C.AdamWArgs()
    st = torch.zeros(32, dtype=torch.float32, device=DEV)
    rc = dgn_lib.dgn_zero_adamw(comms[0]._h, ptrs, ptrs, counts, 1, _C.I32, st.data_ptr(), st.data_ptr(),
                                st.data_ptr(), st.data_ptr(), None, ctypes.byref(args), None, None)
    assert rc == _C.ERR_UNSUPPORTED
    rc = dgn_lib.dgn_zero_adamw(comms[0]._h, ptrs, ptrs, counts, 1, _C.F32, st.data_ptr() + 4, st.data_ptr(),
                                st.data_ptr(), st.data_ptr(), None, ctypes.byref(args), None, None)
    assert rc == _C.ERR_ARG and b"aligned" in dgn_lib.dgn_last_error_string()
    rc = dgn_lib.dgn_zero_adamw(comms[0]._h, ptrs, ptrs, counts, 1, _C.F32, st.data_ptr(), st.data_ptr(),
                                st.data_ptr(), st.data_ptr(), None, None, None, None)
    assert rc == _C.ERR_ARG
