"""dgn_allreduce_static: the all-reduce for callers that may not allocate.

Some users of this library run where cudaMalloc is off limits: inside a
framework whose memory planner has already handed out the whole device pool,
or on a serving path that cannot afford the allocator's device-wide
synchronisation.  They cannot build a communicator (it allocates a
workspace), so the library offers one entry point whose scratch memory is a
fixed array inside the library image.  This test calls it through the C-ABI
twice in a row and checks both results, bit for bit, against the regular
entry point (dgn_allreduce on an emulated communicator) and against the CPU
oracle directly, and watches the driver's free-memory figure around the calls.

This file sorts last on purpose: if the extra entry point ever breaks, a run
that stops at the first failure has already exercised everything else.
"""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_allreduce(lib, ins, outs, dgn_dtype, redop):
    from dragon_b200 import _C
    n = len(ins)
    in_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in ins])
    out_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in outs])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _C.check(lib.dgn_allreduce_static(n, in_ptrs, out_ptrs, ins[0].numel(), dgn_dtype, redop, stream))


def _reference_allreduce(nranks, ins, reduction):
    from dragon_b200.comm import Communicator
    comms = Communicator.emulated(nranks, 0)
    try:
        outs = [torch.empty_like(t) for t in ins]
        for c, i, o in zip(comms, ins, outs):
            c.all_reduce([i], [o], reduction)
        torch.cuda.synchronize()
        return outs
    finally:
        for c in comms:
            c.destroy()


def test_static_scratch_allreduce_matches_regular_entry_point(dgn_lib):
    from dragon_b200 import _C
    from dragon_b200.comm import dgn_dtype
    dev = "cuda:0"
    torch.cuda.set_device(0)
    # Two calls in a row on one stream, different rank counts, sizes and types:
    # the second call reuses the array the first one left dirty.
    cases = [
        (4, 4093, torch.float32, "MEAN"),   # 16372 bytes: just under the limit, ragged tail
        (8, 2500, torch.float16, "SUM"),
    ]
    gen = torch.Generator(device="cpu").manual_seed(1234)
    inputs, outputs = [], []
    for n, count, dtype, reduction in cases:
        ins = [(torch.rand(count, generator=gen) * 2 - 1).to(dtype).to(dev) for _ in range(n)]
        outs = [torch.full_like(t, float("nan")) for t in ins]
        inputs.append(ins)
        outputs.append(outs)
    # First calls outside the watched region: they look up the array's address
    # and load the kernel of each element type, which the driver may back with
    # memory of its own.
    for dtype in sorted({c[2] for c in cases}, key=str):
        warm = [torch.zeros(4, dtype=dtype, device=dev) for _ in range(2)]
        _static_allreduce(dgn_lib, warm, warm, dgn_dtype(dtype), _C.SUM)
    torch.cuda.synchronize()
    # torch's counter cannot see a cudaMalloc inside the library; the driver's
    # free-bytes figure can (nothing else runs on this device meanwhile).
    before_torch = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()
    for (n, count, dtype, reduction), ins, outs in zip(cases, inputs, outputs):
        _static_allreduce(dgn_lib, ins, outs, dgn_dtype(dtype), _C.REDOPS[reduction])
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == before_torch
    assert free_after == free_before, "device memory in use changed by {} bytes".format(free_before - free_after)
    assert dgn_lib.dgn_allreduce_static_status(0) == _C.OK   # no block gave up
    from oracle import oracle
    kinds = {torch.float32: oracle.F32, torch.float16: oracle.F16}
    for (n, count, dtype, reduction), ins, outs in zip(cases, inputs, outputs):
        want = _reference_allreduce(n, ins, reduction)
        want_oracle = oracle.allreduce([t.cpu().numpy() for t in ins], kinds[dtype], reduction)
        for r in range(n):
            got_bits = outs[r].cpu().numpy().view(np.uint8)
            want_bits = want[r].cpu().numpy().view(np.uint8)
            assert np.array_equal(got_bits, want_bits), "rank {} of the {}-rank call differs".format(r, n)
            assert np.array_equal(got_bits, np.ascontiguousarray(want_oracle).view(np.uint8)), \
                "rank {} of the {}-rank call differs from the oracle".format(r, n)


def test_static_scratch_allreduce_in_place_and_repeatable(dgn_lib):
    from dragon_b200 import _C
    dev = "cuda:0"
    torch.cuda.set_device(0)
    n, count = 2, 1000
    a = [torch.arange(count, dtype=torch.int32, device=dev) * (r + 1) for r in range(n)]
    want = (torch.arange(count, dtype=torch.int32, device=dev) * 3)
    for _ in range(2):  # same call twice: the result must not depend on leftovers
        bufs = [t.clone() for t in a]
        _static_allreduce(dgn_lib, bufs, bufs, _C.I32, _C.SUM)
        torch.cuda.synchronize()
        assert all(torch.equal(b, want) for b in bufs)


def test_static_scratch_allreduce_rejects_oversize(dgn_lib):
    from dragon_b200 import _C
    dev = "cuda:0"
    x = [torch.zeros(4097, dtype=torch.float32, device=dev) for _ in range(2)]  # 16388 bytes
    with pytest.raises(_C.DgnError) as e:
        _static_allreduce(dgn_lib, x, x, _C.F32, _C.SUM)
    assert e.value.status == _C.ERR_ARG
    assert "16384" in str(e.value)
