"""Child process of tests/test_multigpu.py: one rank on its own GPU, joined to
the other through the library's file rendezvous and CUDA IPC."""

import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, rdv = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    import time

    import numpy as np
    import torch

    from dragon_b200.comm import Communicator
    from oracle import oracle
    from tests import helpers as H

    torch.cuda.set_device(rank)
    dev = "cuda:{}".format(rank)
    # The parent starts these workers with DGN_NVLS=0: a worker that leaves early
    # (a failed check) must not be bound to an NVSwitch multicast object.  The
    # multicast kernels are covered inside one process by tests/test_multigpu.py.
    comm = Communicator.create(rank, world, rank, rdv, "ipc-test", timeout_ms=120000)
    comm.set_wait_limit_ms(20000)
    try:
        assert not comm.has_nvls()
        for variant in (4, 5, 1, 2, 7):
            comm.set_tuning(variant=variant)
            for dtype, count, redop in ((oracle.F16, 300001, "MEAN"), (oracle.F32, 1 << 22, "SUM")):
                arrays = [H.make_input(r, count, dtype) for r in range(world)]
                x = H.to_torch(arrays[rank], dtype, dev)
                comm.all_reduce([x], None, redop)
                torch.cuda.synchronize()
                assert comm.status() == 0
                H.assert_bits_equal(H.to_numpy(x, dtype), oracle.allreduce(arrays, dtype, redop))
        comm.set_tuning()
        idx = [np.arange(1000, dtype=np.int64) * (r + 1) for r in range(world)]
        out = torch.empty(world * 1000, dtype=torch.int64, device=dev)
        comm.all_gather(torch.from_numpy(idx[rank]).to(dev), out)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), np.concatenate(idx))
        # Host-memory all-reduce (synchronous), right after device collectives.
        counts = comm.all_reduce_host(np.array([rank + 1, 10 * (rank + 1)], dtype=np.int64), "SUM")
        assert counts.tolist() == [3, 30]
        flag = comm.all_reduce_host(np.array([0.25 * (rank + 1)], dtype=np.float32), "MAX")
        assert flag.tolist() == [0.5]
        try:
            comm.all_reduce_host(np.zeros(2000, dtype=np.float32))
            raise AssertionError("an oversize host all-reduce must be refused")
        except Exception as e:  # noqa: BLE001
            assert "4096" in str(e)
        ok = True
    except BaseException:
        ok = False
        raise
    finally:
        # Every way out passes here: leave only after the peer has finished too
        # (a last all-reduce is the barrier; its device-side wait is bounded, so a
        # peer that is gone costs the wait limit, not a hang), then free the
        # communicator.
        try:
            comm.set_tuning()
            done = torch.ones(1, device=dev)
            comm.all_reduce([done], None, "SUM")
            torch.cuda.synchronize()
            time.sleep(0.5)
        except Exception:  # noqa: BLE001 - the communicator may already be unusable
            pass
        comm.destroy()
    if ok:
        print("WORKER_OK", rank)


if __name__ == "__main__":
    main()
