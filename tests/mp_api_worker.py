"""Child process of tests/test_multiprocess_gpu.py: one rank per GPU, the
world provided by torch.distributed (gloo), collectives issued through
dragon.distributed -> operator layer -> C-ABI."""

import datetime
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(rank), WORLD_SIZE=str(world))
    import numpy as np
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = "cuda:{}".format(rank)
    dist.init_process_group(backend="gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))

    from dragon_b200 import distributed
    from dragon_b200 import torch_distributed as tdist
    from oracle import oracle
    from tests import helpers as H

    # The parent starts the workers with DGN_NVLS=0, so that a worker that leaves
    # early is never bound to an NVSwitch multicast object; every wait below is
    # bounded (gloo timeout, device-side wait limit), so a failure ends all ranks.
    ok = False
    try:
        body(rank, world, dev, dist, distributed, tdist, oracle, H, np, torch)
        ok = True
    finally:
        try:
            dist.barrier()
            distributed.finalize()
            dist.barrier()
        except Exception:  # noqa: BLE001 - a peer may be gone already
            pass
        dist.destroy_process_group()
    if ok:
        print("WORKER_OK", rank)


def body(rank, world, dev, dist, distributed, tdist, oracle, H, np, torch):
    assert distributed.get_rank() == rank and distributed.get_world_size() == world
    group = distributed.new_group(list(range(world)), backend="NCCL")
    assert group.size == world and distributed.get_rank(group) == rank

    # dragon.distributed.all_reduce returns a new tensor; MEAN is fused.
    arrays = [H.make_input(r, 300001, oracle.F16) for r in range(world)]
    x = H.to_torch(arrays[rank], oracle.F16, dev)
    with group.as_default():
        y = distributed.all_reduce(x, "mean")
    torch.cuda.synchronize()
    H.assert_bits_equal(H.to_numpy(y, oracle.F16), oracle.allreduce(arrays, oracle.F16, "MEAN"))
    H.assert_bits_equal(H.to_numpy(x, oracle.F16), arrays[rank])

    # torch frontend, in place, and a bucketed gradient list.
    z = torch.full((1000,), float(rank + 1), device=dev)
    assert tdist.all_reduce(z, "sum", group) is z
    grads_host = [[H.make_input(r, k, oracle.F32, seed=9 + i) for i, k in enumerate((7, 5000, 123457))]
                  for r in range(world)]
    grads = [H.to_torch(a, oracle.F32, dev) for a in grads_host[rank]]
    distributed.all_reduce_coalesced(grads, "sum", group, bucket_size=1 << 20)
    g = distributed.all_gather(torch.arange(5, device=dev) + 10 * rank, group)
    b = tdist.broadcast(torch.full((3,), float(rank), device=dev), src=world - 1, group=group)
    torch.cuda.synchronize()
    assert torch.equal(z, torch.full((1000,), world * (world + 1) / 2.0, device=dev))
    for i in range(3):
        want = oracle.allreduce([grads_host[r][i] for r in range(world)], oracle.F32, "SUM")
        H.assert_bits_equal(H.to_numpy(grads[i], oracle.F32), want)
    assert np.array_equal(g.cpu().numpy(), np.stack([np.arange(5) + 10 * r for r in range(world)]))
    assert torch.equal(b, torch.full((3,), float(world - 1), device=dev))

    # SyncBatchNorm statistics the way the reference runs them: the batch count
    # through the blocking host all-reduce, 2C floats through the device kernel.
    from dragon_b200.distributed import ops
    channels = 256
    parts = [np.random.default_rng(40 + r).normal(0, 8, 2 * channels).astype(np.float32) for r in range(world)]
    stats = torch.from_numpy(parts[rank].copy()).to(dev)
    total = ops.sync_batch_norm_statistics(stats, 16 + rank, group)
    torch.cuda.synchronize()
    assert total == sum(16 + r for r in range(world))
    H.assert_bits_equal(H.to_numpy(stats, oracle.F32), oracle.allreduce(parts, oracle.F32, "SUM"))

    # A sub-group that leaves the last rank out: every process still calls new_group.
    if world > 2:
        sub = distributed.new_group(list(range(world - 1)))
        w = torch.ones(64, device=dev)
        tdist.all_reduce(w, group=sub)
        torch.cuda.synchronize()
        expect = float(world - 1) if rank < world - 1 else 1.0
        assert torch.equal(w, torch.full((64,), expect, device=dev))



if __name__ == "__main__":
    main()
