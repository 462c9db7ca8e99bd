"""Child process of tests/test_multiprocess_cpu.py: one gloo rank that runs the
group-creation host logic against a recording stand-in for the communicator."""

import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class FakeCommunicator(object):
    """Records what group creation does with a communicator; needs no GPU."""

    def __init__(self, rank, size, device):
        self.rank, self.size, self.device = rank, size, device
        self.connected = None

    @classmethod
    def init_local(cls, rank, nranks, device):
        return cls(rank, nranks, device)

    def handle_bytes(self):
        return "handle:{}:{}:{}".format(self.rank, self.size, os.getpid()).encode()

    def connect(self, handles):
        self.connected = list(handles)
        return self

    def destroy(self):
        pass


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    import dragon_b200.comm as comm_module
    comm_module.Communicator = FakeCommunicator
    from dragon_b200.distributed import backend
    backend._TorchWorld.device = lambda self: 0

    assert backend.get_world_size() == world and backend.get_rank() == rank

    full = backend.new_group(list(range(world)), backend="MPI")
    c = backend.communicator(full)
    assert c.rank == rank and c.size == world
    assert [h.split(b":")[1] for h in c.connected] == [str(r).encode() for r in range(world)]
    assert len({h.split(b":")[3] for h in c.connected}) == world  # one process per rank
    assert backend.get_rank(full) == rank

    # Every process calls new_group, members or not.
    last_only = backend.new_group([world - 1], backend="MPI")
    c = backend.communicator(last_only)
    if rank == world - 1:
        assert c is not None and c.size == 1 and c.rank == 0
    else:
        assert c is None

    reverse = backend.new_group(list(reversed(range(world))), backend="MPI")
    c = backend.communicator(reverse)
    assert c.rank == world - 1 - rank and backend.get_rank(reverse) == world - 1 - rank
    assert [h.split(b":")[1] for h in c.connected] == [str(r).encode() for r in range(world)]

    assert full.arguments["group"] != reverse.arguments["group"]
    assert repr(full) == "MPI:{}".format(full.arguments["group"])
    with full.as_default():
        assert backend.get_group() is full
        with reverse.as_default():
            assert backend.get_group() is reverse
        assert backend.get_group() is full
    assert backend.get_group() is None

    dist.barrier()
    dist.destroy_process_group()
    print("WORKER_OK", rank)


if __name__ == "__main__":
    main()
