"""One process per GPU through the whole stack: torch.distributed (gloo) as
the world, dragon.distributed / torch frontend -> C++ operator -> C-ABI ->
kernels over CUDA IPC.  Skipped where fewer than two GPUs are visible."""

import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def gpu_count():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two GPUs")
def test_python_api_one_process_per_gpu(dgn_lib):
    world = min(gpu_count(), 8)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = str(s.getsockname()[1])
    s.close()
    env = dict(os.environ, DGN_NVLS="0", PYTHONFAULTHANDLER="1")  # workers may leave early: keep them off the multicast object
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "mp_api_worker.py"), str(r), str(world), port],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env) for r in range(world)]
    # Every wait in a worker is bounded, so the workers leave on their own.
    outs = [p.communicate()[0] for p in procs]
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "WORKER_OK {}".format(r) in out, out[-3000:]
