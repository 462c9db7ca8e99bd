"""World-size-2 and -3 runs of the group bootstrap over gloo on CPU, and the
reference arm of the benchmark (the CPU restatement timed as rank processes)."""

import json
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return str(port)


@pytest.mark.parametrize("world", [2, 3])
def test_group_creation_over_gloo(world):
    port = free_port()
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "mp_worker.py"), str(r), str(world), port],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "WORKER_OK {}".format(r) in out, out[-2000:]


@pytest.mark.parametrize("gpus", [1, 2])
def test_bench_reference_arm(gpus):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", str(gpus),
                          "--steps", "2", "--warmup", "1", "--size-mib", "4"],
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    assert len(out.stdout.strip().splitlines()) == 1, out.stdout[-500:]   # the JSON line is alone on standard output
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] == gpus
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["gpu_launches"] == 0


def test_bench_keeps_library_chatter_off_standard_output():
    """What a library writes to file descriptor 1 behind Python's back (NCCL prints
    its version there) must not land beside the JSON line."""
    code = ("import os, sys; sys.path.insert(0, {!r}); import bench; bench.keep_stdout_for_the_result(); "
            "os.write(1, b'NCCL version x.y\\n'); print('python chatter'); bench.emit_result({{'value': 1}})").format(ROOT)
    out = subprocess.run([sys.executable, "-c", code], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                         timeout=120, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout == '{"value": 1}\n', out.stdout
    assert "NCCL version x.y" in out.stderr and "python chatter" in out.stderr


def test_bench_reference_arm_other_ranks_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""
