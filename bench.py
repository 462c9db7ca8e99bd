#!/usr/bin/env python
"""Benchmark of the `Collective` hot path: all-reduce bus bandwidth and latency.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference --gpus N ...      (CPU path, rank 0 only)

One step = one ALLREDUCE (MEAN, fp32) through the dgn C-ABI.  At N = 1 the
communicator has one rank and the step is the out-of-place local-copy path on
the largest message of the size sweep (1 GiB, HBM bound); at N >= 2 it is the
peer-memory all-reduce over NVLink on a 256 MiB message and `value` is the bus
bandwidth S/t * 2(N-1)/N.  Before anything is timed at N >= 2, every kernel
variant the library can pick at this rank count is run once and its whole
output is compared, on every rank, with the CPU oracle (`parity` in the JSON
line); a mismatch ends the run with a non-zero exit code.  Rank 0 prints one
JSON line.
"""

import argparse
import json
import os
import statistics
import sys
import threading
import time
import zlib

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MiB = 1 << 20
METRIC = "allreduce bus GB/s & latency vs msg size at 2/4/8 B200 (frac of 900 GB/s)"
NVLINK_NOMINAL_GBS = 900.0      # per direction per GPU
NVLINK_MEASURED_P2P_GBS = 770.0  # peer copy measured on this pool
HBM_FALLBACK_GBS = 6650.0
VARIANT_NAMES = {0: "local copy", 1: "one-shot", 2: "two-shot", 3: "staged ring, multicast", 4: "LL one-shot",
                 5: "LL two-shot", 6: "in place, multicast", 7: "staged ring, peer loads/stores"}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size-mib", type=float, default=None,
                    help="message bytes per rank of the timed step (default: 1024 at one GPU, 256 otherwise)")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f16", "bf16"])
    ap.add_argument("--reduction", default="MEAN")
    ap.add_argument("--sweep", default="auto", choices=["auto", "off", "full"],
                    help="message-size sweep beside the headline (auto: up to 256 MiB)")
    ap.add_argument("--configs", default="auto", choices=["auto", "off", "zero"],
                    help="operator configurations (gradient buckets, gather/broadcast shapes) beside the headline")
    ap.add_argument("--no-nccl", action="store_true", help="skip the NCCL comparison in the sweep")
    ap.add_argument("--no-symm", action="store_true", help="N>=2: skip the symmetric-memory (in-place multicast) rows")
    ap.add_argument("--no-parity", action="store_true", help="N>=2: skip the parity pass (profiling runs only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-emulated", action="store_true", help="N=1: skip the emulated 8-rank timings")
    ap.add_argument("--emulated-only", action="store_true",
                    help="N=1: run only multi-rank kernels on 8 virtual ranks of one GPU (profiling target)")
    ap.add_argument("--emulated-case", default="default",
                    help="with --emulated-only: one of " + ", ".join(sorted(EMULATED_CASES)) +
                    ", fused_adam_64MiB, zero_adamw_64MiB_fp16, 'all' or 'default'")
    args = ap.parse_args()
    if args.size_mib is None:
        multi = args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1
        args.size_mib = 256.0 if multi else 1024.0
    return args


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return HBM_FALLBACK_GBS, "fallback"


class ClockSampler(object):
    """Polls SM clock and throttle reasons of one GPU through NVML while a
    timed region runs."""

    def __init__(self, index, period_s=0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: report nothing rather than guess
            self.nv = None

    _NAMES = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
    }

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self._NAMES.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def torch_dtype_of(name):
    import torch
    return {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "i64": torch.int64}[name]


def make_message(rank, count, dtype_name, device):
    """Seeded uniform[-1, 1) message of `count` elements on `device`."""
    import torch
    from dragon_b200 import workloads
    x = torch.from_numpy(workloads.uniform_message(rank, count))
    return x.to(device=device, dtype=torch_dtype_of(dtype_name))


def time_steps(fn, steps, warmup, barrier=None):
    """Runs fn() warmup + steps times on the current stream; returns the list of
    per-step device durations in ms (CUDA events) and the whole-region ms."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record()
    for i in range(steps):
        fn()
        evs[i + 1].record()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
    return per, evs[0].elapsed_time(evs[steps])


def time_e2e(comm, xh, yh, bufs_in, bufs_out, reduction, steps, warmup, barrier=None):
    """End to end through the public call with HOST buffers: every step copies
    the input from pinned host memory to the device, runs the all-reduce and
    copies the result back to pinned host memory.  Three streams and two
    device buffers let the H2D copy of step i+1, the collective of step i and
    the D2H copy of step i-1 overlap, as a training loop with pinned staging
    buffers would.  Returns milliseconds for `steps` steps (first H2D issued to
    last D2H finished)."""
    import torch
    s_in, s_op, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ops = [comm.prepare_all_reduce([a], [b], reduction) for a, b in zip(bufs_in, bufs_out)]
    nb = len(bufs_in)
    free = [None] * nb  # D2H of the step that last used buffer k has finished

    def step(i):
        k = i % nb
        with torch.cuda.stream(s_in):
            if free[k] is not None:
                s_in.wait_event(free[k])
            bufs_in[k].copy_(xh, non_blocking=True)
            e_in = torch.cuda.Event()
            e_in.record(s_in)
        with torch.cuda.stream(s_op):
            s_op.wait_event(e_in)
            ops[k](s_op)
            e_op = torch.cuda.Event()
            e_op.record(s_op)
        with torch.cuda.stream(s_out):
            s_out.wait_event(e_op)
            yh.copy_(bufs_out[k], non_blocking=True)
            free[k] = torch.cuda.Event()
            free[k].record(s_out)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(s_in)
    for i in range(warmup, warmup + steps):
        step(i)
    stop.record(s_out)
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    return start.elapsed_time(stop)


def time_host_copies(xh, yh, dbuf, barrier=None, reps=3):
    """PCIe rates of this rank alone per direction, all ranks copying at the same
    time: GB/s of pinned host -> device and device -> pinned host."""
    import torch
    out = {}
    for name, fn in (("h2d_gbs", lambda: dbuf.copy_(xh, non_blocking=True)),
                     ("d2h_gbs", lambda: yh.copy_(dbuf, non_blocking=True))):
        fn()
        torch.cuda.synchronize()
        if barrier is not None:
            barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        out[name] = xh.numel() * xh.element_size() * reps / (a.elapsed_time(b) * 1e-3) / 1e9
    return out


def pin_rank_to_its_cores(local, world):
    """One process per GPU: give each rank its own slice of the host cores this
    job may use, before its pinned buffers are allocated, so that the ranks'
    copy threads and first-touch pages do not pile up on the same cores."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        per = max(1, len(cores) // max(1, world))
        mine = cores[local * per:(local + 1) * per] or cores
        os.sched_setaffinity(0, mine)
        return len(mine)
    except (AttributeError, OSError):
        return None


def cpu_config1_baseline():
    """CPU restatement of the MPI path on the reference's own CPU case: 2 rank
    processes, 16 MiB fp32 SUM, in place."""
    from dragon_b200 import workloads
    from oracle import oracle
    bufs = [workloads.uniform_message(r, 4194304) for r in range(2)]
    secs, _ = oracle.mp_allreduce(bufs, oracle.F32, "SUM", iters=20)
    t = statistics.median(secs)
    s = bufs[0].nbytes
    return {"value": s / t / 1e9, "unit": "GB/s", "cores": 2, "kind": "port",
            "sample": "20 in-place all-reduces of 16 MiB fp32 SUM over 2 rank processes on shared memory "
                      "(median); bus GB/s = S/t * 2(n-1)/n", "ms_per_op": t * 1e3,
            "host_cores": os.cpu_count()}


def cpu_multi_baseline(n, reduction, sample_bytes=64 * MiB, iters=4):
    """The oracle's MPI-shaped multi-process all-reduce at the same rank count,
    on a bounded sample of the message (rank 0 only; the other ranks wait)."""
    from dragon_b200 import workloads
    from oracle import oracle
    count = sample_bytes // 4
    bufs = [workloads.uniform_message(r, count) for r in range(n)]
    secs, _ = oracle.mp_allreduce(bufs, oracle.F32, reduction, iters=iters)
    t = statistics.median(secs[1:])
    cores = os.cpu_count() or 1
    return {"value": bufs[0].nbytes / t / 1e9 * 2.0 * (n - 1) / n, "unit": "GB/s", "cores": min(n, cores), "kind": "port",
            "sample": "{} in-place all-reduces of a {} MiB fp32 {} sample per rank over {} rank processes on shared "
                      "memory (median of the last {}); bus GB/s = S/t * 2(n-1)/n; Open MPI is not installed on this "
                      "machine, so the CPU restatement of the MPI path is timed".format(
                          iters, sample_bytes // MiB, reduction, n, iters - 1),
            "ms_per_op": t * 1e3, "host_cores": cores}


# --------------------------------------------------------------------------
# N = 1

def bench_single(args):
    import torch
    from dragon_b200 import _C
    from dragon_b200.comm import Communicator

    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    esize = torch.tensor([], dtype=torch_dtype_of(args.dtype)).element_size()
    count = int(args.size_mib * MiB) // esize
    S = count * esize
    comm = Communicator.init_local(0, 1, 0)
    x = make_message(0, count, args.dtype, dev)
    y = torch.empty_like(x)
    op = comm.prepare_all_reduce([x], [y], args.reduction)
    lib = _C.lib()

    sampler = ClockSampler(0)
    with sampler:
        launches0 = lib.dgn_launch_count()
        per, total_ms = time_steps(op, args.steps, args.warmup)
        launches = lib.dgn_launch_count() - launches0 - args.warmup
        # End to end: host buffers in, host result out, copies inside the timed region.
        xh = x.cpu().pin_memory()
        yh = torch.empty_like(xh).pin_memory()
        e2e_steps = max(3, min(args.steps, 10))
        x2, y2 = torch.empty_like(x), torch.empty_like(y)
        e2e_ms = time_e2e(comm, xh, yh, [x, x2], [y, y2], args.reduction, e2e_steps, 2)
        copies = time_host_copies(xh, yh, x2)
        del x2, y2
    assert torch.equal(yh, xh), "local-copy path returned different bytes"
    ms = total_ms / args.steps
    kernel_ms = statistics.mean(per)
    peak, peak_kind = hbm_peak()
    achieved = 2.0 * S / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC,
        "value": S / (ms * 1e-3) / 1e9,
        "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic",
        "config": {
            "workload": "Collective ALLREDUCE reduction={} {} {:g} MiB per rank, out of place, comm_size=1 "
                        "(local-copy path; value = algorithm GB/s S/t)".format(args.reduction, args.dtype, args.size_mib),
            "message_bytes": S, "world_size": 1,
            "l2": "message ({:g} MiB) larger than the 126 MB L2; no flush between steps".format(args.size_mib),
            "values": "uniform[-1,1) from numpy default_rng(1000+rank)",
        },
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak,
                     # 1.8261 DRAM bytes per message byte (read + write) in the ncu capture of this kernel.
                     "traffic": 1.8261 * S,
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at 256 MiB "
                                       "(profiles/local_copy_kernel_256MiB.md), scaled by the message size; "
                                       "not measured in this run",
                     "peak_kind": peak_kind,
                     "algorithmic_bytes_per_launch": 2 * S, "kernel": "local_copy_kernel",
                     "kernel_ms": kernel_ms},
        "e2e": {"value": S / (e2e_ms / e2e_steps * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": S, "d2h_bytes_per_step": S, "ms_per_step": e2e_ms / e2e_steps,
                "pipeline": "H2D, all-reduce and D2H on three streams, two device buffers",
                "h2d_alone_gbs": copies["h2d_gbs"], "d2h_alone_gbs": copies["d2h_gbs"]},
        "gpu_launches": int(launches),
        "clocks": sampler.summary(),
    }
    del x, y
    if not args.no_emulated:
        line["emulated_ranks_one_gpu"] = bench_emulated(args)
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_local_copy_baseline(args)
        line["cpu_baseline_config1"] = cpu_config1_baseline()
    comm.destroy()
    return line


# Kernels of the multi-rank paths on 8 virtual ranks of ONE device: name ->
# (operation, forced variant, bytes per rank, tuning).  All "peer" traffic is
# local HBM traffic there; the cases exist so that each kernel can be timed
# and captured under a profiler on a single GPU.
EMULATED_CASES = {
    "ll_oneshot_64KiB": ("allreduce", 4, 64 << 10, {}),
    "ll_twoshot_1MiB": ("allreduce", 5, 1 << 20, {}),
    "oneshot_256KiB": ("allreduce", 1, 256 << 10, {}),
    "twoshot_lockstep_4MiB": ("allreduce", 2, 4 << 20, {}),
    "twoshot_64MiB": ("allreduce", 2, 64 << 20, {}),
    "ring_64MiB": ("allreduce", 7, 64 << 20, {}),
    "allgather_ll_64KiB": ("allgather", 4, 64 << 10, {}),
    "allgather_8MiB": ("allgather", 2, 8 << 20, {}),
    "allgather_pull_8MiB": ("allgather", 1, 8 << 20, {}),
    "allgather_staged_loads_8MiB": ("allgather", 8, 8 << 20, {}),
    "allgather_staged_stores_8MiB": ("allgather", 7, 8 << 20, {}),
    "broadcast_staged_16MiB": ("broadcast", 7, 16 << 20, {}),
    "broadcast_pull_512KiB": ("broadcast", 1, 512 << 10, {}),
    "broadcast_scatter_64MiB": ("broadcast", 2, 64 << 20, {}),
    "reducescatter_8MiB": ("reducescatter", 2, 8 << 20, {}),
}


def run_emulated_case(comms, name, iters=10, warm=3):
    import torch
    kind, variant, nbytes, tuning = EMULATED_CASES[name]
    n = len(comms)
    count = nbytes // 4
    for c in comms:
        c.set_tuning(variant=variant, **tuning)
    try:
        if kind == "allreduce":
            xs = [make_message(r, count, "f32", "cuda:0") for r in range(n)]
            ops = [c.prepare_all_reduce([x], [x], "MEAN") for c, x in zip(comms, xs)]
            step = lambda: [op() for op in ops]  # noqa: E731
        elif kind == "allgather":
            xs = [make_message(r, count, "f32", "cuda:0") for r in range(n)]
            ys = [torch.empty(n * count, device="cuda:0") for _ in range(n)]
            step = lambda: [c.all_gather(x, y) for c, x, y in zip(comms, xs, ys)]  # noqa: E731
        elif kind == "broadcast":
            xs = [make_message(r, count, "f32", "cuda:0") for r in range(n)]
            step = lambda: [c.broadcast(x, 0) for c, x in zip(comms, xs)]  # noqa: E731
        else:
            xs = [make_message(r, n * count, "f32", "cuda:0") for r in range(n)]
            ys = [torch.empty(count, device="cuda:0") for _ in range(n)]
            step = lambda: [c.reduce_scatter(x, y, "SUM") for c, x, y in zip(comms, xs, ys)]  # noqa: E731
        _, total = time_steps(step, iters, warm)
        return {"ms": total / iters, "bytes_per_rank": nbytes, "launch": comms[0].last_launch()}
    finally:
        for c in comms:
            c.set_tuning()


def bench_emulated(args):
    """The multi-rank kernels with 8 virtual ranks on this one GPU (all "peer"
    traffic is local HBM traffic): times the kernels the multi-GPU runs use."""
    import torch
    from dragon_b200.comm import Communicator
    out = {}
    comms = Communicator.emulated(8, 0)
    try:
        names = sorted(EMULATED_CASES) if args.emulated_case in ("default", "all") else \
            [n for n in (args.emulated_case,) if n in EMULATED_CASES]
        if args.emulated_case == "default" and not args.emulated_only:
            names = ["ll_oneshot_64KiB", "twoshot_64MiB", "ring_64MiB", "allgather_8MiB"]
        for name in names:
            out[name] = run_emulated_case(comms, name)
        if args.emulated_case in ("all", "fused_adam_64MiB"):
            # All-reduce fused with the Adam update: eight fp32 tensors of 2 Mi elements per rank (64 MiB of gradients).
            from dragon_b200.fused_optim import FusedAdam
            fopts = []
            for r, c in enumerate(comms):
                g = torch.Generator(device="cuda:0").manual_seed(2000 + r)
                params = [torch.randn(2 << 20, generator=g, device="cuda:0") for _ in range(8)]
                for p in params:
                    p.grad = torch.randn(2 << 20, generator=g, device="cuda:0") * 1e-2
                fopts.append(FusedAdam(params, lr=1e-4, comm=c))
            _, total = time_steps(lambda: [o.step() for o in fopts], 10, 3)
            out["fused_adam_64MiB"] = {"ms": total / 10, "bytes_per_rank": 64 << 20, "launch": comms[0].last_launch()}
            del fopts
        if args.emulated_case in ("default", "all", "zero_adamw_64MiB_fp16"):
            # The sharded AdamW step: eight fp16 tensors of 4 Mi elements per rank (64 MiB), overflow check on.
            from dragon_b200.zero import ZeroAdamW
            opts, found = [], []
            for r, c in enumerate(comms):
                g = torch.Generator(device="cuda:0").manual_seed(1000 + r)
                params = [torch.randn(4 << 20, generator=g, device="cuda:0").to(torch.float16) for _ in range(8)]
                for p in params:
                    p.grad = (torch.randn(4 << 20, generator=g, device="cuda:0") * 1e-2).to(torch.float16)
                opts.append(ZeroAdamW(params, c, lr=1e-4))
                found.append(torch.zeros(1, device="cuda:0"))

            def zero_step():
                for o, f in zip(opts, found):
                    o.step(found_inf=f)

            per, total = time_steps(zero_step, 10, 3)
            out["zero_adamw_64MiB_fp16"] = {"ms": total / 10, "launch": comms[0].last_launch(),
                                            "found_inf": float(found[0].item())}
            del opts
    finally:
        torch.cuda.synchronize()
        for c in comms:
            c.destroy()
    return out


def cpu_local_copy_baseline(args):
    """The oracle's comm_size-1 out-of-place path on one host core, on the
    message of the timed step (a few passes)."""
    import numpy as np
    from dragon_b200 import workloads
    from oracle import oracle
    count = int(args.size_mib * MiB) // 4
    x = workloads.uniform_message(0, count)
    y = np.zeros_like(x)
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or time.perf_counter() - t0 < 3.0:
        oracle.allreduce([x], oracle.F32, "MEAN", out=y)
        reps += 1
    t = (time.perf_counter() - t0) / reps
    assert np.array_equal(x, y)
    return {"value": x.nbytes / t / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": "{} passes of the oracle's comm_size=1 all-reduce over the {} MiB fp32 message".format(
                reps, x.nbytes // MiB), "host_cores": os.cpu_count()}


# --------------------------------------------------------------------------
# N >= 2: parity of every variant against the CPU oracle, before anything is timed

def _np_message(rank, count, kind, seed_shift=0):
    """Seeded per-rank input in oracle storage (bf16 as uint16 bit patterns);
    every rank can rebuild every other rank's input, so no data is exchanged."""
    import numpy as np
    from oracle import oracle
    rng = np.random.default_rng(1000 + rank + 100 * seed_shift)
    if kind == "i64":
        return rng.integers(0, 1 << 40, count, dtype=np.int64)
    x = rng.uniform(-1.0, 1.0, count).astype(np.float32)
    if kind == "f16":
        return x.astype(np.float16)
    if kind == "bf16":
        return oracle.f32_to_bf16_bits(x)
    return x


def _to_device(arr, kind, dev):
    import torch
    t = torch.from_numpy(arr.copy())
    if kind == "bf16":
        t = t.view(torch.int16).view(torch.bfloat16) if t.dtype != torch.uint16 else t.view(torch.bfloat16)
    return t.to(dev)


def _to_host(t, kind):
    import numpy as np
    import torch
    t = t.detach().cpu().contiguous()
    if kind == "bf16":
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def parity_pass(comm, rank, world, dev, dist, headline):
    """Runs every kernel variant the planner can pick at this rank count once,
    on messages that span several rounds / chunks and end in a ragged tail, and
    checks the WHOLE output on EVERY rank against the CPU oracle: bit for bit
    for the kernels that add in ascending rank order and for everything that
    only moves bytes; for the kernels that let the NVSwitch add, within the
    tolerance contract of an fp64 host sum, with identical bits on all ranks.
    Returns {case: {"elements", "max_rel_err", "bit_exact", "ranks_identical", "variant", "ok"}}."""
    import numpy as np
    import torch
    from oracle import oracle

    okind = {"f32": oracle.F32, "f16": oracle.F16, "bf16": oracle.BF16, "i64": oracle.I64}
    results = {}

    def same_on_all_ranks(arrays):
        crc = 0
        for a in arrays:
            crc = zlib.crc32(np.ascontiguousarray(a).view(np.uint8), crc)
        box = [None] * world
        dist.all_gather_object(box, crc)
        return len(set(box)) == 1

    def all_ranks(flag):
        box = [None] * world
        dist.all_gather_object(box, bool(flag))
        return all(box)

    def judge(name, kind, got_list, want_list, ref64_list, ordered, variant):
        elements = int(sum(g.size for g in got_list))
        exact = all(np.array_equal(np.ascontiguousarray(g).view(np.uint8), np.ascontiguousarray(w).view(np.uint8))
                    for g, w in zip(got_list, want_list))
        err = 0.0
        if ref64_list is not None:
            err = max(oracle.max_rel_err(g, r64, okind[kind]) for g, r64 in zip(got_list, ref64_list))
        tol = oracle.TOLERANCE.get(okind[kind], 0.0)
        same = same_on_all_ranks(got_list)
        ok = (exact if ordered else err <= tol) and same and comm.status() == 0
        results[name] = {"elements": elements, "max_rel_err": err, "bit_exact": bool(exact),
                         "ranks_identical": bool(same), "ordered": bool(ordered), "variant": variant,
                         "ok": all_ranks(ok)}

    def tune(variant=0, **kw):
        knobs = {k: kw.pop(k) for k in list(kw) if k in ("flow_depth", "nvls_unroll", "gather_mode")}
        comm.set_tuning(variant=variant, **kw)
        for k in ("flow_depth", "nvls_unroll", "gather_mode"):
            comm.set_knob(k, knobs.get(k, 0))

    def allreduce_case(name, variant, kind, count, redop, ordered=True, symm=False, shift=0, want_rounds=0, **shape):
        tune(variant, **shape)
        ins = [_np_message(r, count, kind, shift) for r in range(world)]
        if symm:
            comm.symm_reset()
            x = comm.symm_empty(count, torch_dtype_of(kind))
            x.copy_(_to_device(ins[rank], kind, dev))
        else:
            x = _to_device(ins[rank], kind, dev)
        comm.all_reduce([x], None, redop)
        torch.cuda.synchronize()
        launch = comm.last_launch()
        got = _to_host(x, kind)
        want = oracle.allreduce(ins, okind[kind], redop)
        ref = oracle.fp64_sum(ins, okind[kind], mean=(redop == "MEAN")) if kind != "i64" else None
        judge(name, kind, [got], [want], None if ref is None else [ref], ordered, launch["variant"])
        if variant and launch["variant"] != variant:
            results[name]["ok"] = False
            results[name]["note"] = "asked for variant {}, ran {}".format(variant, launch["variant"])
        if want_rounds and launch["rounds"] < want_rounds:
            results[name]["ok"] = False
            results[name]["note"] = "expected at least {} rounds, ran {}".format(want_rounds, launch["rounds"])
        if symm:
            del x
            comm.symm_reset()

    def bucket_case(name, variant, kind, counts, redop, ordered=True, **shape):
        tune(variant, **shape)
        ins = [[_np_message(r, k, kind, 7 + i) for i, k in enumerate(counts)] for r in range(world)]
        xs = [_to_device(a, kind, dev) for a in ins[rank]]
        comm.all_reduce(xs, None, redop)
        torch.cuda.synchronize()
        launch = comm.last_launch()
        got = [_to_host(x, kind) for x in xs]
        want = [oracle.allreduce([ins[r][i] for r in range(world)], okind[kind], redop) for i in range(len(counts))]
        ref = [oracle.fp64_sum([ins[r][i] for r in range(world)], okind[kind], mean=(redop == "MEAN"))
               for i in range(len(counts))]
        judge(name, kind, got, want, ref, ordered, launch["variant"])

    nvls = comm.has_nvls()
    symm = nvls and comm.symm_capacity() >= 32 * MiB
    ragged_bucket = [70001, 3, 1 << 19, 257, (1 << 20) + 1, 64]

    allreduce_case("allreduce/ll_oneshot", 4, "f32", 4099, "MEAN")
    allreduce_case("allreduce/ll_twoshot", 5, "f16", 300001, "MEAN")
    allreduce_case("allreduce/oneshot", 1, "bf16", 70001, "SUM")
    allreduce_case("allreduce/twoshot_lockstep", 2, "f32", 1000003, "MEAN")
    allreduce_case("allreduce/twoshot_warp_specialised", 2, "f32", 2000003, "MEAN", want_rounds=3,
                   blocks=8, chunk_bytes=16 << 10)
    allreduce_case("allreduce/twoshot_int64_sum", 2, "i64", 70001, "SUM")
    allreduce_case("allreduce/staged_ring_peer", 7, "f16", 3000001, "MEAN", want_rounds=9, chunk_bytes=256 << 10,
                   flow_depth=4)
    bucket_case("allreduce/bucket_twoshot", 2, "f32", ragged_bucket, "MEAN")
    bucket_case("allreduce/bucket_ll_twoshot", 5, "f16", [4099, 1, 77, 30000], "MEAN")
    if nvls:
        allreduce_case("allreduce/staged_ring_multicast_f32", 3, "f32", (1 << 22) + 3, "MEAN", ordered=(world == 2),
                       want_rounds=9, chunk_bytes=1 << 20, nvls_unroll=4)
        allreduce_case("allreduce/staged_ring_multicast_f16", 3, "f16", (1 << 23) + 1, "MEAN", ordered=False,
                       want_rounds=9, chunk_bytes=1 << 20, nvls_unroll=16, flow_depth=4)
        allreduce_case("allreduce/staged_ring_multicast_bf16_one_chunk", 3, "bf16", 70001, "SUM", ordered=False)
        bucket_case("allreduce/bucket_staged_ring_multicast", 3, "f32", ragged_bucket, "MEAN", ordered=(world == 2),
                    chunk_bytes=1 << 20)
    if symm:
        allreduce_case("allreduce/in_place_multicast_f32", 6, "f32", (1 << 22) + 4, "MEAN", ordered=(world == 2),
                       symm=True)
        allreduce_case("allreduce/in_place_multicast_bf16", 6, "bf16", 1 << 21, "SUM", ordered=False, symm=True)
    tune(0)

    # ALLGATHER / BROADCAST / REDUCESCATTER: bytes move, everything is bit-exact.
    def gather_case(name, variant, kind, count, **shape):
        tune(variant, **shape)
        ins = [_np_message(r, count, kind, 3) for r in range(world)]
        x = _to_device(ins[rank], kind, dev)
        y = torch.empty(world * count, dtype=x.dtype, device=dev)
        comm.all_gather(x, y)
        torch.cuda.synchronize()
        judge(name, kind, [_to_host(y, kind)], [oracle.allgather(ins, okind[kind])], None, True,
              comm.last_launch()["variant"])

    def broadcast_case(name, variant, kind, count, root, **shape):
        tune(variant, **shape)
        ins = [_np_message(r, count, kind, 5 + root) for r in range(world)]
        x = _to_device(ins[rank], kind, dev)
        comm.broadcast(x, root)
        torch.cuda.synchronize()
        judge(name, kind, [_to_host(x, kind)], [ins[root]], None, True, comm.last_launch()["variant"])

    def reducescatter_case(name, kind, count, redop):
        tune(0)
        ins = [_np_message(r, world * count, kind, 9) for r in range(world)]
        x = _to_device(ins[rank], kind, dev)
        y = torch.empty(count, dtype=x.dtype, device=dev)
        comm.reduce_scatter(x, y, redop)
        torch.cuda.synchronize()
        want = oracle.reducescatter(ins, okind[kind], redop)[rank]
        got = _to_host(y, kind)
        exact = np.array_equal(got.view(np.uint8), np.ascontiguousarray(want).view(np.uint8))
        results[name] = {"elements": int(got.size), "max_rel_err": 0.0, "bit_exact": bool(exact),
                         "ranks_identical": None, "ordered": True, "variant": comm.last_launch()["variant"],
                         "ok": all_ranks(exact and comm.status() == 0)}

    gather_case("allgather/low_latency", 4, "i64", 4099)
    gather_case("allgather/push_int64", 2, "i64", 65536)
    gather_case("allgather/push_bf16_many_rounds", 2, "bf16", (1 << 21) + 3, blocks=8, chunk_bytes=32 << 10)
    gather_case("allgather/pull_bf16_many_rounds", 1, "bf16", (1 << 21) + 3, blocks=8, chunk_bytes=32 << 10)
    gather_case("allgather/staged_peer_stores", 7, "f16", (1 << 20) + 5, blocks=2, chunk_bytes=16 << 10)
    gather_case("allgather/staged_peer_loads", 8, "bf16", (1 << 21) + 3, chunk_bytes=64 << 10)
    gather_case("allgather/planner_choice_large", 0, "f32", (1 << 22) + 1)
    if nvls:
        gather_case("allgather/staged_multicast", 3, "bf16", (1 << 21) + 3, chunk_bytes=32 << 10)
        gather_case("allgather/staged_multicast_default_shape", 3, "i64", (1 << 20) + 1)
    for root in sorted({0, world - 1}):
        broadcast_case("broadcast/pull_root{}".format(root), 1, "i64", 65536, root)
        broadcast_case("broadcast/staged_peer_stores_root{}".format(root), 7, "bf16", (1 << 20) + 3, root,
                       chunk_bytes=16 << 10, gather_mode=1)
        broadcast_case("broadcast/staged_shards_peer_stores_root{}".format(root), 7, "bf16", (1 << 20) + 3, root,
                       chunk_bytes=64 << 10, gather_mode=2)
        if world > 2:
            broadcast_case("broadcast/scatter_root{}".format(root), 2, "bf16", (1 << 22) + 3, root)
        if nvls:
            broadcast_case("broadcast/multicast_root{}".format(root), 3, "bf16", (1 << 22) + 3, root,
                           chunk_bytes=128 << 10, gather_mode=1)
            broadcast_case("broadcast/multicast_shards_root{}".format(root), 3, "bf16", (1 << 22) + 3, root,
                           chunk_bytes=512 << 10, gather_mode=2)
            broadcast_case("broadcast/planner_choice_large_root{}".format(root), 0, "f32", (1 << 22) + 1, root)
    reducescatter_case("reducescatter/f32_mean", "f32", 300001, "MEAN")
    reducescatter_case("reducescatter/int64_sum", "i64", 4099, "SUM")
    tune(0)

    # The timed message itself, with the variant the planner picks for it: whole
    # output, every rank, checked slice by slice against regenerated inputs.
    x, count, kind, reduction = headline
    x0 = x.clone()
    comm.all_reduce([x], None, reduction)
    torch.cuda.synchronize()
    launch = comm.last_launch()
    ordered = launch["variant"] not in (3, 6) or world == 2
    got = _to_host(x, kind)
    rngs = [np.random.default_rng(1000 + r) for r in range(world)]
    exact, err, piece = True, 0.0, 1 << 22
    for lo in range(0, count, piece):
        hi = min(count, lo + piece)
        ins = []
        for g in rngs:
            v = g.uniform(-1.0, 1.0, hi - lo).astype(np.float32)
            ins.append(v if kind == "f32" else (v.astype(np.float16) if kind == "f16" else oracle.f32_to_bf16_bits(v)))
        want = oracle.allreduce(ins, okind[kind], reduction)
        exact = exact and np.array_equal(got[lo:hi].view(np.uint8), np.ascontiguousarray(want).view(np.uint8))
        err = max(err, oracle.max_rel_err(got[lo:hi], oracle.fp64_sum(ins, okind[kind], mean=(reduction == "MEAN")),
                                          okind[kind]))
    same = same_on_all_ranks([got])
    ok = (exact if ordered else err <= oracle.TOLERANCE[okind[kind]]) and same and comm.status() == 0
    results["allreduce/timed_message"] = {"elements": int(count), "max_rel_err": err, "bit_exact": bool(exact),
                                          "ranks_identical": bool(same), "ordered": bool(ordered),
                                          "variant": launch["variant"], "ok": all_ranks(ok)}
    x.copy_(x0)
    torch.cuda.synchronize()
    return results


def link_bytes_per_direction(variant, S, n):
    """NVLink bytes one rank sends (= receives) per launch, from the algorithm of the variant."""
    if variant in (3, 6):
        return S * (1.0 + 1.0 / n)          # ld_reduce serves S, st sends S / n (and the reverse inbound)
    if variant in (1, 4):
        return S * (n - 1) * (2.0 if variant == 4 else 1.0)   # whole message to every peer; lines are half flags
    if variant == 5:
        return 4.0 * S * (n - 1) / n
    return 2.0 * S * (n - 1) / n             # two-shot and the staged ring with peer loads / stores


# --------------------------------------------------------------------------
# N >= 2 (one process per GPU under torch.distributed.run)

def bench_multi(args):
    import torch
    import torch.distributed as dist
    from dragon_b200 import _C
    from dragon_b200.comm import Communicator

    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    own_cores = pin_rank_to_its_cores(local, world)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group(backend="gloo")  # plumbing only: handle exchange, barriers, max over ranks

    def barrier():
        dist.barrier()

    def max_over_ranks(v):
        t = torch.tensor([float(v)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def min_over_ranks(v):
        t = torch.tensor([float(v)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return float(t.item())

    # 256 MiB of symmetric memory per rank for the in-place multicast rows.
    comm = Communicator.init_local(rank, world, local, symm_bytes=0 if args.no_symm else 256 * MiB)
    handles = [None] * world
    dist.all_gather_object(handles, comm.handle_bytes())
    comm.connect(handles)
    barrier()
    lib = _C.lib()
    stream = torch.cuda.current_stream().cuda_stream

    nccl = None
    if not args.no_nccl:
        from baseline.nccl_backend import NcclBackend

        def exchange(payload):
            box = [payload]
            dist.broadcast_object_list(box, src=0)
            return box[0]

        # All ranks must agree before anyone enters ncclCommInitRank.
        try:
            from baseline.nccl_backend import _find_library
            _find_library()
            have = 1.0
        except Exception:
            have = 0.0
        flag = torch.tensor([have], dtype=torch.float64)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        nccl = NcclBackend(rank, world, exchange) if flag.item() > 0 else None

    tdtype = torch_dtype_of(args.dtype)
    esize = torch.tensor([], dtype=tdtype).element_size()
    count = int(args.size_mib * MiB) // esize
    S = count * esize
    x = make_message(rank, count, args.dtype, dev)
    x0 = x.clone()
    op = comm.prepare_all_reduce([x], [x], args.reduction)
    factor = 2.0 * (world - 1) / world

    # Parity first: nothing is timed, and no row is printed, before every variant has matched the oracle.
    parity = None
    if not args.no_parity:
        parity = parity_pass(comm, rank, world, dev, dist, (x, count, args.dtype, args.reduction.upper()))
        bad = sorted(k for k, v in parity.items() if not v["ok"])
        if bad:
            if rank == 0:
                emit_result({"metric": METRIC, "n_gpus": world, "parity_failed": bad, "parity": parity})
            barrier()
            torch.cuda.synchronize()
            if nccl is not None:
                nccl.destroy()
            comm.destroy()
            dist.destroy_process_group()
            sys.exit(3)

    sampler = ClockSampler(local)
    with sampler:
        launches0 = lib.dgn_launch_count()
        per, total_ms = time_steps(op, args.steps, args.warmup, barrier)
        launches = lib.dgn_launch_count() - launches0 - args.warmup
        launch = comm.last_launch()
        xh = x0.cpu().pin_memory()
        yh = torch.empty_like(xh).pin_memory()
        e2e_steps = max(3, min(args.steps, 10))
        x2 = torch.empty_like(x)
        e2e_ms = time_e2e(comm, xh, yh, [x, x2], [x, x2], args.reduction, e2e_steps, 2, barrier)
        copies = time_host_copies(xh, yh, x2, barrier)
        del x2
    ms = max_over_ranks(total_ms) / args.steps
    kernel_ms = max_over_ranks(statistics.mean(per))
    e2e_ms = max_over_ranks(e2e_ms) / e2e_steps
    h2d = min_over_ranks(copies["h2d_gbs"])
    d2h = min_over_ranks(copies["d2h_gbs"])
    busbw = S / (ms * 1e-3) / 1e9 * factor
    del xh, yh

    cpu = None
    if not args.no_cpu_baseline:
        if rank == 0:
            cpu = cpu_multi_baseline(world, args.reduction)
        barrier()

    sweep = run_sweep(args, comm, nccl, rank, world, dev, stream, barrier, max_over_ranks) if args.sweep != "off" else []
    extras = {}
    if args.configs == "auto":
        extras = run_operator_configs(comm, nccl, rank, world, dev, barrier, max_over_ranks)
    if args.configs != "off":
        extras["zero_adamw_bert_base_fp16"] = run_zero_config(comm, nccl, rank, world, dev, barrier, max_over_ranks)

    # Last, so that a failure here cannot cost the numbers above.
    symmetric = None
    if not args.no_symm:
        try:
            symmetric = run_symmetric(comm, rank, world, barrier, max_over_ranks)
        except Exception as e:  # noqa: BLE001 - report, do not lose the line
            symmetric = {"error": str(e)[:300]}

    line = None
    if rank == 0:
        achieved = S / (kernel_ms * 1e-3) / 1e9 * factor
        link = link_bytes_per_direction(launch["variant"], S, world)
        line = {
            "metric": METRIC,
            "value": busbw, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": args.dtype, "data": "synthetic",
            "config": {
                "workload": "Collective ALLREDUCE reduction={} {} {:g} MiB per rank, in place, comm_size={}".format(
                    args.reduction, args.dtype, args.size_mib, world),
                "message_bytes": S, "world_size": world,
                "busbw": "S/t * 2(n-1)/n", "frac_of_900": busbw / NVLINK_NOMINAL_GBS,
                "l2": "message ({:g} MiB) larger than the 126 MB L2; sweep points rotate over buffers "
                      "totalling >= 256 MiB".format(args.size_mib),
                "values": "uniform[-1,1) from numpy default_rng(1000+rank)",
                "launch": launch, "kernel": VARIANT_NAMES.get(launch["variant"], "?"),
            },
            "roofline": {"bound": "nvlink", "achieved": achieved, "peak": NVLINK_NOMINAL_GBS, "unit": "GB/s",
                         "frac": achieved / NVLINK_NOMINAL_GBS,
                         "traffic": link,
                         "traffic_kind": "NVLink bytes one rank sends (and receives) per launch, from the algorithm "
                                         "of the variant that ran; DRAM bytes need an ncu capture, which a "
                                         "multi-rank run does not take",
                         "link_gbs_per_direction": link / (kernel_ms * 1e-3) / 1e9,
                         "peak_kind": "nominal per direction per GPU; measured peer copy on this pool is "
                                      "{:g} GB/s".format(NVLINK_MEASURED_P2P_GBS),
                         "frac_of_measured_p2p": achieved / NVLINK_MEASURED_P2P_GBS,
                         "algorithmic_bytes_per_launch": S * factor, "kernel_ms": kernel_ms},
            "e2e": {"value": S / (e2e_ms * 1e-3) / 1e9 * factor, "unit": "GB/s",
                    "h2d_bytes_per_step": S, "d2h_bytes_per_step": S, "ms_per_step": e2e_ms,
                    "pipeline": "H2D, all-reduce and D2H on three streams, two device buffers",
                    "h2d_alone_gbs_per_rank": h2d, "d2h_alone_gbs_per_rank": d2h,
                    "host_cores_per_rank": own_cores,
                    "note": "every rank moves its message over PCIe in both directions at the same time; the "
                            "per-rank copy rates above (slowest rank, all ranks copying) bound the step"},
            "gpu_launches": int(launches),
            "clocks": sampler.summary(),
            "parity": parity,
            "sweep": sweep,
            "operator_configs": extras,
            "nvls": comm.has_nvls(),
            "symmetric_memory": symmetric,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
    barrier()
    torch.cuda.synchronize()
    if nccl is not None:
        nccl.destroy()
    comm.destroy()
    dist.destroy_process_group()
    return line


def run_operator_configs(comm, nccl, rank, world, dev, barrier, max_over_ranks):
    """The gradient-bucket and gather/broadcast configurations, operator to
    operator: ours is one fused launch per bucket; the NCCL backend restated as
    the reference runs it (concat copies, ncclAllReduce, split copies, one
    scale launch per tensor for MEAN)."""
    import torch
    from dragon_b200 import workloads
    out = {}
    stream_of = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731

    def timed(fn, iters=10, warm=3):
        _, total = time_steps(fn, iters, warm, barrier)
        return max_over_ranks(total) / iters

    def gen(shapes, std, dtype):
        g = torch.Generator(device=dev).manual_seed(1000 + rank)
        return [(torch.randn(workloads.numel(s), generator=g, device=dev) * std).to(dtype) for s in shapes]

    # ResNet-50: 161 fp32 tensors, one bucket, MEAN.
    shapes = workloads.resnet50_shapes()
    grads = gen(shapes, 1e-3, torch.float32)
    nbytes = sum(g.numel() * 4 for g in grads)
    op = comm.prepare_all_reduce(grads, grads, "MEAN")
    row = {"tensors": len(grads), "bytes": nbytes, "ours_us": timed(op) * 1e3, "launch": comm.last_launch()}
    if nccl is not None:
        scratch = torch.empty(nbytes // 4, device=dev)
        row["nccl_us"] = timed(lambda: nccl.operator_all_reduce(grads, "MEAN", stream_of(), bucket=scratch)) * 1e3
        row["nccl_unbucketed_us"] = timed(lambda: nccl.operator_all_reduce(grads, "MEAN", stream_of())) * 1e3
        row["speedup"] = row["nccl_us"] / row["ours_us"]
        del scratch
    row["ours_busbw"] = nbytes / (row["ours_us"] * 1e-6) / 1e9 * 2.0 * (world - 1) / world
    out["resnet50_fp32_one_bucket_mean"] = row
    del op

    # The same gradients with the optimizer update fused into the all-reduce
    # (momentum SGD on all 161 tensors): one kernel against the reference's
    # all-reduce followed by its update operator.
    from dragon_b200.fused_optim import FusedSGD
    params = gen(shapes, 1.0, torch.float32)
    for p, g in zip(params, grads):
        p.grad = g
    opt = FusedSGD(params, 0.1, momentum=0.9, weight_decay=1e-4, comm=comm)
    row = {"tensors": len(grads), "bytes": nbytes, "ours_us": timed(opt.step) * 1e3, "launch": comm.last_launch()}
    if nccl is not None:
        scratch = torch.empty(nbytes // 4, device=dev)
        momenta = [torch.zeros_like(p) for p in params]
        hyper = {"lr": 0.1, "momentum": 0.9, "weight_decay": 1e-4, "grad_scale": 1.0 / world}
        try:
            row["nccl_us"] = timed(lambda: nccl.operator_all_reduce_sgd(grads, params, momenta, hyper, stream_of(),
                                                                          bucket=scratch)) * 1e3
            row["speedup"] = row["nccl_us"] / row["ours_us"]
        except (RuntimeError, TypeError, AttributeError) as e:  # a torch build without the fused SGD op
            row["nccl_error"] = str(e)[:200]
        del scratch, momenta
    out["resnet50_fp32_allreduce_fused_with_sgd"] = row
    del grads, params, opt

    # BERT-base: 199 fp16 tensors in 25 MiB buckets, MEAN with fp32 accumulation.
    shapes = workloads.bert_base_shapes()
    grads = gen(shapes, 1e-2, torch.float16)
    buckets = workloads.greedy_buckets(shapes, 2, 25 * MiB)
    ops = [comm.prepare_all_reduce([grads[i] for i in b], [grads[i] for i in b], "MEAN") for b in buckets]
    nbytes = sum(g.numel() * 2 for g in grads)

    def ours_all():
        for o in ops:
            o()

    row = {"tensors": len(grads), "buckets": len(buckets), "bytes": nbytes, "ours_us": timed(ours_all, 5, 2) * 1e3}
    if nccl is not None:
        scratch = torch.empty(max(sum(grads[i].numel() for i in b) for b in buckets), dtype=torch.float16, device=dev)

        def theirs_all():
            for b in buckets:
                nccl.operator_all_reduce([grads[i] for i in b], "MEAN", stream_of(), bucket=scratch if len(b) > 1 else None)

        row["nccl_us"] = timed(theirs_all, 5, 2) * 1e3
        row["speedup"] = row["nccl_us"] / row["ours_us"]
        del scratch
    row["ours_busbw"] = nbytes / (row["ours_us"] * 1e-6) / 1e9 * 2.0 * (world - 1) / world
    out["bert_base_fp16_25MiB_buckets_mean"] = row
    del grads, ops

    # ALLGATHER / BROADCAST(root 0): int64 [65536] and bf16 [8192, 4096].
    for label, make in (("int64_65536", lambda: torch.randint(0, 1 << 40, (65536,), device=dev, dtype=torch.int64)),
                        ("bf16_8192x4096", lambda: torch.randn(8192, 4096, device=dev).to(torch.bfloat16))):
        x = make()
        y = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=dev)
        sbytes = x.numel() * x.element_size()
        iters = 50 if sbytes < MiB else 10
        t_ag = timed(lambda: comm.all_gather(x, y), iters)
        ag_launch = comm.last_launch()
        t_bc = timed(lambda: comm.broadcast(x, 0), iters)
        row = {"shard_bytes": sbytes, "allgather_us": t_ag * 1e3,
               "allgather_busbw": world * sbytes / t_ag / 1e6 * (world - 1) / world,
               "broadcast_us": t_bc * 1e3, "broadcast_busbw": sbytes / t_bc / 1e6,
               "allgather_variant": ag_launch["variant"], "broadcast_variant": comm.last_launch()["variant"]}
        if nccl is not None:
            row["nccl_allgather_us"] = timed(lambda: nccl.all_gather(x, y, stream_of()), iters) * 1e3
            row["nccl_broadcast_us"] = timed(lambda: nccl.broadcast(x, 0, stream_of()), iters) * 1e3
        out[label] = row
        del x, y

    # SyncBatchNorm statistics: per layer one all-reduce of 2C floats (sum and sum
    # of squares per channel), the latency path of normalization/batch_norm_op.cc:29-43.
    rows = []
    for channels in (64, 256, 2048):
        s = torch.randn(2 * channels, device=dev)
        op = comm.prepare_all_reduce([s], [s], "SUM")
        r = {"channels": channels, "bytes": 8 * channels, "ours_us": timed(op, 200, 10) * 1e3,
             "ours_graph_us": max_over_ranks(time_graph(op, 20, 10, barrier)) * 1e3}
        if nccl is not None:
            theirs = lambda: nccl.operator_all_reduce([s], "SUM", stream_of())  # noqa: E731
            r["nccl_us"] = timed(theirs, 200, 10) * 1e3
            r["nccl_graph_us"] = max_over_ranks(time_graph(theirs, 20, 10, barrier)) * 1e3
        rows.append(r)
        del s, op
    out["syncbn_statistics_2C_floats"] = rows
    return out


def run_symmetric(comm, rank, world, barrier, max_over_ranks):
    """MEAN all-reduce in place on buffers from the communicator's symmetric
    arena (dgn_comm_symm_alloc): the switch reduces the buffers themselves,
    nothing is staged.  Each size rotates over views that cover 256 MiB.  The
    kernel is forced here (at two ranks it is not the default); its parity was
    checked in the parity pass."""
    import torch
    if not comm.has_nvls() or comm.symm_capacity() < 256 * MiB:
        return {"available": False}
    factor = 2.0 * (world - 1) / world
    rows = []
    comm.set_tuning(variant=6)
    try:
        for dtype_name, sizes in (("f32", (4, 16, 64, 128, 256)), ("f16", (64, 256))):
            tdtype = torch_dtype_of(dtype_name)
            esize = 2 if dtype_name == "f16" else 4
            comm.symm_reset()
            arena = comm.symm_empty(256 * MiB // esize, tdtype)
            arena.copy_(make_message(rank, arena.numel(), dtype_name, arena.device))
            for mib in sizes:
                count = mib * MiB // esize
                nbuf = max(1, 256 // mib)
                views = [arena[k * count:(k + 1) * count] for k in range(nbuf)]
                ops = [comm.prepare_all_reduce([v], [v], "MEAN") for v in views]
                state = {"i": 0}

                def step():
                    ops[state["i"] % nbuf]()
                    state["i"] += 1

                iters = 40 if mib <= 64 else 10
                _, total = time_steps(step, iters, 5, barrier)
                t = max_over_ranks(total) / iters
                busbw = mib * MiB / (t * 1e-3) / 1e9 * factor
                rows.append({"dtype": dtype_name, "bytes": mib * MiB, "us": t * 1e3, "busbw": busbw,
                             "frac_of_900": busbw / NVLINK_NOMINAL_GBS, "variant": comm.last_launch()["variant"],
                             "launch": comm.last_launch()})
                del ops, views
            del arena
    finally:
        comm.set_tuning()
        comm.symm_reset()
    return {"available": True, "rows": rows,
            "note": "buffers allocated with dgn_comm_symm_alloc (same offset on every rank), reduced in place"}


def run_zero_config(comm, nccl, rank, world, dev, barrier, max_over_ranks):
    """One sharded AdamW step over the BERT-base parameter list (199 fp16
    tensors, one bucket, overflow check on): ours is two kernels per step
    (dgn_zero_adamw); the baseline is the sequence the reference's ZeroAdamW
    operator enqueues, with NCCL for its two collectives."""
    import torch
    from dragon_b200 import workloads
    from dragon_b200.zero import ZeroAdamW
    shapes = workloads.bert_base_shapes()
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    gp = torch.Generator(device=dev).manual_seed(5)
    params = [torch.randn(workloads.numel(s), generator=gp, device=dev).to(torch.float16) for s in shapes]
    grads = [(torch.randn(workloads.numel(s), generator=g, device=dev) * 1e-2).to(torch.float16) for s in shapes]
    for p, gr in zip(params, grads):
        p.grad = gr
    total = sum(p.numel() for p in params)
    found = torch.zeros(1, dtype=torch.float32, device=dev)
    opt = ZeroAdamW(params[::-1], comm, lr=1e-4, weight_decay=0.01)

    def timed(fn, iters=10, warm=3):
        _, ms = time_steps(fn, iters, warm, barrier)
        return max_over_ranks(ms) / iters

    row = {"tensors": len(params), "bytes": total * 2, "shard_elements": -(-total // world),
           "ours_us": timed(lambda: opt.step(found_inf=found)) * 1e3, "found_inf": float(found.item())}
    if nccl is not None:
        rc = -(-total // world)
        state = {"flat": torch.zeros(rc * (world + 1), dtype=torch.float16, device=dev),
                 "master": torch.zeros(rc, device=dev), "m": torch.zeros(rc, device=dev),
                 "v": torch.zeros(rc, device=dev), "step": torch.ones(1, device=dev)}
        hyper = {"lr": 1e-4, "beta1": 0.9, "beta2": 0.999, "eps": 1e-8, "weight_decay": 0.01,
                 "grad_scale": 1.0 / world}
        stream_of = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
        try:
            row["nccl_us"] = timed(lambda: nccl.operator_zero_adamw(grads, params, state, hyper, stream_of())) * 1e3
            row["speedup"] = row["nccl_us"] / row["ours_us"]
        except (RuntimeError, TypeError, AttributeError) as e:  # e.g. a torch build without the fused AdamW op
            row["nccl_error"] = str(e)[:200]
    # Link bytes per rank and direction: (n-1)/n of the gradients out, the same of the parameters in.
    row["ours_busbw"] = total * 2 / (row["ours_us"] * 1e-6) / 1e9 * 2.0 * (world - 1) / world
    return row


def time_graph(fn, ops_per_graph, replays, barrier):
    """Device time per call of fn() with the host out of the way: `ops_per_graph`
    calls are captured into one CUDA graph and the graph is replayed."""
    import torch
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(ops_per_graph):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    barrier()
    return start.elapsed_time(stop) / (replays * ops_per_graph)


def run_sweep(args, comm, nccl, rank, world, dev, stream, barrier, max_over_ranks):
    """Latency and bus bandwidth per message size, ours beside the NCCL
    backend (operator to operator: MEAN includes the reference's scale launch).
    Every point is timed eagerly (one host call per op, CUDA events around the
    loop); points up to 1 MiB are also timed as replayed CUDA graphs, which
    takes the host launch path out of the latency."""
    import torch
    from dragon_b200 import workloads
    hi = (1 << 30) if args.sweep == "full" else (256 << 20)
    factor = 2.0 * (world - 1) / world
    rows = []
    for dtype_name in ("f32", "f16"):
        esize = 4 if dtype_name == "f32" else 2
        for nbytes in workloads.sweep_sizes(1 << 10, hi):
            count = nbytes // esize
            nbuf = max(1, min(32, (256 << 20) // nbytes))
            base = make_message(rank, count, dtype_name, dev)
            bufs = [base.clone() for _ in range(nbuf)]
            iters = 200 if nbytes <= (1 << 20) else (40 if nbytes <= (64 << 20) else 10)
            ops = [comm.prepare_all_reduce([b], [b], "MEAN") for b in bufs]
            state = {"i": 0}

            def ours():
                ops[state["i"] % nbuf]()
                state["i"] += 1

            def theirs():
                b = bufs[state["i"] % nbuf]
                nccl.operator_all_reduce([b], "MEAN", torch.cuda.current_stream().cuda_stream)
                state["i"] += 1

            _, total = time_steps(ours, iters, 5, barrier)
            t_ours = max_over_ranks(total) / iters
            row = {"dtype": dtype_name, "bytes": nbytes, "ours_us": t_ours * 1e3,
                   "ours_busbw": nbytes / (t_ours * 1e-3) / 1e9 * factor,
                   "variant": comm.last_launch()["variant"]}
            if nccl is not None:
                _, total = time_steps(theirs, iters, 5, barrier)
                t_nccl = max_over_ranks(total) / iters
                row["nccl_us"] = t_nccl * 1e3
                row["nccl_busbw"] = nbytes / (t_nccl * 1e-3) / 1e9 * factor
                row["speedup"] = t_nccl / t_ours
            if nbytes <= (1 << 20):
                row["ours_graph_us"] = max_over_ranks(time_graph(ours, 20, 10, barrier)) * 1e3
                if nccl is not None:
                    row["nccl_graph_us"] = max_over_ranks(time_graph(theirs, 20, 10, barrier)) * 1e3
                    row["graph_speedup"] = row["nccl_graph_us"] / row["ours_graph_us"]
            row["frac_of_900"] = row["ours_busbw"] / NVLINK_NOMINAL_GBS
            rows.append(row)
            del bufs, ops, base
    return rows


# --------------------------------------------------------------------------
# reference arm: the CPU path on the host cores

def bench_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    import numpy as np
    from dragon_b200 import workloads
    from oracle import oracle
    n = max(1, args.gpus)
    nbytes = int(args.size_mib * MiB)   # the same message as the other arm
    count = nbytes // 4
    cores = os.cpu_count() or 1
    steps = max(2, min(args.steps, 6))  # each step is one whole all-reduce of that message on the host cores
    warm = min(args.warmup, 1)
    if n == 1:
        x = workloads.uniform_message(0, count)
        y = np.zeros_like(x)
        for _ in range(warm):
            oracle.allreduce([x], oracle.F32, args.reduction, out=y)
        times = []
        for _ in range(steps):
            t0 = time.perf_counter()
            oracle.allreduce([x], oracle.F32, args.reduction, out=y)
            times.append(time.perf_counter() - t0)
        t = statistics.median(times)
        value, used = x.nbytes / t / 1e9, 1
        what = "comm_size=1 out-of-place all-reduce (copy) on one core"
    else:
        bufs = [workloads.uniform_message(r, count) for r in range(n)]
        secs, out = oracle.mp_allreduce(bufs, oracle.F32, args.reduction, iters=steps + warm)
        t = statistics.median(secs[warm:])
        value, used = bufs[0].nbytes / t / 1e9 * 2.0 * (n - 1) / n, min(n, cores)
        what = "{} rank processes over shared memory, reduce-scatter + all-gather".format(n)
    sample = "{} timed all-reduces of {} MiB fp32 {} per rank ({}); Open MPI is not installed on this machine, so " \
             "the CPU restatement of the MPI path is timed".format(steps, nbytes // MiB, args.reduction, what)
    where = "out of place, comm_size=1 (local-copy path; value = algorithm GB/s S/t)" if n == 1 else \
        "in place, comm_size={}".format(n)
    return {
        "impl": "reference",
        "metric": METRIC,
        "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "Collective ALLREDUCE reduction={} f32 {:g} MiB per rank, {}".format(
                       args.reduction, args.size_mib, where),
                   "message_bytes": nbytes, "world_size": n, "timed_steps": steps,
                   "values": "uniform[-1,1) from numpy default_rng(1000+rank)"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": used, "kind": "port", "sample": sample,
                         "host_cores": cores},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


_RESULT_FD = None


def keep_stdout_for_the_result():
    """Libraries write to file descriptor 1 on their own (NCCL prints its version
    there when the comparison arm creates its communicator); the one JSON line
    must be alone on standard output, so everything else goes to standard error."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit_result(obj):
    data = (json.dumps(obj) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    args = parse_args()
    keep_stdout_for_the_result()
    if args.impl == "reference":
        line = bench_reference(args)
    elif args.emulated_only:
        line = {"emulated_ranks_one_gpu": bench_emulated(args)}
    elif args.gpus <= 1 and int(os.environ.get("WORLD_SIZE", "1")) <= 1:
        line = bench_single(args)
    else:
        line = bench_multi(args)
    if line is not None:
        emit_result(line)


if __name__ == "__main__":
    main()
