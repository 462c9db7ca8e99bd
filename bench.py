#!/usr/bin/env python
"""Benchmark of the `Collective` hot path: all-reduce bus bandwidth and latency.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference --gpus N ...      (CPU path, rank 0 only)

One step = one ALLREDUCE (MEAN, fp32, 256 MiB per rank by default) through the
dgn C-ABI.  At N = 1 the communicator has one rank and the step is the
out-of-place local-copy path (HBM bound); at N >= 2 it is the peer-memory
all-reduce over NVLink and `value` is the bus bandwidth
S/t * 2(N-1)/N.  Rank 0 prints one JSON line.
"""

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MiB = 1 << 20
NVLINK_NOMINAL_GBS = 900.0      # per direction per GPU
NVLINK_MEASURED_P2P_GBS = 770.0  # peer copy measured on this pool
HBM_FALLBACK_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size-mib", type=float, default=256.0, help="message bytes per rank of the timed step")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f16", "bf16"])
    ap.add_argument("--reduction", default="MEAN")
    ap.add_argument("--sweep", default="auto", choices=["auto", "off", "full"],
                    help="message-size sweep beside the headline (auto: up to 256 MiB)")
    ap.add_argument("--configs", default="auto", choices=["auto", "off", "zero"],
                    help="operator configurations (gradient buckets, gather/broadcast shapes) beside the headline")
    ap.add_argument("--no-nccl", action="store_true", help="skip the NCCL comparison in the sweep")
    ap.add_argument("--no-symm", action="store_true", help="N>=2: skip the symmetric-memory (in-place multicast) rows")
    ap.add_argument("--tune", default="off", choices=["off", "symm", "pipe", "bcast", "all"],
                    help="N>=2: instead of the benchmark, time the multicast kernels over launch shapes, chunk "
                         "sizes and variants and print one JSON object of rows (input for the thresholds)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-emulated", action="store_true", help="N=1: skip the emulated 8-rank timings")
    ap.add_argument("--emulated-only", action="store_true",
                    help="N=1: run only the emulated multi-rank kernels (profiling target)")
    return ap.parse_args()


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
    return {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[name]


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
        e2e_ms = time_e2e(comm, xh, yh, [x, torch.empty_like(x)], [y, torch.empty_like(y)], args.reduction,
                          e2e_steps, 2)
    assert torch.equal(yh, xh), "local-copy path returned different bytes"
    ms = total_ms / args.steps
    kernel_ms = statistics.mean(per)
    peak, peak_kind = hbm_peak()
    achieved = 2.0 * S / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": "allreduce bus GB/s & latency vs msg size (frac of 900 GB/s at 2/4/8 GPUs; "
                  "at 1 GPU: local-copy path, algorithm GB/s = S/t)",
        "value": S / (ms * 1e-3) / 1e9,
        "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic",
        "config": {
            "workload": "Collective ALLREDUCE reduction={} {} {:g} MiB per rank, out of place, comm_size=1 "
                        "(local-copy path)".format(args.reduction, args.dtype, args.size_mib),
            "message_bytes": S, "world_size": 1,
            "l2": "message ({:g} MiB) larger than the 126 MB L2; no flush between steps".format(args.size_mib),
            "values": "uniform[-1,1) from numpy default_rng(1000+rank)",
        },
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "peak_kind": peak_kind,
                     "algorithmic_bytes_per_launch": 2 * S, "kernel": "local_copy_kernel",
                     "kernel_ms": kernel_ms},
        "e2e": {"value": S / (e2e_ms / e2e_steps * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": S, "d2h_bytes_per_step": S, "ms_per_step": e2e_ms / e2e_steps,
                "pipeline": "H2D, all-reduce and D2H on three streams, two device buffers"},
        "gpu_launches": int(launches),
        "clocks": sampler.summary(),
    }
    # DRAM traffic of the copy kernel from its ncu capture (profiles/local_copy_kernel_256MiB.md):
    # 268.5 MB read + 221.7 MB written per 256 MiB message; the rest of the
    # written lines is still in the 126 MB L2 when the kernel ends.  Traffic
    # grows with the vectors copied, so it is scaled by the message size.
    line["roofline"]["traffic"] = (268.46e6 + 221.73e6) * (S / float(256 * MiB))
    if not args.no_emulated:
        line["emulated_ranks_one_gpu"] = bench_emulated(args)
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_local_copy_baseline(args)
        line["cpu_baseline_config1"] = cpu_config1_baseline()
    comm.destroy()
    return line


def bench_emulated(args):
    """The multi-rank kernels with 8 virtual ranks on this one GPU (all "peer"
    traffic is local HBM traffic): times the two-shot and one-shot kernels the
    multi-GPU runs use."""
    import torch
    from dragon_b200.comm import Communicator
    out = {}
    comms = Communicator.emulated(8, 0)
    try:
        for label, nbytes in (("lowlatency_64KiB", 64 << 10), ("twoshot_64MiB", 64 << 20)):
            count = nbytes // 4
            xs = [make_message(r, count, "f32", "cuda:0") for r in range(8)]
            ops = [c.prepare_all_reduce([x], [x], "MEAN") for c, x in zip(comms, xs)]

            def step():
                for op in ops:
                    op()

            per, total = time_steps(step, 10, 3)
            out[label] = {"ms_per_allreduce": total / 10, "launch": comms[0].last_launch()}
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
        out["zero_adamw_64MiB_fp16"] = {"ms_per_step": total / 10, "launch": comms[0].last_launch(),
                                        "found_inf": float(found[0].item())}
        del opts
    finally:
        torch.cuda.synchronize()
        for c in comms:
            c.destroy()
    return out


def cpu_local_copy_baseline(args):
    """The oracle's comm_size-1 out-of-place path on one host core, on a
    bounded sample of the message."""
    import numpy as np
    from dragon_b200 import workloads
    from oracle import oracle
    count = min(int(args.size_mib * MiB) // 4, 16 * MiB)  # 64 MiB fp32 sample
    x = workloads.uniform_message(0, count)
    y = np.zeros_like(x)
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or time.perf_counter() - t0 < 3.0:
        oracle.allreduce([x], oracle.F32, "MEAN", out=y)
        reps += 1
    t = (time.perf_counter() - t0) / reps
    assert np.array_equal(x, y)
    return {"value": x.nbytes / t / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": "{} passes of the oracle's comm_size=1 all-reduce over a {} MiB fp32 sample".format(
                reps, x.nbytes // MiB), "host_cores": os.cpu_count()}


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
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group(backend="gloo")  # plumbing only: handle exchange, barriers, max over ranks

    def barrier():
        dist.barrier()

    def max_over_ranks(v):
        t = torch.tensor([float(v)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
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

    # Parity spot check of the headline message before timing (fp64 host sum of
    # a slice; the full parity suite lives in tests/).
    op()
    torch.cuda.synchronize()
    check = x[:4096].double().cpu()
    parts = [None] * world
    dist.all_gather_object(parts, x0[:4096].double().cpu())
    ref = sum(parts) / (world if args.reduction.upper() == "MEAN" else 1)
    tol = {"f32": 1e-6, "f16": 2e-3, "bf16": 1e-2}[args.dtype]
    err = float((check - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
    assert err <= tol, "headline all-reduce off by {} (tolerance {})".format(err, tol)
    x.copy_(x0)

    sampler = ClockSampler(local)
    with sampler:
        launches0 = lib.dgn_launch_count()
        per, total_ms = time_steps(op, args.steps, args.warmup, barrier)
        launches = lib.dgn_launch_count() - launches0 - args.warmup
        xh = x0.cpu().pin_memory()
        yh = torch.empty_like(xh).pin_memory()
        e2e_steps = max(3, min(args.steps, 10))
        x2 = torch.empty_like(x)
        e2e_ms = time_e2e(comm, xh, yh, [x, x2], [x, x2], args.reduction, e2e_steps, 2, barrier)
        del x2
    ms = max_over_ranks(total_ms) / args.steps
    kernel_ms = max_over_ranks(statistics.mean(per))
    e2e_ms = max_over_ranks(e2e_ms) / e2e_steps
    launch = comm.last_launch()
    busbw = S / (ms * 1e-3) / 1e9 * factor

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
        line = {
            "metric": "allreduce bus GB/s & latency vs msg size at 2/4/8 B200 (frac of 900 GB/s)",
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
                "launch": launch,
            },
            "roofline": {"bound": "nvlink", "achieved": achieved, "peak": NVLINK_NOMINAL_GBS, "unit": "GB/s",
                         "frac": achieved / NVLINK_NOMINAL_GBS, "traffic": None,
                         "peak_kind": "nominal per direction per GPU; measured peer copy on this pool is "
                                      "{:g} GB/s".format(NVLINK_MEASURED_P2P_GBS),
                         "frac_of_measured_p2p": achieved / NVLINK_MEASURED_P2P_GBS,
                         "algorithmic_bytes_per_launch": S * factor, "kernel_ms": kernel_ms},
            "e2e": {"value": S / (e2e_ms * 1e-3) / 1e9 * factor, "unit": "GB/s",
                    "h2d_bytes_per_step": S, "d2h_bytes_per_step": S, "ms_per_step": e2e_ms,
                    "pipeline": "H2D, all-reduce and D2H on three streams, two device buffers"},
            "gpu_launches": int(launches),
            "clocks": sampler.summary(),
            "sweep": sweep,
            "operator_configs": extras,
            "nvls": comm.has_nvls(),
            "symmetric_memory": symmetric,
        }
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
    row = {"tensors": len(grads), "bytes": nbytes, "ours_us": timed(op) * 1e3}
    if nccl is not None:
        scratch = torch.empty(nbytes // 4, device=dev)
        row["nccl_us"] = timed(lambda: nccl.operator_all_reduce(grads, "MEAN", stream_of(), bucket=scratch)) * 1e3
        row["nccl_unbucketed_us"] = timed(lambda: nccl.operator_all_reduce(grads, "MEAN", stream_of())) * 1e3
        row["speedup"] = row["nccl_us"] / row["ours_us"]
        del scratch
    row["ours_busbw"] = nbytes / (row["ours_us"] * 1e-6) / 1e9 * 2.0 * (world - 1) / world
    out["resnet50_fp32_one_bucket_mean"] = row
    del grads, op

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
        t_bc = timed(lambda: comm.broadcast(x, 0), iters)
        row = {"shard_bytes": sbytes, "allgather_us": t_ag * 1e3,
               "allgather_busbw": world * sbytes / t_ag / 1e6 * (world - 1) / world,
               "broadcast_us": t_bc * 1e3, "broadcast_busbw": sbytes / t_bc / 1e6}
        if nccl is not None:
            row["nccl_allgather_us"] = timed(lambda: nccl.all_gather(x, y, stream_of()), iters) * 1e3
            row["nccl_broadcast_us"] = timed(lambda: nccl.broadcast(x, 0, stream_of()), iters) * 1e3
        out[label] = row
        del x, y
    return out


def run_tuning(args):
    """Times the NVSwitch-multicast kernels beside the other variants over the
    knobs that set their defaults: blocks and threads of the in-place kernel on
    symmetric memory; chunk size and switch blocks of the pipelined variant
    against the automatic choice, the two-shot and the staged kernel; blocks of
    the broadcast through the switch against the automatic choice."""
    import torch
    import torch.distributed as dist
    from dragon_b200.comm import Communicator

    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group(backend="gloo")
    comm = Communicator.init_local(rank, world, local, symm_bytes=256 * MiB)
    handles = [None] * world
    dist.all_gather_object(handles, comm.handle_bytes())
    comm.connect(handles)
    dist.barrier()

    def max_over_ranks(v):
        t = torch.tensor([float(v)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, iters):
        _, total = time_steps(fn, iters, 3, dist.barrier)
        return max_over_ranks(total) / iters * 1e3  # us

    factor = 2.0 * (world - 1) / world
    rows = []
    what = args.tune
    if not comm.has_nvls():
        rows.append({"error": "NVSwitch multicast is not available on this box"})
        what = "none"
    if what in ("symm", "all"):
        arena = comm.symm_empty(64 * MiB, torch.float32)
        arena.uniform_(-1, 1)
        for mib in (4, 16, 64, 256):
            count = mib * MiB // 4
            nbuf = max(1, 256 // mib)
            views = [arena[k * count:(k + 1) * count] for k in range(nbuf)]
            for blocks in (16, 32, 64, 100, 148):
                for threads in (128, 256, 512):
                    comm.set_tuning(variant=6, blocks=blocks, threads=threads)
                    ops = [comm.prepare_all_reduce([v], [v], "MEAN") for v in views]
                    state = {"i": 0}

                    def step():
                        ops[state["i"] % nbuf]()
                        state["i"] += 1

                    us = timed(step, 20)
                    rows.append({"kernel": "symm", "mib": mib, "blocks": blocks, "threads": threads, "us": us,
                                 "busbw": mib * MiB / us / 1e3 * factor})
        del arena
        comm.symm_reset()
    if what in ("pipe", "all"):
        for mib in (8, 16, 64, 256, 1024):
            x = torch.empty(mib * MiB // 4, device="cuda").uniform_(-1, 1)
            shapes = [(0, 0, 0), (2, 0, 0), (3, 0, 0), (7, 0, 0)]
            shapes += [(7, c * MiB, b) for c in (4, 16, 32, 64) if c * 2 <= mib for b in (16, 32, 64)]
            for variant, chunk, blocks in shapes:
                comm.set_tuning(variant=variant, chunk_bytes=chunk, blocks=blocks)
                op = comm.prepare_all_reduce([x], [x], "MEAN")
                us = timed(op, 10)
                rows.append({"kernel": "pipe", "mib": mib, "variant": variant, "chunk_mib": chunk // MiB,
                             "switch_blocks": blocks, "us": us, "busbw": mib * MiB / us / 1e3 * factor,
                             "launch": comm.last_launch()})
            del x
    if what in ("bcast", "all"):
        for mib in (1, 4, 16, 64, 256):
            x = torch.empty(mib * MiB // 4, device="cuda").uniform_(-1, 1)
            for variant, blocks, threads in ((0, 0, 0), (1, 0, 0), (2, 0, 0), (3, 0, 0), (3, 32, 0), (3, 148, 0),
                                             (3, 64, 256)):
                comm.set_tuning(variant=variant, blocks=blocks, threads=threads)
                us = timed(lambda: comm.broadcast(x, 0), 10)
                rows.append({"kernel": "bcast", "mib": mib, "variant": variant, "blocks": blocks, "threads": threads,
                             "us": us, "gbs": mib * MiB / us / 1e3, "launch": comm.last_launch()})
            del x
    comm.set_tuning()
    dist.barrier()
    torch.cuda.synchronize()
    comm.destroy()
    dist.destroy_process_group()
    return {"tuning": args.tune, "n_gpus": world, "rows": rows} if rank == 0 else None


def run_symmetric(comm, rank, world, barrier, max_over_ranks):
    """MEAN all-reduce in place on buffers from the communicator's symmetric
    arena (dgn_comm_symm_alloc): the switch reduces the buffers themselves,
    nothing is staged.  Each size rotates over views that cover 256 MiB."""
    import torch
    if not comm.has_nvls() or comm.symm_capacity() < 256 * MiB:
        return {"available": False}
    factor = 2.0 * (world - 1) / world
    rows = []
    for dtype_name, sizes in (("f32", (1, 4, 16, 64, 128, 256)), ("f16", (64, 256))):
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
    sample_bytes = min(int(args.size_mib * MiB), 64 * MiB)
    count = sample_bytes // 4
    cores = os.cpu_count() or 1
    if n == 1:
        x = workloads.uniform_message(0, count)
        y = np.zeros_like(x)
        for _ in range(min(args.warmup, 2)):
            oracle.allreduce([x], oracle.F32, args.reduction, out=y)
        times = []
        for _ in range(min(args.steps, 10)):
            t0 = time.perf_counter()
            oracle.allreduce([x], oracle.F32, args.reduction, out=y)
            times.append(time.perf_counter() - t0)
        t = statistics.median(times)
        value, used = x.nbytes / t / 1e9, 1
        what = "comm_size=1 out-of-place all-reduce (copy) on one core"
    else:
        bufs = [workloads.uniform_message(r, count) for r in range(n)]
        iters = max(2, min(args.steps, 10))
        secs, out = oracle.mp_allreduce(bufs, oracle.F32, args.reduction, iters=iters + min(args.warmup, 2))
        t = statistics.median(secs[min(args.warmup, 2):])
        value, used = bufs[0].nbytes / t / 1e9 * 2.0 * (n - 1) / n, min(n, cores)
        what = "{} rank processes over shared memory, reduce-scatter + all-gather".format(n)
    sample = "{} MiB fp32 {} per rank ({}); Open MPI is not installed on this machine, so the CPU " \
             "restatement of the MPI path is timed".format(sample_bytes // MiB, args.reduction, what)
    return {
        "impl": "reference",
        "metric": "allreduce bus GB/s & latency vs msg size at 2/4/8 B200 (frac of 900 GB/s)"
                  if n > 1 else "allreduce bus GB/s & latency vs msg size (frac of 900 GB/s at 2/4/8 GPUs; "
                                "at 1 GPU: local-copy path, algorithm GB/s = S/t)",
        "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "Collective ALLREDUCE reduction={} f32, CPU path, comm_size={}".format(args.reduction, n),
                   "message_bytes": sample_bytes, "world_size": n},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": used, "kind": "port", "sample": sample,
                         "host_cores": cores},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    args = parse_args()
    if args.impl == "reference":
        line = bench_reference(args)
    elif args.emulated_only:
        line = {"emulated_ranks_one_gpu": bench_emulated(args)}
    elif args.gpus <= 1 and int(os.environ.get("WORLD_SIZE", "1")) <= 1:
        line = bench_single(args)
    elif args.tune != "off":
        line = run_tuning(args)
    else:
        line = bench_multi(args)
    if line is not None:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
