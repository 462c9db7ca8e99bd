"""In-tree build of the native libraries (nvcc, sm_100a only).

``python -m dragon_b200.build`` produces

* ``dragon_b200/lib/libdgn.so``      -- the C-ABI collective library (include/dgn.h)
* ``dragon_b200/lib/libdragon_collective.so`` -- the C++ operator layer over it
  (built when its sources are present)

Objects are rebuilt only when a source or header is newer.  nvcc cross-compiles
without a GPU, so this runs on any machine with the CUDA toolkit.
"""

import concurrent.futures
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(ROOT)
CSRC = os.path.join(ROOT, "csrc")
LIB = os.path.join(ROOT, "lib")
OBJ = os.path.join(ROOT, "build")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall"]


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the dgn library cannot be built")
    return nvcc


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: {}\n{}".format(" ".join(cmd), proc.stdout))
    return proc.stdout


def _headers():
    hdrs = [os.path.join(REPO, "include", "dgn.h")]
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cuh", ".h")):
            hdrs.append(os.path.join(CSRC, name))
    return hdrs


def build(verbose=False, extra_flags=()):
    """Build everything that is out of date; returns the path of libdgn.so."""
    nvcc = _nvcc()
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    hdrs = _headers()
    jobs = []  # (object, command)
    inst_src = os.path.join(CSRC, "dgn_kernels_inst.cu")
    for inst in range(9):
        obj = os.path.join(OBJ, "dgn_kernels_inst_{}.o".format(inst))
        cmd = [nvcc] + NVCC_FLAGS + list(extra_flags) + ["-DDGN_INST={}".format(inst), "-c", inst_src, "-o", obj]
        jobs.append((obj, cmd, [inst_src] + hdrs))
    for name in sorted(os.listdir(CSRC)):
        if name.endswith(".cu") and name != "dgn_kernels_inst.cu":
            src = os.path.join(CSRC, name)
            obj = os.path.join(OBJ, name[:-3] + ".o")
            cmd = [nvcc] + NVCC_FLAGS + list(extra_flags) + ["-c", src, "-o", obj]
            jobs.append((obj, cmd, [src] + hdrs))
    stale = [(o, c) for o, c, deps in jobs if _newer(o, deps)]
    if stale:
        workers = min(len(stale), os.cpu_count() or 4)
        with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
            for out in pool.map(lambda oc: _run(oc[1]), stale):
                if verbose and out.strip():
                    print(out)
    objs = [o for o, _, _ in jobs]
    lib = os.path.join(LIB, "libdgn.so")
    if _newer(lib, objs):
        _run([nvcc] + ARCH + ["-shared", "-o", lib] + objs + ["-Xlinker", "--no-undefined"])

    # The C++ operator layer (host code; nvcc drives g++ and links the CUDA
    # runtime) links against libdgn.
    op_dir = os.path.join(ROOT, "operators")
    if os.path.isdir(op_dir):
        srcs = [os.path.join(op_dir, f) for f in sorted(os.listdir(op_dir)) if f.endswith(".cc")]
        op_hdrs = [os.path.join(op_dir, f) for f in sorted(os.listdir(op_dir)) if f.endswith(".h")]
        op_lib = os.path.join(LIB, "libdragon_collective.so")
        if srcs and _newer(op_lib, srcs + op_hdrs + [lib] + hdrs):
            _run([nvcc, "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-shared", "-o", op_lib]
                 + srcs + ["-I", os.path.join(REPO, "include"), "-I", op_dir, "-L", LIB, "-ldgn",
                           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN", "-Xlinker", "--no-undefined"])
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
