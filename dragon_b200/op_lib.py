"""Eager execution of operators of the C++ operator layer on torch tensors.

This plays the part of Dragon's ``OpLib.execute`` / ``Function.apply``
(dragon/python/core/autograph/op_lib.py:98-235,
torch/core/autograd/function.py:99-231): build an operator definition from
keyword arguments, bind inputs and outputs by name in a workspace and call
``Workspace::RunOperator`` in ``libdragon_collective.so``.  torch tensors are
fed as external memory; an output the operator has to create (``None`` in
``outputs``) is allocated by torch from the shape rule of the operation.
"""

import ctypes
import itertools
import os
import threading

import torch

from dragon_b200 import _C

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libdragon_collective.so")
_lib = None
_tls = threading.local()
_uid = itertools.count(1)

_DTYPE_NAMES = {
    torch.uint8: "uint8", torch.int8: "int8", torch.int32: "int32", torch.int64: "int64",
    torch.float16: "float16", torch.bfloat16: "bfloat16", torch.float32: "float32",
    torch.float64: "float64",
}


class OperatorError(RuntimeError):
    """A fatal error raised inside the operator layer (Dragon would abort)."""


def lib():
    global _lib
    if _lib is None:
        _C.lib()  # libdgn.so first: the operator library links against it
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError("{} is missing: build it with `python -m dragon_b200.build`".format(_LIB_PATH))
        h = ctypes.CDLL(_LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        h.dragon_last_error.restype = ctypes.c_char_p
        h.dragon_workspace_create.restype = ctypes.c_void_p
        h.dragon_workspace_destroy.argtypes = [ctypes.c_void_p]
        h.dragon_workspace_feed_external.argtypes = [
            ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64), ctypes.c_int,
            ctypes.c_char_p, ctypes.c_int, ctypes.c_int64]
        h.dragon_workspace_remove_tensor.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
        h.dragon_workspace_run_operator.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
        h.dragon_set_external_stream.argtypes = [ctypes.c_int, ctypes.c_void_p]
        h.dragon_operator_is_registered.argtypes = [ctypes.c_char_p]
        h.dragon_registry_rejects_duplicate.argtypes = [ctypes.c_char_p]
        h.dragon_schema_allows_inplace.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
        _lib = h
    return _lib


def _check(rc):
    if rc != 0:
        raise OperatorError(lib().dragon_last_error().decode("utf-8", "replace"))


def get_workspace():
    """The calling thread's workspace (one thread per workspace, as in Dragon)."""
    ws = getattr(_tls, "ws", None)
    if ws is None:
        ws = _tls.ws = ctypes.c_void_p(lib().dragon_workspace_create())
    return ws


def collective_args(**kwargs):
    """Argument getter of the `Collective` operator: names and defaults of
    dragon/python/core/autograph/op_args.py:98-108, plus `root`, which the
    reference's getter leaves out."""
    return {
        "operation": kwargs.get("operation", ""),
        "reduction": kwargs.get("reduction", "SUM"),
        "root": kwargs.get("root", 0),
        "bucket_size": kwargs.get("bucket_size", 0),
        "comm": kwargs.get("comm", 0),
        "group": kwargs.get("group", 0),
        "backend": kwargs.get("backend", "MPI"),
        "ranks": kwargs.get("ranks", None),
    }


def _def_text(op_type, in_names, out_names, device_index, args, cache_key=None, name=None):
    lines = ["type {}".format(op_type)]
    if name:
        lines.append("name {}".format(name))
    lines += ["input {}".format(n) for n in in_names]
    lines += ["output {}".format(n) for n in out_names]
    lines.append("device 1 {}".format(device_index))
    for key, value in args.items():
        if value is None:
            continue
        if isinstance(value, str):
            lines.append("arg_s {} {}".format(key, value))
        elif isinstance(value, (list, tuple)) and any(isinstance(v, float) for v in value):
            lines.append("arg_floats {} {}".format(key, " ".join(repr(float(v)) for v in value)))
        elif isinstance(value, (list, tuple)):
            lines.append("arg_ints {} {}".format(key, " ".join(str(int(v)) for v in value)))
        elif isinstance(value, float):
            lines.append("arg_f {} {}".format(key, repr(value)))
        else:
            lines.append("arg_i {} {}".format(key, int(value)))
    if cache_key:
        lines.append("arg_s cache_key {}".format(cache_key))  # must stay the last argument
    return "\n".join(lines).encode()


def _feed(ws, name, tensor):
    if not tensor.is_cuda:
        raise ValueError("the Collective operator of this library runs on CUDA tensors only")
    if not tensor.is_contiguous():
        raise ValueError("tensors must be contiguous")
    if tensor.dtype not in _DTYPE_NAMES:
        raise TypeError("Unsupported data type: {}".format(tensor.dtype))
    dims = (ctypes.c_int64 * max(tensor.dim(), 1))(*tensor.shape)
    _check(lib().dragon_workspace_feed_external(
        ws, name.encode(), ctypes.c_void_p(tensor.data_ptr()), dims, tensor.dim(),
        _DTYPE_NAMES[tensor.dtype].encode(), tensor.device.index, tensor.numel() * tensor.element_size()))


def _output_like(operation, x, group_size):
    """Shape rule of the operation (collective_op.cc:60-80)."""
    if operation == "ALLGATHER":
        return torch.empty((group_size,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    if operation == "REDUCESCATTER":
        if x.dim() == 0 or x.shape[0] % group_size != 0:
            raise ValueError("the first dimension must be divisible by the group size")
        return torch.empty((x.shape[0] // group_size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    return torch.empty_like(x)


def run_collective(inputs, outputs=None, group_size=0, stream=None, cache_key=None, **kwargs):
    """Runs the `Collective` operator eagerly.

    inputs: list of CUDA tensors.  outputs: None (fresh tensors), or a list
    whose entries are tensors (may be the inputs themselves: in place) or None.
    cache_key: reuse the operator instance created under that key (the
    workspace re-points it at the new tensors), as Dragon's eager mode does.
    Returns the list of output tensors.  Nothing is synchronised.
    """
    inputs = list(inputs)
    if not inputs:
        return []
    args = collective_args(**kwargs)
    device = inputs[0].device
    if outputs is None:
        outputs = [None] * len(inputs)
    outputs = list(outputs)
    if len(outputs) != len(inputs):
        raise ValueError("inputs and outputs differ in length")
    for i, out in enumerate(outputs):
        if out is None:
            outputs[i] = _output_like(args["operation"], inputs[i], group_size)
    ws = get_workspace()
    tag = next(_uid)
    in_names = ["collective/{}/in:{}".format(tag, i) for i in range(len(inputs))]
    out_names = []
    for i, (x, y) in enumerate(zip(inputs, outputs)):
        _feed(ws, in_names[i], x)
        if y.data_ptr() == x.data_ptr() and y.numel() == x.numel():
            out_names.append(in_names[i])  # in place: one tensor, as OperatorDef input == output
        else:
            name = "collective/{}/out:{}".format(tag, i)
            _feed(ws, name, y)
            out_names.append(name)
    cuda_stream = stream if stream is not None else torch.cuda.current_stream(device)
    handle = cuda_stream if isinstance(cuda_stream, int) else cuda_stream.cuda_stream
    lib().dragon_set_external_stream(device.index, ctypes.c_void_p(handle))
    try:
        _check(lib().dragon_workspace_run_operator(
            ws, _def_text("Collective", in_names, out_names, device.index, args, cache_key), 0, 0))
    finally:
        for name in set(in_names + out_names):
            lib().dragon_workspace_remove_tensor(ws, name.encode())
    return outputs


# ---- the ZeroAdamW operator -----------------------------------------------------------

_HYPER_KEYS = ("lr", "beta1", "beta2", "eps", "weight_decay", "grad_scale", "clip_norm", "clip_value")


def _feed_host_scalar(ws, name, value, keep):
    """A one-element float32 host tensor (device id -1), as the optimizers of
    the reference feed their hyper-parameters (torch/core/optim/zero.py:83-95)."""
    import numpy as np
    arr = np.array([value], dtype=np.float32)
    keep.append(arr)  # must outlive the run
    dims = (ctypes.c_int64 * 1)(1)
    _check(lib().dragon_workspace_feed_external(ws, name.encode(), ctypes.c_void_p(arr.ctypes.data), dims, 0,
                                                b"float32", -1, 4))


def run_zero_adamw(grads, params, hyper, name="ZeroAdamW", bucket_name="Bucket_1", lr_scales=None,
                   found_inf=None, stream=None, **group_args):
    """Runs the `ZeroAdamW` operator eagerly on one bucket, the way the
    reference's ZeroOptimizer._update_group does (torch/core/optim/zero.py:96-112):
    gradients are the inputs, the parameters (plus `found_inf`, if given) the
    outputs, the hyper-parameters travel as host tensors "<name>/<key>", and
    the operator instance is cached per (name, bucket) so that its step count
    and its state tensors "<name>/<bucket_name>/master|m|v" live on.

    hyper: dict with lr, beta1, beta2, eps, weight_decay, grad_scale,
    clip_norm, clip_value (plain values; grad_scale already divided by the
    group size).  group_args: comm, group, backend, ranks."""
    grads, params = list(grads), list(params)
    if len(grads) != len(params) or not params:
        raise ValueError("one gradient per parameter is required")
    device = params[0].device
    ws = get_workspace()
    tag = next(_uid)
    keep = []
    for key in _HYPER_KEYS:
        _feed_host_scalar(ws, "{}/{}".format(name, key), hyper[key], keep)
    in_names = ["zero/{}/grad:{}".format(tag, i) for i in range(len(grads))]
    out_names = ["zero/{}/param:{}".format(tag, i) for i in range(len(params))]
    for n, t in zip(in_names + out_names, grads + params):
        _feed(ws, n, t)
    if found_inf is not None:
        out_names.append("zero/{}/found_inf".format(tag))
        _feed(ws, out_names[-1], found_inf)
    scales = [float(x) for x in (lr_scales if lr_scales is not None else [1.0] * len(params))]
    args = {
        "bucket_name": bucket_name,
        "lr_scales": scales,
        "use_lr_scales": int(any(x != 1.0 for x in scales)),
        "comm": group_args.get("comm", 0),
        "group": group_args.get("group", 0),
        "backend": group_args.get("backend", "MPI"),
        "ranks": group_args.get("ranks", None),
    }
    cuda_stream = stream if stream is not None else torch.cuda.current_stream(device)
    handle = cuda_stream if isinstance(cuda_stream, int) else cuda_stream.cuda_stream
    lib().dragon_set_external_stream(device.index, ctypes.c_void_p(handle))
    try:
        _check(lib().dragon_workspace_run_operator(
            ws, _def_text("ZeroAdamW", in_names, out_names, device.index, args,
                          cache_key="{}/{}".format(name, bucket_name), name=name), 0, 0))
    finally:
        for n in set(in_names + out_names):
            lib().dragon_workspace_remove_tensor(ws, n.encode())


def run_sync_bn_stats(stats, batch_size, count_on_device=False, stream=None, **group_args):
    """Runs the `SyncBNStats` operator eagerly: the statistics exchange of
    synchronized batch normalization (normalization/batch_norm_op.cc:29-43).

    stats: float32 CUDA tensor of 2C partial sums (sum and sum of squares per
    channel), reduced in place; with count_on_device it holds 2C + 1 values and
    this function writes float(batch_size) into the last one first, so that the
    global count arrives with the statistics and nothing blocks.  Otherwise the
    count goes through the blocking host all-reduce, as in the reference, and
    is returned.  group_args: comm, group, backend, ranks."""
    import numpy as np
    device = stats.device
    ws = get_workspace()
    tag = next(_uid)
    name = "syncbn/{}/stats".format(tag)
    _feed(ws, name, stats)
    out_names = [name]
    total = np.zeros(1, dtype=np.int64)
    if count_on_device:
        stats[-1] = float(batch_size)
    else:
        out_names.append("syncbn/{}/count".format(tag))
        dims = (ctypes.c_int64 * 1)(1)
        _check(lib().dragon_workspace_feed_external(ws, out_names[1].encode(), ctypes.c_void_p(total.ctypes.data), dims,
                                                    1, b"int64", -1, 8))
    args = {
        "batch_size": int(batch_size),
        "count_on_device": int(bool(count_on_device)),
        "comm": group_args.get("comm", 0),
        "group": group_args.get("group", 0),
        "backend": group_args.get("backend", "MPI"),
        "ranks": group_args.get("ranks", None),
    }
    cuda_stream = stream if stream is not None else torch.cuda.current_stream(device)
    handle = cuda_stream if isinstance(cuda_stream, int) else cuda_stream.cuda_stream
    lib().dragon_set_external_stream(device.index, ctypes.c_void_p(handle))
    try:
        _check(lib().dragon_workspace_run_operator(ws, _def_text("SyncBNStats", [name], out_names, device.index, args), 0, 0))
    finally:
        for n in out_names:
            lib().dragon_workspace_remove_tensor(ws, n.encode())
    return None if count_on_device else int(total[0])


class _DevicePointer(object):
    def __init__(self, ptr, count):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def zero_state(name, bucket_name, key, device):
    """A copy of the operator's fp32 state tensor "<name>/<bucket_name>/<key>"
    (master, m or v) in this thread's workspace."""
    dims = (ctypes.c_int64 * 8)()
    ndim, ptr = ctypes.c_int(), ctypes.c_void_p()
    dtype = ctypes.create_string_buffer(16)
    h = lib()
    h.dragon_workspace_tensor_info.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_int64),
                                               ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_char_p,
                                               ctypes.c_int, ctypes.POINTER(ctypes.c_void_p)]
    _check(h.dragon_workspace_tensor_info(get_workspace(), "{}/{}/{}".format(name, bucket_name, key).encode(),
                                          dims, 8, ctypes.byref(ndim), dtype, 16, ctypes.byref(ptr)))
    return torch.as_tensor(_DevicePointer(ptr.value, int(dims[0])), device=device).clone()
