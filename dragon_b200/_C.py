"""ctypes binding of the dgn C-ABI (include/dgn.h).

The shared library is the only compute path: if it is missing this module
raises, there is no fallback.
"""

import ctypes
import os

_LIB_PATH = os.environ.get("DGN_LIBRARY") or os.path.join(
    os.path.dirname(os.path.abspath(__file__)), "lib", "libdgn.so")

HANDLE_BYTES = 256
MAX_RANKS = 8

OK, ERR_ARG, ERR_CUDA, ERR_TIMEOUT, ERR_PEER, ERR_STATE, ERR_UNSUPPORTED = range(7)

U8, I8, I32, I64, F16, BF16, F32, F64 = range(8)
SUM, MEAN, PROD, MIN, MAX = range(5)
(VARIANT_AUTO, VARIANT_ONESHOT, VARIANT_TWOSHOT, VARIANT_NVLS, VARIANT_LL, VARIANT_LL2, VARIANT_SYMM,
 VARIANT_RING, VARIANT_RING_PULL) = range(9)

REDOPS = {"SUM": SUM, "MEAN": MEAN, "PROD": PROD, "MIN": MIN, "MAX": MAX}

# Every symbol include/dgn.h declares: name -> (restype, argtypes).
_c_void_pp = ctypes.POINTER(ctypes.c_void_p)
_c_i64_p = ctypes.POINTER(ctypes.c_int64)
_c_int_p = ctypes.POINTER(ctypes.c_int)
SIGNATURES = {
    "dgn_version": (ctypes.c_int, []),
    "dgn_dtype_size": (ctypes.c_size_t, [ctypes.c_int]),
    "dgn_last_error_string": (ctypes.c_char_p, []),
    "dgn_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "dgn_comm_init_local": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, _c_void_pp]),
    "dgn_comm_get_handle": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "dgn_comm_connect": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "dgn_comm_create": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_char_p,
                                       ctypes.c_char_p, ctypes.c_int, _c_void_pp]),
    "dgn_comm_create_emulated": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _c_void_pp]),
    "dgn_comm_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "dgn_comm_rank": (ctypes.c_int, [ctypes.c_void_p]),
    "dgn_comm_size": (ctypes.c_int, [ctypes.c_void_p]),
    "dgn_comm_device": (ctypes.c_int, [ctypes.c_void_p]),
    "dgn_comm_status": (ctypes.c_int, [ctypes.c_void_p]),
    "dgn_comm_set_wait_limit_ms": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int]),
    "dgn_comm_set_tuning": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                           ctypes.c_int64]),
    "dgn_comm_set_knob": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int64]),
    "dgn_comm_has_nvls": (ctypes.c_int, [ctypes.c_void_p]),
    "dgn_allreduce": (ctypes.c_int, [ctypes.c_void_p, _c_void_pp, _c_void_pp, _c_i64_p, ctypes.c_int,
                                     ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "dgn_allgather": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                     ctypes.c_int, ctypes.c_void_p]),
    "dgn_broadcast": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                     ctypes.c_int, ctypes.c_void_p]),
    "dgn_reducescatter": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                         ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "dgn_allreduce_host": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                          ctypes.c_int, ctypes.c_int]),
    "dgn_allreduce_static": (ctypes.c_int, [ctypes.c_int, _c_void_pp, _c_void_pp, ctypes.c_int64, ctypes.c_int,
                                            ctypes.c_int, ctypes.c_void_p]),
    "dgn_allreduce_static_status": (ctypes.c_int, [ctypes.c_int]),
    "dgn_launch_count": (ctypes.c_int64, []),
    "dgn_comm_last_launch": (ctypes.c_int, [ctypes.c_void_p, _c_int_p, _c_int_p, _c_int_p, _c_i64_p,
                                            _c_int_p]),
}



class AdamWArgs(ctypes.Structure):
    """dgn_adamw_args of include/dgn.h."""
    _fields_ = [("lr", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float),
                ("eps", ctypes.c_float), ("weight_decay", ctypes.c_float), ("grad_scale", ctypes.c_float),
                ("clip_norm", ctypes.c_float), ("clip_value", ctypes.c_float)]


class UpdateArgs(ctypes.Structure):
    """dgn_update_args of include/dgn.h."""
    _fields_ = [("kind", ctypes.c_int), ("lr", ctypes.c_float), ("momentum", ctypes.c_float),
                ("beta1", ctypes.c_float), ("beta2", ctypes.c_float), ("eps", ctypes.c_float),
                ("weight_decay", ctypes.c_float), ("grad_scale", ctypes.c_float), ("clip_value", ctypes.c_float)]


UPDATE_MOMENTUM_SGD, UPDATE_NESTEROV_SGD, UPDATE_ADAM, UPDATE_ADAMW = range(4)


class StagedPlan(ctypes.Structure):
    """dgn_staged_plan of include/dgn.h."""
    _fields_ = [("variant", ctypes.c_int), ("blocks", ctypes.c_int), ("threads", ctypes.c_int), ("chunks", ctypes.c_int),
                ("chunk_vectors", ctypes.c_int64), ("staged", ctypes.c_int), ("depth", ctypes.c_int),
                ("first_role_blocks", ctypes.c_int), ("second_role_blocks", ctypes.c_int), ("mode", ctypes.c_int),
                ("ring_bytes_needed", ctypes.c_int64), ("ring_bytes_available", ctypes.c_int64),
                ("inbox_bytes_needed", ctypes.c_int64), ("inbox_bytes_available", ctypes.c_int64),
                ("inbox_offset_in_half", ctypes.c_int64)]


SIGNATURES.update({
    "dgn_allreduce_update": (ctypes.c_int, [ctypes.c_void_p, _c_void_pp, _c_void_pp, _c_void_pp, _c_void_pp, _c_i64_p,
                                            ctypes.c_int, ctypes.c_int, ctypes.POINTER(UpdateArgs), ctypes.c_void_p]),
    "dgn_comm_init_symmetric": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int64, _c_void_pp]),
    "dgn_comm_symm_capacity": (ctypes.c_int64, [ctypes.c_void_p]),
    "dgn_comm_symm_alloc": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, _c_void_pp]),
    "dgn_comm_symm_reset": (ctypes.c_int, [ctypes.c_void_p]),
    "dgn_plan_query": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int,
                                      _c_int_p, _c_int_p, _c_int_p, _c_i64_p, _c_int_p]),
    "dgn_plan_query_staged": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int64,
                                             ctypes.POINTER(StagedPlan)]),
    "dgn_zero_shard_count": (ctypes.c_int64, [ctypes.c_int, ctypes.c_int64]),
    "dgn_zero_state_count": (ctypes.c_int64, [ctypes.c_int, ctypes.c_int64, ctypes.c_int]),
    "dgn_zero_state_offset": (ctypes.c_int64, [ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int]),
    "dgn_zero_init_master": (ctypes.c_int, [ctypes.c_void_p, _c_void_pp, _c_i64_p, ctypes.c_int, ctypes.c_int,
                                            ctypes.c_void_p, ctypes.c_void_p]),
    "dgn_zero_adamw": (ctypes.c_int, [ctypes.c_void_p, _c_void_pp, _c_void_pp, _c_i64_p, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                      ctypes.c_void_p, ctypes.POINTER(ctypes.c_float),
                                      ctypes.POINTER(AdamWArgs), ctypes.c_void_p, ctypes.c_void_p]),
})

_lib = None


class DgnError(RuntimeError):
    """A dgn entry point returned a non-OK status."""

    def __init__(self, status, message):
        super().__init__("dgn status {} ({}): {}".format(status, _status_name(status), message))
        self.status = status


def _status_name(status):
    names = ["OK", "ERR_ARG", "ERR_CUDA", "ERR_TIMEOUT", "ERR_PEER", "ERR_STATE", "ERR_UNSUPPORTED"]
    return names[status] if 0 <= status < len(names) else "?"


def lib_path():
    return _LIB_PATH


def lib():
    """Load libdgn.so once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                "{} is missing: build it with `python -m dragon_b200.build` "
                "(there is no fallback path)".format(_LIB_PATH))
        handle = ctypes.CDLL(_LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status):
    if status != OK:
        raise DgnError(status, lib().dgn_last_error_string().decode("utf-8", "replace"))
