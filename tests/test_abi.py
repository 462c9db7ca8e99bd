"""The C-ABI library loads without a GPU and exports exactly what
include/dgn.h declares; the ctypes binding covers every declared symbol."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dgn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dgn_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ("dgn_comm_init_local", "dgn_comm_get_handle", "dgn_comm_connect", "dgn_comm_create",
                 "dgn_comm_create_emulated", "dgn_comm_destroy", "dgn_allreduce", "dgn_allgather",
                 "dgn_broadcast", "dgn_reducescatter", "dgn_comm_status", "dgn_allreduce_static"):
        assert must in names


def test_library_exports_every_declared_symbol(dgn_lib):
    for name in declared_symbols():
        assert hasattr(dgn_lib, name), "libdgn.so does not export {}".format(name)


def test_binding_covers_every_declared_symbol():
    from dragon_b200 import _C
    assert sorted(_C.SIGNATURES) == declared_symbols()


def test_entry_points_without_a_device(dgn_lib):
    """Calls that need no GPU: version, dtype sizes, status strings, argument checks."""
    from dragon_b200 import _C
    assert dgn_lib.dgn_version() >= 100
    assert [dgn_lib.dgn_dtype_size(t) for t in range(8)] == [1, 1, 4, 8, 2, 2, 4, 8]
    assert dgn_lib.dgn_dtype_size(99) == 0
    assert dgn_lib.dgn_status_string(_C.ERR_TIMEOUT) == b"timed out waiting for a peer"
    comm = ctypes.c_void_p()
    assert dgn_lib.dgn_comm_init_local(0, 9, 0, ctypes.byref(comm)) == _C.ERR_ARG
    assert b"nranks" in dgn_lib.dgn_last_error_string()
    assert dgn_lib.dgn_comm_init_local(3, 2, 0, ctypes.byref(comm)) == _C.ERR_ARG
    assert dgn_lib.dgn_allreduce(None, None, None, None, 0, 0, 0, None) == _C.ERR_ARG
    assert dgn_lib.dgn_comm_status(None) == _C.ERR_ARG
    assert dgn_lib.dgn_comm_rank(None) == -1 and dgn_lib.dgn_comm_size(None) == 0
    assert dgn_lib.dgn_comm_set_knob(None, b"gather_mode", 1) == _C.ERR_ARG
    assert dgn_lib.dgn_comm_set_tuning(None, 0, 0, 0, 0) == _C.ERR_ARG
    assert dgn_lib.dgn_comm_has_nvls(None) == 0


def test_missing_library_is_an_error(monkeypatch):
    from dragon_b200 import _C
    monkeypatch.setattr(_C, "_lib", None)
    monkeypatch.setattr(_C, "_LIB_PATH", "/nonexistent/libdgn.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _C.lib()


def test_operator_layer_registry(dgn_lib):
    """`Collective` is registered for CUDA once; a second registration is
    refused, as Dragon's registry refuses duplicates; in place is allowed."""
    from dragon_b200 import op_lib
    lib = op_lib.lib()
    assert lib.dragon_operator_is_registered(b"Collective") == 1
    assert lib.dragon_operator_is_registered(b"Conv2d") == 0
    assert lib.dragon_registry_rejects_duplicate(b"Collective") == 1
    assert lib.dragon_schema_allows_inplace(b"Collective", 0, 0) == 1
    assert lib.dragon_schema_allows_inplace(b"Collective", 3, 3) == 1
    for name in (b"ZeroAdamW", b"SyncBNStats"):
        assert lib.dragon_operator_is_registered(name) == 1
    assert lib.dragon_schema_allows_inplace(b"SyncBNStats", 0, 0) == 1
    assert lib.dragon_schema_allows_inplace(b"SyncBNStats", 0, 1) == 0
