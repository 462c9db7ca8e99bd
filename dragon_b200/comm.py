"""Communicator: a thin object layer over the dgn C-ABI for torch CUDA tensors.

torch supplies device memory and streams only; every collective is one call
into libdgn.so (see include/dgn.h).
"""

import ctypes

import torch

from dragon_b200 import _C

_TORCH_TO_DGN = {
    torch.uint8: _C.U8,
    torch.int8: _C.I8,
    torch.int32: _C.I32,
    torch.int64: _C.I64,
    torch.float16: _C.F16,
    torch.bfloat16: _C.BF16,
    torch.float32: _C.F32,
    torch.float64: _C.F64,
}


def dgn_dtype(torch_dtype):
    """Map a torch dtype onto the dgn_dtype enum (the reference's Numerical list)."""
    try:
        return _TORCH_TO_DGN[torch_dtype]
    except KeyError:
        raise TypeError("Unsupported data type: {}".format(torch_dtype))


def redop_code(reduction):
    """'sum' / 'MEAN' / ... -> dgn_redop; unknown names are an error, as in the
    reference's op map (collective_op_impl_mpi.cc:111-126)."""
    code = _C.REDOPS.get(str(reduction).upper())
    if code is None:
        raise ValueError("Unsupported reduction: {}".format(reduction))
    return code


def _stream_ptr(stream, device):
    if stream is None:
        stream = torch.cuda.current_stream(device)
    if isinstance(stream, int):
        return ctypes.c_void_p(stream)
    return ctypes.c_void_p(stream.cuda_stream)


def _check_tensor(t, device):
    if not t.is_cuda or t.device.index != device:
        raise ValueError("tensor must live on cuda:{} (got {})".format(device, t.device))
    if not t.is_contiguous():
        raise ValueError("tensor must be contiguous")


class _RawDeviceBytes(object):
    """Device memory owned by the library, exposed to torch without a copy."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PreparedAllReduce(object):
    """An all-reduce over a fixed tensor list with its argument arrays built once."""

    def __init__(self, comm, inputs, outputs, reduction):
        n = len(inputs)
        if len(outputs) != n:
            raise ValueError("inputs and outputs differ in length")
        dtype = inputs[0].dtype if n else torch.float32
        for a, b in zip(inputs, outputs):
            _check_tensor(a, comm.device)
            _check_tensor(b, comm.device)
            if a.dtype != dtype or b.dtype != dtype:
                raise TypeError("all tensors of one all-reduce must share a dtype")
            if a.numel() != b.numel():
                raise ValueError("input/output sizes differ")
        self._keep = (list(inputs), list(outputs))
        self._comm = comm
        self._n = n
        self._in = (ctypes.c_void_p * max(n, 1))(*[t.data_ptr() for t in inputs])
        self._out = (ctypes.c_void_p * max(n, 1))(*[t.data_ptr() for t in outputs])
        self._counts = (ctypes.c_int64 * max(n, 1))(*[t.numel() for t in inputs])
        self._dtype = dgn_dtype(dtype)
        self._redop = redop_code(reduction)
        self._fn = _C.lib().dgn_allreduce

    def __call__(self, stream=None):
        rc = self._fn(self._comm._h, self._in, self._out, self._counts, self._n, self._dtype,
                      self._redop, _stream_ptr(stream, self._comm.device))
        if rc != _C.OK:
            _C.check(rc)


class Communicator(object):
    """One rank of a dgn communicator."""

    def __init__(self, handle):
        self._h = ctypes.c_void_p(handle)
        lib = _C.lib()
        self.rank = lib.dgn_comm_rank(self._h)
        self.size = lib.dgn_comm_size(self._h)
        self.device = lib.dgn_comm_device(self._h)

    # -- construction ------------------------------------------------------
    @classmethod
    def init_local(cls, rank, nranks, device, symm_bytes=None):
        """Step 1 of the handle-exchange bootstrap.  `symm_bytes` asks for a
        symmetric arena of that size (see symm_empty); every rank must ask for
        the same."""
        h = ctypes.c_void_p()
        if symm_bytes is None:
            _C.check(_C.lib().dgn_comm_init_local(rank, nranks, device, ctypes.byref(h)))
        else:
            _C.check(_C.lib().dgn_comm_init_symmetric(rank, nranks, device, int(symm_bytes), ctypes.byref(h)))
        return cls(h.value)

    def handle_bytes(self):
        buf = ctypes.create_string_buffer(_C.HANDLE_BYTES)
        _C.check(_C.lib().dgn_comm_get_handle(self._h, buf))
        return buf.raw

    def connect(self, all_handles):
        blob = b"".join(all_handles)
        if len(blob) != self.size * _C.HANDLE_BYTES:
            raise ValueError("expected {} handles".format(self.size))
        _C.check(_C.lib().dgn_comm_connect(self._h, blob))
        return self

    @classmethod
    def create(cls, rank, nranks, device, rendezvous_dir, tag, timeout_ms=60000):
        """File-rendezvous bootstrap (no external channel needed)."""
        h = ctypes.c_void_p()
        _C.check(_C.lib().dgn_comm_create(rank, nranks, device, str(rendezvous_dir).encode(),
                                          str(tag).encode(), int(timeout_ms), ctypes.byref(h)))
        return cls(h.value)

    @classmethod
    def emulated(cls, nranks, device=0):
        """`nranks` virtual ranks on one device; a collective runs once every
        virtual rank has issued it."""
        arr = (ctypes.c_void_p * nranks)()
        _C.check(_C.lib().dgn_comm_create_emulated(nranks, device, arr))
        return [cls(arr[i]) for i in range(nranks)]

    def destroy(self):
        if self._h is not None and self._h.value:
            _C.lib().dgn_comm_destroy(self._h)
            self._h = None

    # -- knobs ---------------------------------------------------------------
    def status(self):
        return _C.lib().dgn_comm_status(self._h)

    def has_nvls(self):
        """True if the NVSwitch multicast variant was set up for this communicator."""
        return bool(_C.lib().dgn_comm_has_nvls(self._h))

    # -- symmetric memory --------------------------------------------------------
    def symm_capacity(self):
        """Bytes of the symmetric arena (0 without NVSwitch multicast)."""
        return int(_C.lib().dgn_comm_symm_capacity(self._h))

    def symm_empty(self, numel, dtype):
        """A tensor of `numel` elements in the symmetric arena.  Every rank must
        make the same sequence of symm_empty calls.  An in-place all-reduce on
        it (a whole number of 16-byte vectors) is done by the switch on the
        buffers themselves.  The memory belongs to the communicator."""
        nbytes = int(numel) * torch.empty((), dtype=dtype).element_size()
        p = ctypes.c_void_p()
        _C.check(_C.lib().dgn_comm_symm_alloc(self._h, nbytes, ctypes.byref(p)))
        holder = _RawDeviceBytes(p.value, max(nbytes, 1))
        flat = torch.as_tensor(holder, device=torch.device("cuda", self.device))
        return flat[:nbytes].view(dtype)

    def symm_reset(self):
        _C.check(_C.lib().dgn_comm_symm_reset(self._h))

    def set_wait_limit_ms(self, ms):
        _C.check(_C.lib().dgn_comm_set_wait_limit_ms(self._h, int(ms)))

    def set_tuning(self, variant=0, blocks=0, threads=0, chunk_bytes=0):
        _C.check(_C.lib().dgn_comm_set_tuning(self._h, variant, blocks, threads, chunk_bytes))

    def set_knob(self, name, value):
        """Named launch parameter or size threshold (dgn_comm_set_knob); 0 restores the default."""
        _C.check(_C.lib().dgn_comm_set_knob(self._h, name.encode(), int(value)))

    def last_launch(self):
        v, b, t, r = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        cb = ctypes.c_int64()
        _C.check(_C.lib().dgn_comm_last_launch(self._h, ctypes.byref(v), ctypes.byref(b), ctypes.byref(t),
                                               ctypes.byref(cb), ctypes.byref(r)))
        return {"variant": v.value, "blocks": b.value, "threads": t.value, "chunk_bytes": cb.value,
                "rounds": r.value}

    # -- collectives -----------------------------------------------------------
    def prepare_all_reduce(self, inputs, outputs=None, reduction="SUM"):
        if outputs is None:
            outputs = inputs
        return PreparedAllReduce(self, list(inputs), list(outputs), reduction)

    def all_reduce(self, inputs, outputs=None, reduction="SUM", stream=None):
        """ALLREDUCE of a tensor list as one message (in place when outputs is None)."""
        if isinstance(inputs, torch.Tensor):
            inputs = [inputs]
        if isinstance(outputs, torch.Tensor):
            outputs = [outputs]
        self.prepare_all_reduce(inputs, outputs, reduction)(stream)

    def all_reduce_host(self, values, reduction="SUM"):
        """Synchronous all-reduce of a small numpy array that lives in host memory."""
        import numpy as np
        codes = {np.dtype(np.uint8): _C.U8, np.dtype(np.int8): _C.I8, np.dtype(np.int32): _C.I32,
                 np.dtype(np.int64): _C.I64, np.dtype(np.float16): _C.F16, np.dtype(np.float32): _C.F32,
                 np.dtype(np.float64): _C.F64}
        arr = np.ascontiguousarray(values)
        if arr.dtype not in codes:
            raise TypeError("Unsupported data type: {}".format(arr.dtype))
        out = np.empty_like(arr)
        _C.check(_C.lib().dgn_allreduce_host(self._h, arr.ctypes.data, out.ctypes.data, arr.size,
                                             codes[arr.dtype], redop_code(reduction)))
        return out

    def all_gather(self, tensor, output, stream=None):
        """output[r] = rank r's tensor; output holds size * tensor.numel() elements."""
        _check_tensor(tensor, self.device)
        _check_tensor(output, self.device)
        if output.dtype != tensor.dtype:
            raise TypeError("dtype mismatch")
        if output.numel() != self.size * tensor.numel():
            raise ValueError("output must hold size * tensor.numel() elements")
        _C.check(_C.lib().dgn_allgather(self._h, tensor.data_ptr(), output.data_ptr(), tensor.numel(),
                                        dgn_dtype(tensor.dtype), _stream_ptr(stream, self.device)))

    def broadcast(self, tensor, root=0, stream=None):
        _check_tensor(tensor, self.device)
        _C.check(_C.lib().dgn_broadcast(self._h, tensor.data_ptr(), tensor.numel(),
                                        dgn_dtype(tensor.dtype), int(root), _stream_ptr(stream, self.device)))

    def reduce_scatter(self, tensor, output, reduction="SUM", stream=None):
        _check_tensor(tensor, self.device)
        _check_tensor(output, self.device)
        if output.dtype != tensor.dtype:
            raise TypeError("dtype mismatch")
        if tensor.numel() != self.size * output.numel():
            raise ValueError("input must hold size * output.numel() elements")
        _C.check(_C.lib().dgn_reducescatter(self._h, tensor.data_ptr(), output.data_ptr(), output.numel(),
                                            dgn_dtype(tensor.dtype), redop_code(reduction),
                                            _stream_ptr(stream, self.device)))
