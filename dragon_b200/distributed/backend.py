"""Distributed backend: process groups over dgn communicators.

Same public surface as dragon/python/core/distributed/backend.py:25-314
(Backend, ProcessGroup, new_group, get_rank, get_world_size, get_group,
get_backend, is_*_available, is_initialized, finalize).  Where the reference
bootstraps through MPI (mpiInitialize / mpiCreateGroup,
dragon/modules/python/mpi.h:36-115), this module needs a "world": who am I,
how many are we, and a way to all-gather a few bytes.  Three worlds exist:

* torch.distributed, when it is initialised (one process per GPU);
* a single-process world of size 1 (the default);
* an emulated world (``init_emulated_world``): n virtual ranks inside one
  process on one device, the current one chosen with ``as_rank``; used to run
  multi-rank code where fewer GPUs than ranks are available.

The `comm` / `group` integers a group hands to the operator are handles of
this library (the reference passes MPI_Comm / MPI_Group pointer values).
"""

import atexit
import contextlib
import itertools
import threading


class _Stack(threading.local):
    """Thread-local stack with a default (dragon/python/core/util/tls.py)."""

    def __init__(self):
        super().__init__()
        self._items = []

    def get_default(self):
        return self._items[-1] if self._items else None

    @contextlib.contextmanager
    def get_controller(self, default):
        self._items.append(default)
        try:
            yield default
        finally:
            self._items.pop()


class Backend(object):
    """Names of the collective backends a group can ask for (MPI, NCCL, CNCL,
    or AUTO for "whichever is there").  `Backend(name)` returns the canonical
    upper-case string, as `dragon.distributed.Backend` does
    (dragon/python/core/distributed/backend.py); the strings are kept for
    compatibility only: on a CUDA tensor every backend runs the same
    peer-memory kernels of this library."""

    UNDEFINED = "UNDEFINED"
    AUTO = "AUTO"
    MPI = "MPI"
    NCCL = "NCCL"
    CNCL = "CNCL"

    # backends that exist only where their library is present: name -> probe
    _NEEDS = {"NCCL": lambda: is_nccl_available(), "CNCL": lambda: is_cncl_available()}

    def __new__(cls, name):
        if not isinstance(name, str):
            raise ValueError("Backend name must be a string, but got: {}".format(name))
        canonical = getattr(cls, name.upper(), cls.UNDEFINED)
        if canonical == cls.UNDEFINED or canonical not in (cls.AUTO, cls.MPI, cls.NCCL, cls.CNCL):
            raise ValueError("Invalid backend: " + name)
        if canonical == cls.AUTO:
            present = [b for b, probe in cls._NEEDS.items() if probe()]
            return present[0] if present else cls.MPI
        probe = cls._NEEDS.get(canonical)
        if probe is not None and not probe():
            raise ValueError("{} backend is not available.".format(canonical))
        return canonical


class ProcessGroup(object):
    """A set of ranks that run collectives together.  `arguments` is what the
    collective operators receive (communicator, group handle, backend, ranks),
    under the keys the reference's operators read."""

    def __init__(self, ranks, comm, handle, backend):
        self._ranks, self._comm, self._handle = ranks, comm, handle
        self._backend = Backend("AUTO" if backend is None else backend)
        self._arguments = dict(comm=comm, group=handle, backend=self._backend, ranks=ranks)

    arguments = property(lambda self: self._arguments, doc="Operator arguments of this group.")
    backend = property(lambda self: self._backend, doc="Backend of this group.")
    ranks = property(lambda self: self._ranks, doc="Ranks of this group (None: not a member).")

    @property
    def size(self):
        """Number of ranks; 0 for a group this process is not part of."""
        return 0 if self._ranks is None else len(self._ranks)

    def as_default(self):
        """Context manager that makes this group the default one (a group this
        process is not part of clears the default instead)."""
        target = None if self._ranks is None else self
        return _GLOBAL_PROCESS_GROUP_STACK.get_controller(target)

    def __repr__(self):
        return "{}:{}".format(self._backend, self._handle)


# ---- worlds -------------------------------------------------------------------

class _SingleWorld(object):
    def rank(self):
        return 0

    def size(self):
        return 1

    def device(self):
        import torch
        return torch.cuda.current_device()

    def create(self, ranks):
        from dragon_b200.comm import Communicator
        if list(ranks) != [0]:
            raise ValueError("a single-process world holds rank 0 only, got ranks {}".format(list(ranks)))
        return {0: Communicator.init_local(0, 1, self.device())}


class _TorchWorld(object):
    """One process per rank; torch.distributed moves the handles."""

    def __init__(self, dist):
        self.dist = dist

    def rank(self):
        return self.dist.get_rank()

    def size(self):
        return self.dist.get_world_size()

    def device(self):
        import torch
        return torch.cuda.current_device()

    def create(self, ranks):
        # Called by every process of the world, members or not
        # (the rule of MPI_Comm_create, modules/python/mpi.h:73-115).
        from dragon_b200.comm import Communicator
        me, ranks = self.rank(), list(ranks)
        comm, handle = None, None
        if me in ranks:
            comm = Communicator.init_local(ranks.index(me), len(ranks), self.device())
            handle = comm.handle_bytes()
        gathered = [None] * self.size()
        self.dist.all_gather_object(gathered, handle)
        if comm is None:
            return {}
        comm.connect([gathered[r] for r in ranks])
        return {me: comm}


class _EmulatedWorld(object):
    """n virtual ranks in this process, all on one device."""

    def __init__(self, size, device):
        self._size, self._device = int(size), int(device)
        self._current = threading.local()

    def rank(self):
        return getattr(self._current, "rank", 0)

    def size(self):
        return self._size

    def device(self):
        return self._device

    @contextlib.contextmanager
    def as_rank(self, rank):
        if not 0 <= rank < self._size:
            raise ValueError("rank {} outside the world of {}".format(rank, self._size))
        prev = self.rank()
        self._current.rank = int(rank)
        try:
            yield
        finally:
            self._current.rank = prev

    def create(self, ranks):
        from dragon_b200.comm import Communicator
        ranks = list(ranks)
        if any(not 0 <= r < self._size for r in ranks):
            raise ValueError("ranks {} outside the world of {}".format(ranks, self._size))
        comms = Communicator.emulated(len(ranks), self._device)
        return {r: c for r, c in zip(ranks, comms)}


_WORLD = None
_GROUPS = {}  # handle -> {world rank: Communicator}
_HANDLES = itertools.count(1)
_GLOBAL_MPI_CONTEXT = None
_GLOBAL_PROCESS_GROUP_STACK = _Stack()


def _world():
    global _WORLD
    if _WORLD is None:
        try:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized():
                _WORLD = _TorchWorld(dist)
        except ImportError:
            pass
        if _WORLD is None:
            _WORLD = _SingleWorld()
    return _WORLD


def init_emulated_world(size, device=0):
    """Make this process a world of `size` virtual ranks on one device."""
    global _WORLD
    finalize()
    _WORLD = _EmulatedWorld(size, device)
    _maybe_initialize()
    return _WORLD


def as_rank(rank):
    """Context manager: act as virtual rank `rank` of an emulated world."""
    world = _world()
    if not isinstance(world, _EmulatedWorld):
        raise RuntimeError("as_rank() needs init_emulated_world()")
    return world.as_rank(rank)


def communicator(group, rank=None):
    """The dgn communicator behind `group` for `rank` (default: this rank)."""
    if group is None or group.ranks is None:
        return None
    comms = _GROUPS.get(group.arguments["group"], {})
    return comms.get(_world().rank() if rank is None else rank)


def comm_argument(group):
    """Value of the operator's `comm` argument for the calling rank: the raw
    dgn_comm_t of this rank in `group`, 0 if it is not a member."""
    c = communicator(group)
    return 0 if c is None else int(c._h.value)


# ---- the reference's functions ---------------------------------------------------

def is_initialized():
    """Return whether the distributed environment is initialized."""
    return _GLOBAL_MPI_CONTEXT is not None


def is_cncl_available():
    """Return whether the CNCL backend is available (never: no MLU here)."""
    return False


def is_mpi_available():
    """Return whether the MPI backend is available.

    MPI's part in the reference -- ranks, sizes and group creation -- is
    played by the world of this module, which always exists."""
    return True


def is_nccl_available():
    """Return whether the NCCL backend is available: here, whether the CUDA
    collective library can run (a CUDA device and a built libdgn.so)."""
    try:
        import torch
        if not torch.cuda.is_available():
            return False
        from dragon_b200 import _C
        _C.lib()
        return True
    except Exception:
        return False


def finalize():
    """Finalize the distributed environment."""
    global _GLOBAL_MPI_CONTEXT, _WORLD
    for comms in _GROUPS.values():
        for c in comms.values():
            c.destroy()
    _GROUPS.clear()
    _GLOBAL_MPI_CONTEXT = None
    _WORLD = None


def get_backend(group):
    """Return the backend of given process group."""
    return group.backend


def get_group():
    """Return the current default process group."""
    return _GLOBAL_PROCESS_GROUP_STACK.get_default()


def get_rank(group=None):
    """Return the rank of current process.

    If ``group`` is **None**, return the world rank.
    Otherwise, return the rank in the group."""
    _maybe_initialize()
    world_rank = _world().rank()
    if group is not None:
        for i, rank in enumerate(group.ranks):
            if rank == world_rank:
                return i
    return world_rank


def get_world_size():
    """Return the world size of distributed env."""
    _maybe_initialize()
    return _world().size()


def new_group(ranks=None, backend=None, verbose=False):
    """Create a new communication group.

    The ``ranks`` can be set to **None** to create an empty group for
    disabling the distributed utilities.  This function should be called from
    all processes, even if they are not going to be included in this group."""
    if ranks is None:
        return ProcessGroup(None, None, None, backend)
    _maybe_initialize()
    ranks = _flatten(ranks)
    if len(set(ranks)) != len(ranks):
        raise ValueError("ranks must be distinct, got {}".format(ranks))
    handle = next(_HANDLES)
    _GROUPS[handle] = _world().create(ranks)
    if verbose and _world().rank() == ranks[0]:
        print("Rank[{}]: Create a group of {} members.\nGroup: {}".format(ranks[0], len(ranks), ranks))
    # `comm` carries the same handle: the per-rank communicator is looked up
    # when an op runs, because one process may act as several ranks.
    return ProcessGroup(ranks, handle, handle, backend)


def _flatten(seq):
    out = []
    for item in seq:
        if isinstance(item, (list, tuple)):
            out.extend(_flatten(item))
        else:
            out.append(int(item))
    return out


def _maybe_initialize():
    """Maybe initialize the distributed environment."""
    global _GLOBAL_MPI_CONTEXT
    if is_initialized():
        return
    _world()
    _GLOBAL_MPI_CONTEXT = _Context()


class _Context(object):
    """Releases the communicators on program exit."""

    _registered = False

    def __init__(self):
        if not _Context._registered:
            atexit.register(finalize)
            _Context._registered = True
