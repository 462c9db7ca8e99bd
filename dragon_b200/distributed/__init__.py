"""`dragon.distributed`, served by the B200-native collective library.

Exports the names of dragon/python/_api/distributed/__init__.py:17-30.
"""

from dragon_b200.distributed.backend import Backend
from dragon_b200.distributed.backend import ProcessGroup
from dragon_b200.distributed.backend import as_rank
from dragon_b200.distributed.backend import finalize
from dragon_b200.distributed.backend import get_backend
from dragon_b200.distributed.backend import get_group
from dragon_b200.distributed.backend import get_rank
from dragon_b200.distributed.backend import get_world_size
from dragon_b200.distributed.backend import init_emulated_world
from dragon_b200.distributed.backend import is_cncl_available
from dragon_b200.distributed.backend import is_initialized
from dragon_b200.distributed.backend import is_mpi_available
from dragon_b200.distributed.backend import is_nccl_available
from dragon_b200.distributed.backend import new_group
from dragon_b200.distributed.ops import all_gather
from dragon_b200.distributed.ops import all_reduce
from dragon_b200.distributed.ops import all_reduce_coalesced
from dragon_b200.distributed.ops import broadcast
from dragon_b200.distributed.ops import reduce_scatter
