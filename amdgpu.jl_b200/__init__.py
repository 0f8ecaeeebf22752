"""B200-native backend for the dense data-parallel array path of AMDGPU.jl.

Host-side mirror of the reference's operator surface for that path (``ROCArray``, fused
broadcast, ``mapreducedim!`` and the reductions on it, ``accumulate!``/``cumsum``,
``sort!``/``sortperm``, the memory pool and the stream runtime) over the C ABI declared in
``include/b200arrays.h``.  The kernels live in ``lib/libb200arrays.so``; importing this
package fails loudly when that library is missing - there is no CPU fallback.
"""
from . import _lib
from ._lib import B200Error, OutOfMemoryError
from .runtime import (Stream, Event, elapsed_ms, elapsed, ndevices, devices, current_device, device_,
                      current_stream, stream_, using_stream, priority_, synchronize, device_synchronize,
                      device_properties, can_access_peer, versioninfo, functional)
from .memory import (mem_info, parse_memory_limit, configure, reclaim, reclaim_hook, pool_alloc, pool_free,
                     pool_stats, used_memory, cached_memory, AllocCache, cached, PoolCleanup,
                     start_pool_cleanup)
from .array import ROCArray, copyto_, zeros, ones, fill, roc
from . import broadcast
from .broadcast import Broadcasted, materialize_, promote_type
from .mapreduce import mapreducedim_, mapreduce, sum, prod, maximum, minimum   # noqa: A004
from .mapreduce import prepared as mapreduce_prepared
from .mapreduce import precompile as mapreduce_precompile
from .accumulate import accumulate_, accumulate, cumsum, cumprod
from .accumulate import prepared as accumulate_prepared
from .sorting import sort_, sort, sortperm_, sortperm
from .indexing import findall, getindex, getindex_mask, getindex_mask_dim, reverse, reverse_
from . import random
from . import graph
from .graph import Graph, GraphExec, capture, instantiate, launch, update, is_capturing, captured
from . import sharded

__all__ = [n for n in dir() if not n.startswith("_")]
