"""Memory policy on top of the library's stream-ordered pool.

Mirrors src/memory.jl of the reference: limits given as ``"none"``, ``"N MiB"``, ``"N GiB"`` or
``"N %"`` (parse_memory_limit, :37-65), ``pool_alloc`` / ``pool_free`` (:491-536), statistics
(:103-166, :376-404) and the out-of-memory ladder of ``alloc_or_retry!``
(src/runtime/memory/utils.jl:1-47): the library reports B200_OOM and never retries itself, so
the collector of the host language stays outside the C code.
"""
from __future__ import annotations

import ctypes as C
import gc
import math
import os

from . import _lib
from ._lib import OutOfMemoryError, check, lib
from .runtime import Stream, current_device, current_stream

UINT64_MAX = (1 << 64) - 1


def mem_info(dev: int | None = None) -> tuple[int, int]:
    """(free, total) bytes of the device, ``AMDGPU.info()`` (src/memory.jl:7-35)."""
    f, t = C.c_size_t(), C.c_size_t()
    check(lib.b200_mem_info(current_device() if dev is None else dev, C.byref(f), C.byref(t)))
    return f.value, t.value


def parse_memory_limit(limit: str, total_memory: int) -> int:
    """Same grammar and errors as parse_memory_limit (src/memory.jl:37-65)."""
    if limit == "none":
        return UINT64_MAX
    parts = limit.split()
    if len(parts) != 2:
        raise ValueError(f"memory limit must look like '8 GiB', '512 MiB', '50 %' or 'none', got {limit!r}")
    value, unit = parts
    if unit not in ("%", "MiB", "GiB"):
        raise ValueError(f"memory limit must be specified in ('%', 'MiB', 'GiB') units, but `{unit}` was given")
    if unit == "%":
        v = int(value)
        if not 0 < v <= 100:
            raise ValueError(f"invalid percentage value for memory limit `{v}`; must be in (0, 100] or 'none'")
        lim = math.floor(total_memory * (v / 100))
    else:
        lim = int(value) * (1024 ** 2 if unit == "MiB" else 1024 ** 3)
    if lim > total_memory:
        raise ValueError(f"memory limit {lim} B is bigger than the actual memory {total_memory} B; "
                         "set to 'none' to disable the limit")
    return lim


def configure(dev: int | None = None, hard: str | None = None, soft: str | None = None) -> None:
    """Applies hard / soft limits (Preferences keys ``hard_memory_limit`` / ``soft_memory_limit``
    in the reference, src/memory.jl:70-98; environment B200_HARD_MEMORY_LIMIT /
    B200_SOFT_MEMORY_LIMIT here).  The hard limit bounds live bytes; the soft limit becomes the
    pool's release threshold (src/runtime/memory/hip.jl:4-25)."""
    dev = current_device() if dev is None else dev
    total = mem_info(dev)[1]
    hard = hard if hard is not None else os.environ.get("B200_HARD_MEMORY_LIMIT", "none")
    soft = soft if soft is not None else os.environ.get("B200_SOFT_MEMORY_LIMIT", "none")
    check(lib.b200_pool_configure(dev, parse_memory_limit(hard, total), parse_memory_limit(soft, total)))


_reclaim_hooks: list = []


def reclaim_hook(fn) -> None:
    """Registers a callable run when memory is short (src/memory.jl:282, :333-344)."""
    _reclaim_hooks.append(fn)


def reclaim(dev: int | None = None, keep: int = 0) -> None:
    """Returns cached pool memory to the driver (``AMDGPU.reclaim``, src/memory.jl:333-344)."""
    for fn in _reclaim_hooks:
        fn()
    check(lib.b200_pool_trim(current_device() if dev is None else dev, keep))


def _try_alloc(nbytes: int, stream: Stream) -> int:
    p = C.c_void_p()
    check(lib.b200_malloc_async(C.byref(p), nbytes, stream.handle))
    return p.value or 0


def pool_alloc(nbytes: int, stream: Stream | None = None) -> int:
    """Stream-ordered allocation with the reference's retry ladder (alloc_or_retry!,
    src/runtime/memory/utils.jl:1-47): stream sync, device sync, incremental collection, full
    collection, pool trim + reclaim hooks; only out-of-memory is retried
    (src/runtime/memory/hip.jl:51-60)."""
    stream = stream or current_stream()
    if nbytes == 0:
        return 0
    phases = (
        lambda: None,
        lambda: stream.synchronize(),
        lambda: check(lib.b200_device_sync(stream.device)),
        lambda: gc.collect(0),
        lambda: gc.collect(),
        lambda: reclaim(stream.device),
    )
    last: OutOfMemoryError | None = None
    for phase in phases:
        phase()
        try:
            return _try_alloc(nbytes, stream)
        except OutOfMemoryError as e:
            last = e
    assert last is not None
    raise last


def pool_free(ptr: int, stream: Stream | None = None) -> None:
    """Stream-ordered free (src/memory.jl:511-536, src/runtime/memory/hip.jl:82-89)."""
    if ptr:
        check(lib.b200_free_async(C.c_void_p(ptr), (stream or current_stream()).handle))


def pool_stats(dev: int | None = None) -> dict:
    """AllocStats / MemoryStats / pool_status in one record (src/memory.jl:103-166, :376-404)."""
    s = _lib.PoolStats()
    check(lib.b200_pool_stats(current_device() if dev is None else dev, C.byref(s)))
    return {name: getattr(s, name) for name, _ in _lib.PoolStats._fields_}


def used_memory(dev: int | None = None) -> int:
    return pool_stats(dev)["pool_used"]


def cached_memory(dev: int | None = None) -> int:
    s = pool_stats(dev)
    return s["pool_reserved"] - s["pool_used"]
