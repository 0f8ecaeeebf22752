"""Memory policy on top of the library's stream-ordered pool.

Mirrors src/memory.jl of the reference: limits given as ``"none"``, ``"N MiB"``, ``"N GiB"`` or
``"N %"`` (parse_memory_limit, :37-65), ``pool_alloc`` / ``pool_free`` (:491-536), statistics
(:103-166, :376-404) and the out-of-memory ladder of ``alloc_or_retry!``
(src/runtime/memory/utils.jl:1-47): the library reports B200_OOM and never retries itself, so
the collector of the host language stays outside the C code.
"""
from __future__ import annotations

import builtins
import contextlib
import ctypes as C
import gc
import math
import os
import threading

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
    """Returns cached pool memory to the driver (``AMDGPU.reclaim``, src/memory.jl:333-344): the
    registered hooks run, every open stream of the device gives up its operator scratch, then the
    pool is trimmed to `keep` bytes."""
    from .runtime import live_streams
    dev = current_device() if dev is None else dev
    for fn in _reclaim_hooks:
        fn()
    for st in live_streams(dev):
        st.release_scratch()
        st.synchronize()             # the stream-ordered frees must have run before the trim
    check(lib.b200_pool_trim(dev, keep))


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


# ---- allocation cache (GPUArrays.AllocCache / @cached, hooked in src/array.jl:24-32) --------------------

class AllocCache:
    """Buffers allocated while the cache is active (``with cached(cache):``) belong to the cache:
    the arrays' finalisers and ``unsafe_free_`` leave them alone, leaving the block marks them
    free, and the next pass through the block gets the same buffers back for requests of the same
    size on the same stream.  Repeated iterations then make no allocator calls at all, which is
    also what lets a block with temporaries be captured into a graph
    (test/core/graph_tests.jl:37-55)."""

    def __init__(self):
        self._lock = threading.Lock()
        self.free: dict[tuple, list[int]] = {}           # key: (device, stream, bytes)
        self.busy: list[tuple[tuple, int]] = []

    def take(self, key: tuple, alloc) -> int:
        with self._lock:
            pool = self.free.get(key)
            ptr = pool.pop() if pool else None
        if ptr is None:
            ptr = alloc()
        with self._lock:
            self.busy.append((key, ptr))
        return ptr

    def release_busy(self) -> None:
        with self._lock:
            for key, ptr in self.busy:
                self.free.setdefault(key, []).append(ptr)
            self.busy.clear()

    def sizeof(self) -> int:
        with self._lock:
            return builtins.sum(k[-1] * len(v) for k, v in self.free.items()) + builtins.sum(k[-1] for k, _ in self.busy)

    def unsafe_free_(self, stream: Stream | None = None) -> None:
        """``unsafe_free!(cache)``: hand every buffer back to the pool."""
        with self._lock:
            ptrs = [p for v in self.free.values() for p in v] + [p for _, p in self.busy]
            self.free.clear()
            self.busy.clear()
        for p in ptrs:
            pool_free(p, stream)


class _CacheTLS(threading.local):
    def __init__(self):
        self.stack: list[AllocCache] = []


_cache_tls = _CacheTLS()


def current_cache() -> "AllocCache | None":
    return _cache_tls.stack[-1] if _cache_tls.stack else None


@contextlib.contextmanager
def cached(cache: AllocCache):
    """``GPUArrays.@cached cache expr``."""
    _cache_tls.stack.append(cache)
    try:
        yield cache
    finally:
        _cache_tls.stack.pop()
        cache.release_busy()


# ---- idle pool trimming (pool_cleanup, src/memory.jl:289-321) ------------------------------------------

class PoolCleanup:
    """Every `interval` seconds look at each device's pool: if nothing was allocated from it for
    `idle_periods` consecutive looks, return its cached memory to the driver (``reclaim``).
    `activity(dev)` returns a monotonically growing allocation counter; `trim(dev)` does the
    reclaim - both injectable so the policy can be tested without a device."""

    def __init__(self, devices_fn, activity, trim, interval: float = 60.0, idle_periods: int = 5):
        self.devices_fn, self.activity, self.trim = devices_fn, activity, trim
        self.interval, self.idle_periods = interval, idle_periods
        self._last: dict[int, int] = {}
        self._idle: dict[int, int] = {}
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def step(self) -> list[int]:
        """One look at all devices; returns the devices that were trimmed."""
        trimmed = []
        for dev in self.devices_fn():
            count = self.activity(dev)
            if count is None:
                continue
            if count != self._last.get(dev):
                self._idle[dev] = 0
            else:
                self._idle[dev] = self._idle.get(dev, 0) + 1
            self._last[dev] = count
            if self._idle[dev] >= self.idle_periods:
                self.trim(dev)
                trimmed.append(dev)
        return trimmed

    def start(self) -> "PoolCleanup":
        if self._thread is None:
            def run():
                while not self._stop.wait(self.interval):
                    try:
                        self.step()
                    except Exception:
                        pass
            self._thread = threading.Thread(target=run, name="b200-pool-cleanup", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
            self._thread = None


def start_pool_cleanup(interval: float = 60.0, idle_periods: int = 5) -> PoolCleanup:
    """The reference starts this task with the package (src/memory.jl:289-321); here it is opt-in."""
    from .runtime import devices
    return PoolCleanup(devices, lambda d: pool_stats(d)["alloc_count"], lambda d: reclaim(d),
                       interval, idle_periods).start()
