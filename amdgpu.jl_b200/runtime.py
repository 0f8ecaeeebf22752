"""Devices, streams, events and the thread-local state that selects them.

Mirrors the reference's task-local state (src/tls.jl:1-199: one current device per task and
one lazily created stream per device per task), ``HIPStream``/``HIPEvent``
(src/hip/stream.jl:4-143, src/hip/event.jl:1-75) and the user-facing ``synchronize`` /
``@elapsed`` helpers (src/highlevel.jl:36-81,180-191).  Python threads play the part of Julia
tasks.  Device ordinals are 0-based here, as at the driver (src/hip/device.jl:24-30).
"""
from __future__ import annotations

import ctypes as C
import threading
import weakref
from contextlib import contextmanager

from . import _lib
from ._lib import check, lib


_live_streams: "weakref.WeakSet[Stream]" = weakref.WeakSet()


class Stream:
    """A CUDA stream with a priority in {-1: high, 0: normal, 1: low} (src/hip/stream.jl:17-27)."""

    def __init__(self, device: int | None = None, priority: int = 0, _handle=None, _owned=True):
        self.device = current_device() if device is None else device
        self.priority = priority
        if _handle is None:
            h = C.c_void_p()
            check(lib.b200_stream_create(self.device, priority, C.byref(h)))
            _handle = h
        self.handle = _handle
        self._owned = _owned
        _live_streams.add(self)

    def release_scratch(self) -> None:
        """Returns the operator scratch this stream holds (reduction partials, radix double
        buffers, scan descriptors) to the pool; the next operator allocates it again."""
        if self.handle is not None:
            check(lib.b200_stream_release_scratch(self.handle))

    @classmethod
    def wrap(cls, device: int, cuda_stream: int) -> "Stream":
        """Wraps a ``cudaStream_t`` owned by someone else (for instance a torch stream)."""
        h = C.c_void_p()
        check(lib.b200_stream_wrap(device, C.c_void_p(cuda_stream), C.byref(h)))
        return cls(device, 0, _handle=h, _owned=True)

    def synchronize(self) -> None:
        check(lib.b200_stream_sync(self.handle))

    def isdone(self) -> bool:
        return check(lib.b200_stream_query(self.handle)) == _lib.OK

    @property
    def raw(self) -> int:
        p = C.c_void_p()
        check(lib.b200_stream_raw(self.handle, C.byref(p)))
        return p.value or 0

    def wait(self, event: "Event") -> None:
        check(lib.b200_stream_wait_event(self.handle, event.handle))

    def close(self) -> None:
        if self.handle is not None and self._owned:
            lib.b200_stream_destroy(self.handle)
        self.handle = None

    def __del__(self):  # finalizer, as HIPStream's (src/hip/stream.jl:29-33)
        try:
            self.close()
        except Exception:
            pass


class Event:
    """``HIPEvent`` (src/hip/event.jl:1-75)."""

    def __init__(self, device: int | None = None, timing: bool = False):
        self.device = current_device() if device is None else device
        h = C.c_void_p()
        check(lib.b200_event_create(self.device, 1 if timing else 0, C.byref(h)))
        self.handle = h

    def record(self, stream: Stream | None = None) -> "Event":
        check(lib.b200_event_record(self.handle, (stream or current_stream()).handle))
        return self

    def synchronize(self) -> None:
        check(lib.b200_event_sync(self.handle))

    def isdone(self) -> bool:
        return check(lib.b200_event_query(self.handle)) == _lib.OK

    def __del__(self):
        try:
            if self.handle is not None:
                lib.b200_event_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


def elapsed_ms(start: Event, stop: Event) -> float:
    """Milliseconds between two recorded timing events (src/hip/event.jl:71-75)."""
    ms = C.c_float()
    check(lib.b200_event_elapsed_ms(start.handle, stop.handle, C.byref(ms)))
    return float(ms.value)


# ---- thread-local state (src/tls.jl) --------------------------------------------------------------
class _TLS(threading.local):
    def __init__(self):
        self.device = 0
        self.streams: dict[int, Stream] = {}


_tls = _TLS()


def live_streams(device: int | None = None) -> list:
    """The streams of this process that are still open (all devices, or one)."""
    return [s for s in list(_live_streams) if s.handle is not None and (device is None or s.device == device)]


def ndevices() -> int:
    n = C.c_int32()
    check(lib.b200_device_count(C.byref(n)))
    return n.value


def devices() -> list[int]:
    return list(range(ndevices()))


def current_device() -> int:
    """``AMDGPU.device()`` (src/tls.jl:45)."""
    return _tls.device


def device_(dev: int) -> int:
    """``AMDGPU.device!(dev)`` (src/tls.jl:53-67): switches this thread's device; its stream
    for that device is created on first use."""
    if not 0 <= dev < ndevices():
        raise ValueError(f"device {dev} out of range")
    _tls.device = dev
    return dev


def current_stream() -> Stream:
    """``AMDGPU.stream()`` (src/tls.jl:71-86)."""
    dev = _tls.device
    st = _tls.streams.get(dev)
    if st is None or st.handle is None:
        st = Stream(dev, 0)
        _tls.streams[dev] = st
    return st


def stream_(st: Stream) -> Stream:
    """``AMDGPU.stream!(s)`` (src/tls.jl:93-116): makes `st` this thread's stream (and its
    device the current device)."""
    _tls.device = st.device
    _tls.streams[st.device] = st
    return st


@contextmanager
def using_stream(st: Stream):
    """``AMDGPU.stream!(f, s)`` do-block form (src/tls.jl:118-131)."""
    old_dev, old = _tls.device, _tls.streams.get(st.device)
    stream_(st)
    try:
        yield st
    finally:
        _tls.device = old_dev
        if old is not None:
            _tls.streams[st.device] = old
        else:
            _tls.streams.pop(st.device, None)


def priority_(priority: int) -> Stream:
    """``AMDGPU.priority!(p)`` (src/tls.jl:158-190): replaces this thread's stream by one of the
    requested priority."""
    st = Stream(_tls.device, priority)
    _tls.streams[_tls.device] = st
    return st


def synchronize(stream: Stream | None = None) -> None:
    """``AMDGPU.synchronize`` (src/highlevel.jl:36-61): waits for the stream and surfaces
    errors latched by kernels."""
    (stream or current_stream()).synchronize()


def device_synchronize(dev: int | None = None) -> None:
    check(lib.b200_device_sync(current_device() if dev is None else dev))


@contextmanager
def elapsed(stream: Stream | None = None):
    """``AMDGPU.@elapsed`` (src/highlevel.jl:180-191).  Usage::

        with elapsed() as t: ...
        seconds = t()
    """
    st = stream or current_stream()
    a, b = Event(st.device, timing=True), Event(st.device, timing=True)
    a.record(st)
    result = {}
    try:
        yield lambda: result["s"]
    finally:
        b.record(st)
        b.synchronize()
        result["s"] = elapsed_ms(a, b) / 1e3


def device_properties(dev: int | None = None) -> dict:
    p = _lib.Props()
    check(lib.b200_device_props(current_device() if dev is None else dev, C.byref(p)))
    return {"name": p.name.decode(), "cc": (p.cc_major, p.cc_minor), "sm_count": p.sm_count,
            "l2_mb": p.l2_bytes_mb, "total_mem": p.total_mem, "max_smem_per_block": p.max_smem_per_block,
            "clock_khz": p.clock_khz}


def can_access_peer(dev: int, peer: int) -> bool:
    v = C.c_int32()
    check(lib.b200_can_access_peer(dev, peer, C.byref(v)))
    return bool(v.value)


def versioninfo() -> dict:
    a, b, c = C.c_int32(), C.c_int32(), C.c_int32()
    check(lib.b200_version(C.byref(a), C.byref(b), C.byref(c)))
    return {"cuda_runtime": a.value, "cuda_driver": b.value, "library": c.value}


def functional() -> bool:
    """``AMDGPU.functional()`` (src/utils.jl:136-179): is a usable device present?"""
    try:
        return ndevices() > 0
    except _lib.B200Error:
        return False
