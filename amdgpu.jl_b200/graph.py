"""Graph capture: ``capture`` / ``instantiate`` / ``launch`` / ``update`` / ``is_capturing`` /
``captured``.

Mirrors src/hip/graph.jl:16-168 of the reference.  Every operator of the library only enqueues
kernels and memsets on the stream it is given, so a sequence of them can be recorded once and
replayed with one launch; for the small configurations (tens of microseconds per operator) that
removes the per-call host cost.  Two rules follow from how the library works:

* an operator that needs more per-stream scratch than the stream already holds refuses to run
  inside a capture; ``captured`` therefore does what the reference's ``@captured`` does when its
  first capture fails: it runs the function once normally and captures it again;
* device arrays created inside the captured function must be freed inside it
  (``unsafe_free_``) or come from an ``AllocCache`` (``memory.cached``), as in
  test/core/graph_tests.jl:19-55.
"""
from __future__ import annotations

import ctypes as C
import gc
from contextlib import contextmanager

from ._lib import B200Error, check, lib
from .runtime import Stream, current_stream

MODE_GLOBAL, MODE_THREAD_LOCAL, MODE_RELAXED = 0, 1, 2


class Graph:
    """``HIPGraph``: a captured, not yet executable graph."""

    def __init__(self, handle: int):
        self.handle = handle

    def close(self) -> None:
        if self.handle:
            h, self.handle = self.handle, None
            lib.b200_graph_destroy(C.c_void_p(h))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GraphExec:
    """``HIPGraphExec``: an instantiated graph."""

    def __init__(self, handle: int):
        self.handle = handle

    def close(self) -> None:
        if self.handle:
            h, self.handle = self.handle, None
            lib.b200_graph_exec_destroy(C.c_void_p(h))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def is_capturing(stream: Stream | None = None) -> bool:
    """``AMDGPU.is_capturing(stream)`` (src/hip/graph.jl:118-122)."""
    out = C.c_int32(0)
    check(lib.b200_stream_is_capturing((stream or current_stream()).handle, C.byref(out)))
    return bool(out.value)


@contextmanager
def _gc_paused():
    # a finaliser that frees device memory in the middle of a capture would be recorded too
    was = gc.isenabled()
    gc.disable()
    try:
        yield
    finally:
        if was:
            gc.enable()


def capture(fn, mode: int = MODE_GLOBAL, throw_error: bool = True, stream: Stream | None = None) -> Graph | None:
    """``AMDGPU.capture(f; flags, throw_error)`` (src/hip/graph.jl:36-58): records what `fn()`
    enqueues on the stream; ``None`` when the capture failed and `throw_error` is false."""
    st = stream or current_stream()
    with _gc_paused():
        check(lib.b200_graph_capture_begin(st.handle, mode))
        failure = None
        try:
            fn()
        except Exception as e:      # the capture must be ended whatever happened inside
            failure = e
        out = C.c_void_p()
        status = lib.b200_graph_capture_end(st.handle, C.byref(out))
    if failure is None and status == 0 and out.value:
        return Graph(out.value)
    if out.value:
        lib.b200_graph_destroy(out)
    if not throw_error:
        return None
    if failure is not None:
        raise failure
    check(status)
    raise B200Error(status, "stream capture produced no graph")


def instantiate(graph: Graph) -> GraphExec:
    """``AMDGPU.instantiate(graph)`` (src/hip/graph.jl:66-76)."""
    out = C.c_void_p()
    check(lib.b200_graph_instantiate(C.c_void_p(graph.handle), C.byref(out)))
    return GraphExec(out.value)


def launch(exec_: GraphExec, stream: Stream | None = None) -> None:
    """``AMDGPU.launch(exec, stream)`` (src/hip/graph.jl:85-87)."""
    check(lib.b200_graph_launch(C.c_void_p(exec_.handle), (stream or current_stream()).handle))


def update(exec_: GraphExec, graph: Graph, throw_error: bool = True) -> bool:
    """``AMDGPU.update(exec, graph; throw_error)`` (src/hip/graph.jl:97-109)."""
    ok = C.c_int32(0)
    check(lib.b200_graph_exec_update(C.c_void_p(exec_.handle), C.c_void_p(graph.handle), C.byref(ok)))
    if not ok.value and throw_error:
        raise RuntimeError("failed to update the executable graph: the new graph has a different topology")
    return bool(ok.value)


def captured(fn, stream: Stream | None = None) -> GraphExec:
    """``AMDGPU.@captured expr`` (src/hip/graph.jl:133-168): capture `fn`, instantiate and launch
    it once; if the first capture fails (here: an operator had to grow its scratch), run `fn`
    normally, then capture again and return that graph without another launch."""
    st = stream or current_stream()
    graph = capture(fn, throw_error=False, stream=st)
    if graph is not None:
        exec_ = instantiate(graph)
        launch(exec_, st)
        return exec_
    fn()
    return instantiate(capture(fn, stream=st))
