"""``ROCArray``: a dense column-major device array.

Mirrors src/array.jl of the reference: a reference-counted buffer plus ``dims`` and a byte
``offset`` (:19-39), ``pointer(A) = buffer + offset`` (:353-354), views and reshapes that
share the buffer (``derive``, :111-115), host<->device ``copyto!`` (:215-249), ``fill!``
through a pattern memset for 1/2/4/8-byte elements (:253-266) and ``unsafe_free!``.
Element ``i`` (0-based, column-major linear index) lives at ``ptr + i*itemsize``.
"""
from __future__ import annotations

import ctypes as C
import math
import threading

import numpy as np

from . import _lib
from ._lib import check, lib
from .memory import current_cache, pool_alloc, pool_free
from .runtime import Event, Stream, current_stream


class _Managed:
    """Reference-counted device buffer with the reference's ownership record (``Managed`` +
    ``DataRef``, src/memory.jl:408-418): the stream that touched it last and whether work on that
    stream may still be using it (``dirty``).  An operation on another stream first takes the
    buffer over (:meth:`take_ownership`), and the stream-ordered free goes to the last owner."""

    __slots__ = ("ptr", "nbytes", "stream", "dirty", "freed", "cached", "_lock", "__weakref__")

    def __init__(self, nbytes: int, stream: Stream):
        self.ptr, self.freed = 0, True          # a failed allocation must leave a harmless object
        self.nbytes = nbytes
        self.stream = stream
        self.dirty = True
        self._lock = threading.Lock()
        cache = current_cache()                 # GPUArrays.cached_alloc hook (src/array.jl:27-30)
        self.cached = cache is not None and nbytes > 0
        if self.cached:
            # buffers are only handed back to requests on the stream that used them last
            key = (stream.device, getattr(stream.handle, "value", stream.handle), nbytes)
            self.ptr = cache.take(key, lambda: pool_alloc(nbytes, stream))
        else:
            self.ptr = pool_alloc(nbytes, stream)
        self.freed = False

    def take_ownership(self, stream: Stream) -> None:
        """``take_ownership!(managed; stream)`` (src/memory.jl:431-446).  When the buffer was last
        used on another stream and that work may still be running, the new stream is made to wait
        for it: an event recorded on the old stream and a wait on the new one - the same ordering
        as the reference's ``synchronize(old stream)`` without blocking the host (streams of
        different devices do block)."""
        if self.stream is stream:
            self.dirty = True
            return
        with self._lock:
            old = self.stream
            if (self.dirty and old.handle is not None and stream.handle is not None
                    and old.handle.value != stream.handle.value):
                if old.device == stream.device:
                    stream.wait(Event(old.device).record(old))
                else:
                    old.synchronize()
            self.stream = stream
            self.dirty = True

    def synchronize(self) -> None:
        """``synchronize(managed)`` (src/memory.jl:422-429): wait until the last owner is done."""
        with self._lock:
            if self.dirty and self.stream.handle is not None:
                self.stream.synchronize()
                self.dirty = False

    def free(self) -> None:
        if self.cached:                         # the allocation cache owns the memory
            self.freed = True
            return
        if not self.freed and self.ptr:
            self.freed = True
            try:
                # the last owner's stream; a stale one falls back to the current stream (src/memory.jl:531-536)
                st = self.stream if self.stream.handle is not None else current_stream()
                pool_free(self.ptr, st)
            except Exception:
                pass

    def __del__(self):
        self.free()


def with_managed(stream: Stream, *arrays) -> Stream:
    """``with_managed(f, managed; stream)`` (src/memory.jl:460-469): every buffer an operation
    reads or writes is handed to the launch stream before the launch.  Returns `stream`."""
    for a in arrays:
        if a is not None:
            a.buf.take_ownership(stream)
    return stream


class ROCArray:
    __array_ufunc__ = None      # never let NumPy treat a device array as an object scalar

    def __init__(self, dtype, dims, *, _buf: _Managed | None = None, _offset: int = 0, _strides=None,
                 stream: Stream | None = None):
        """``ROCArray{T}(undef, dims)`` (src/array.jl:24-32): uninitialised storage from the pool.
        With `_strides` (element strides) the object stands for one of the reference's wrapped
        arrays over the same buffer: ``SubArray``, ``PermutedDimsArray``, ``Transpose``
        (``AnyROCArray``, src/array.jl:138-147)."""
        self.dtype = np.dtype(dtype)
        _lib.dtype_code(self.dtype)
        if isinstance(dims, (int, np.integer)):
            dims = (int(dims),)
        self.dims = tuple(int(d) for d in dims)
        if any(d < 0 for d in self.dims):
            raise ValueError("negative dimension")
        if len(self.dims) > _lib.MAX_DIMS:
            raise ValueError(f"at most {_lib.MAX_DIMS} dimensions")
        if _buf is None:
            _buf = _Managed(self.nbytes, stream or current_stream())
        self.buf = _buf
        self.offset = _offset
        self._strides = None if _strides is None else tuple(int(x) for x in _strides)
        if self._strides is not None and self._strides == self._dense_strides():
            self._strides = None

    # ---- basic properties
    @property
    def shape(self): return self.dims
    @property
    def ndim(self): return len(self.dims)
    def __len__(self): return math.prod(self.dims)
    @property
    def size(self): return math.prod(self.dims)
    @property
    def itemsize(self): return self.dtype.itemsize
    @property
    def nbytes(self): return self.size * self.dtype.itemsize
    @property
    def ptr(self) -> int:
        if self.buf.freed:
            raise RuntimeError("use of a ROCArray after unsafe_free!")
        return (self.buf.ptr + self.offset) if self.size else 0
    def _dense_strides(self):
        s, acc = [], 1
        for d in self.dims:
            s.append(acc)
            acc *= d
        return tuple(s)
    @property
    def strides(self):
        """Element strides, column-major (``strides(A)``)."""
        return self._dense_strides() if self._strides is None else self._strides
    @property
    def is_contiguous(self) -> bool:
        """True for a dense column-major array (dimensions of extent 1 may carry any stride)."""
        if self._strides is None:
            return True
        return all(d == 1 or a == b for d, a, b in zip(self.dims, self._strides, self._dense_strides()))
    def dense(self) -> "ROCArray":
        """`self` if it is dense, else a dense copy (what the reference gets from ``copy`` of a view)."""
        return self if self.is_contiguous else self.copy()
    @property
    def device(self) -> int: return self.buf.stream.device

    def tensor(self) -> _lib.Tensor:
        """The descriptor handed across the C ABI."""
        t = _lib.Tensor()
        t.ptr = self.ptr
        t.dtype = _lib.dtype_code(self.dtype)
        t.ndim = self.ndim
        for i, (d, s) in enumerate(zip(self.dims, self.strides)):
            t.shape[i] = d
            t.stride[i] = s
        return t

    # ---- construction / conversion
    @classmethod
    def from_host(cls, a, stream: Stream | None = None) -> "ROCArray":
        """``ROCArray(x::Array)`` (src/array.jl:195-203): upload; the column-major linear order
        of `a` is preserved."""
        a = np.asarray(a)
        out = cls(a.dtype, a.shape, stream=stream)
        out.copy_from_host(a, stream)
        return out

    def copy_from_host(self, a, stream: Stream | None = None) -> "ROCArray":
        """``copyto!(::ROCArray, ::Array)`` (src/array.jl:229-238)."""
        a = np.asarray(a, dtype=self.dtype)
        if a.size != self.size:
            raise ValueError("size mismatch in copyto!")
        if not self.is_contiguous:          # upload densely, then one strided device copy
            copyto_(self, ROCArray.from_host(a.reshape(self.dims, order="F"), stream), stream)
            return self
        flat = np.ascontiguousarray(a.reshape(-1, order="F"))
        st = with_managed(stream or current_stream(), self)
        if flat.nbytes:
            check(lib.b200_memcpy_async(C.c_void_p(self.ptr), C.c_void_p(flat.ctypes.data), flat.nbytes, st.handle))
            st.synchronize()   # pageable source must stay alive until the copy is done
        return self

    def to_host(self, stream: Stream | None = None) -> np.ndarray:
        """``Array(x::ROCArray)`` (src/array.jl:215-227): blocking download."""
        if not self.is_contiguous:
            return self.copy().to_host(stream)
        out = np.empty(self.size, dtype=self.dtype)
        st = with_managed(stream or current_stream(), self)
        if out.nbytes:
            check(lib.b200_memcpy_async(C.c_void_p(out.ctypes.data), C.c_void_p(self.ptr), out.nbytes, st.handle))
        st.synchronize()
        self.buf.dirty = False
        return out.reshape(self.dims, order="F")

    def item(self):
        if self.size != 1:
            raise ValueError("item() needs exactly one element")
        return self.to_host().reshape(-1)[0]

    def similar(self, dtype=None, dims=None, stream: Stream | None = None) -> "ROCArray":
        """``similar(A, T, dims)`` (src/array.jl:109): storage from the pool on the stream in use."""
        return ROCArray(self.dtype if dtype is None else dtype, self.dims if dims is None else dims,
                        stream=stream or current_stream())

    def copy(self, stream: Stream | None = None) -> "ROCArray":
        """``copy(A)`` (src/array.jl:268-272): device-to-device."""
        out = self.similar(stream=stream)
        copyto_(out, self, stream)
        return out

    def reshape(self, *dims) -> "ROCArray":
        """``reshape`` shares the buffer (``derive``, src/array.jl:111-115)."""
        if len(dims) == 1 and not isinstance(dims[0], (int, np.integer)):
            dims = tuple(dims[0])
        if math.prod(dims) != self.size:
            raise ValueError("reshape: total size must not change")
        if not self.is_contiguous:
            raise ValueError("reshape of a strided view: copy it first")
        return ROCArray(self.dtype, dims, _buf=self.buf, _offset=self.offset)

    def view(self, start: int, stop: int) -> "ROCArray":
        """Contiguous 1-D view ``@view A[start+1:stop]`` of the linear index space; the result's
        pointer is ``base + offset`` and need not be 16-byte aligned (src/array.jl:353-354)."""
        if not 0 <= start <= stop <= self.size:
            raise IndexError("view out of range")
        if not self.is_contiguous:
            raise ValueError("linear view of a strided view: copy it first")
        return ROCArray(self.dtype, (stop - start,), _buf=self.buf, _offset=self.offset + start * self.itemsize)

    def subview(self, *index) -> "ROCArray":
        """``@view A[i1, i2, ...]`` with one entry per dimension (``StridedSubROCArray``,
        src/array.jl:138-141; test/core/rocarray_base.jl:55-62).  Entries are 0-based Python
        slices (a positive step is allowed) or integers; an integer drops its dimension, as a
        scalar index does in Julia.  The result shares the buffer."""
        if len(index) != self.ndim:
            raise IndexError("subview needs one index per dimension")
        off, dims, strides = self.offset, [], []
        for ix, d, st in zip(index, self.dims, self.strides):
            if isinstance(ix, (int, np.integer)):
                if not 0 <= ix < d:
                    raise IndexError("subview index out of range")
                off += int(ix) * st * self.itemsize
                continue
            if not isinstance(ix, slice):
                raise TypeError("subview takes slices and integers")
            lo, hi, step = ix.indices(d)
            if step <= 0:
                raise ValueError("subview needs a positive step")
            n = max(0, (hi - lo + step - 1) // step)
            off += lo * st * self.itemsize if n else 0
            dims.append(n)
            strides.append(st * step)
        return ROCArray(self.dtype, tuple(dims), _buf=self.buf, _offset=off, _strides=tuple(strides))

    def permuteddims(self, perm) -> "ROCArray":
        """``PermutedDimsArray(A, perm)``: lazy, shares the buffer; `perm` is 1-based."""
        perm = tuple(int(p) for p in perm)
        if sorted(perm) != list(range(1, self.ndim + 1)):
            raise ValueError("perm must be a permutation of 1:ndims")
        st = self.strides
        return ROCArray(self.dtype, tuple(self.dims[p - 1] for p in perm), _buf=self.buf, _offset=self.offset,
                        _strides=tuple(st[p - 1] for p in perm))

    def transpose(self) -> "ROCArray":
        """``transpose(A)`` (lazy, like ``LinearAlgebra.Transpose``); a vector becomes a 1xN row.
        For the real element types of this path ``adjoint`` is the same thing."""
        if self.ndim == 1:
            return ROCArray(self.dtype, (1, self.dims[0]), _buf=self.buf, _offset=self.offset,
                            _strides=(1, self.strides[0]))
        if self.ndim != 2:
            raise ValueError("transpose needs a vector or a matrix")
        return self.permuteddims((2, 1))

    adjoint = transpose

    def permutedims(self, perm) -> "ROCArray":
        """``permutedims(A, perm)``: dense result."""
        return self.permuteddims(perm).copy()

    def reinterpret(self, dtype) -> "ROCArray":
        dtype = np.dtype(dtype)
        if not self.is_contiguous:
            raise ValueError("reinterpret of a strided view: copy it first")
        if self.nbytes % dtype.itemsize:
            raise ValueError("reinterpret: size is not a multiple of the new element size")
        return ROCArray(dtype, (self.nbytes // dtype.itemsize,), _buf=self.buf, _offset=self.offset)

    def fill_(self, value, stream: Stream | None = None) -> "ROCArray":
        """``fill!(A, x)`` as a bit-pattern memset (src/array.jl:253-266)."""
        if self.size and not self.is_contiguous:
            from .broadcast import Broadcasted, materialize_
            materialize_(self, Broadcasted.leaf(self.dtype.type(value)), stream)
            return self
        if self.size:
            bits = int.from_bytes(np.asarray(value, dtype=self.dtype).tobytes().ljust(8, b"\0"), "little")
            st = with_managed(stream or current_stream(), self)
            check(lib.b200_memset_async(C.c_void_p(self.ptr), bits, self.itemsize, self.size, st.handle))
        return self

    def unsafe_free_(self) -> None:
        """``AMDGPU.unsafe_free!`` (src/array.jl:74-79)."""
        self.buf.free()

    def __repr__(self):
        return f"ROCArray{{{self.dtype.name},{self.ndim}}}{self.dims}"

    # lazy broadcast sugar: x.dot is the operand form of `x` in a dotted expression
    @property
    def dot(self):
        from .broadcast import Broadcasted
        return Broadcasted.leaf(self)


def copyto_(dest: ROCArray, src: ROCArray, stream: Stream | None = None) -> ROCArray:
    """Device-to-device ``copyto!`` (src/array.jl:240-249)."""
    if dest.size != src.size or dest.dtype != src.dtype:
        raise ValueError("copyto!: size or element type mismatch")
    if dest.size and not (dest.is_contiguous and src.is_contiguous):
        # wrapped operands: one pass of the broadcast kernel with the strides in the descriptors
        if dest.dims != src.dims:
            raise ValueError("copyto! between strided arrays needs equal shapes")
        from .broadcast import Broadcasted, materialize_
        materialize_(dest, Broadcasted.leaf(src), stream)
        return dest
    if dest.size:
        st = with_managed(stream or current_stream(), dest, src)
        check(lib.b200_memcpy_async(C.c_void_p(dest.ptr), C.c_void_p(src.ptr), src.nbytes, st.handle))
    return dest


def zeros(dtype, dims) -> ROCArray:
    """``AMDGPU.zeros`` (src/array.jl:358-359)."""
    return ROCArray(dtype, dims).fill_(0)


def ones(dtype, dims) -> ROCArray:
    """``AMDGPU.ones`` (src/array.jl:360-361)."""
    return ROCArray(dtype, dims).fill_(1)


def fill(value, dims, dtype=None) -> ROCArray:
    """``AMDGPU.fill`` (src/array.jl:362-363)."""
    return ROCArray(np.asarray(value).dtype if dtype is None else dtype, dims).fill_(value)


def roc(a) -> ROCArray:
    """``roc(x)`` (src/array.jl:351): upload, Float64 arrays become Float32."""
    a = np.asarray(a)
    if a.dtype == np.float64:
        a = a.astype(np.float32)
    return ROCArray.from_host(a)
