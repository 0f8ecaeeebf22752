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

import numpy as np

from . import _lib
from ._lib import check, lib
from .memory import pool_alloc, pool_free
from .runtime import Stream, current_stream


class _Managed:
    """Reference-counted device buffer tied to the stream that owns it (the role of
    ``Managed`` + ``DataRef``, src/memory.jl:408-418)."""

    __slots__ = ("ptr", "nbytes", "stream", "freed", "__weakref__")

    def __init__(self, nbytes: int, stream: Stream):
        self.ptr, self.freed = 0, True          # a failed allocation must leave a harmless object
        self.nbytes = nbytes
        self.stream = stream
        self.ptr = pool_alloc(nbytes, stream)
        self.freed = False

    def free(self) -> None:
        if not self.freed and self.ptr:
            self.freed = True
            try:
                st = self.stream if self.stream.handle is not None else current_stream()
                pool_free(self.ptr, st)   # stale owner: fall back to the current stream (src/memory.jl:531-536)
            except Exception:
                pass

    def __del__(self):
        self.free()


class ROCArray:
    __array_ufunc__ = None      # never let NumPy treat a device array as an object scalar

    def __init__(self, dtype, dims, *, _buf: _Managed | None = None, _offset: int = 0, stream: Stream | None = None):
        """``ROCArray{T}(undef, dims)`` (src/array.jl:24-32): uninitialised storage from the pool."""
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
    @property
    def strides(self):
        s, acc = [], 1
        for d in self.dims:
            s.append(acc)
            acc *= d
        return tuple(s)
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
        flat = np.ascontiguousarray(a.reshape(-1, order="F"))
        st = stream or current_stream()
        if flat.nbytes:
            check(lib.b200_memcpy_async(C.c_void_p(self.ptr), C.c_void_p(flat.ctypes.data), flat.nbytes, st.handle))
            st.synchronize()   # pageable source must stay alive until the copy is done
        return self

    def to_host(self, stream: Stream | None = None) -> np.ndarray:
        """``Array(x::ROCArray)`` (src/array.jl:215-227): blocking download."""
        out = np.empty(self.size, dtype=self.dtype)
        st = stream or current_stream()
        if out.nbytes:
            check(lib.b200_memcpy_async(C.c_void_p(out.ctypes.data), C.c_void_p(self.ptr), out.nbytes, st.handle))
        st.synchronize()
        return out.reshape(self.dims, order="F")

    def item(self):
        if self.size != 1:
            raise ValueError("item() needs exactly one element")
        return self.to_host().reshape(-1)[0]

    def similar(self, dtype=None, dims=None) -> "ROCArray":
        """``similar(A, T, dims)`` (src/array.jl:109)."""
        return ROCArray(self.dtype if dtype is None else dtype, self.dims if dims is None else dims,
                        stream=self.buf.stream)

    def copy(self) -> "ROCArray":
        """``copy(A)`` (src/array.jl:268-272): device-to-device."""
        out = self.similar()
        copyto_(out, self)
        return out

    def reshape(self, *dims) -> "ROCArray":
        """``reshape`` shares the buffer (``derive``, src/array.jl:111-115)."""
        if len(dims) == 1 and not isinstance(dims[0], (int, np.integer)):
            dims = tuple(dims[0])
        if math.prod(dims) != self.size:
            raise ValueError("reshape: total size must not change")
        return ROCArray(self.dtype, dims, _buf=self.buf, _offset=self.offset)

    def view(self, start: int, stop: int) -> "ROCArray":
        """Contiguous 1-D view ``@view A[start+1:stop]`` of the linear index space; the result's
        pointer is ``base + offset`` and need not be 16-byte aligned (src/array.jl:353-354)."""
        if not 0 <= start <= stop <= self.size:
            raise IndexError("view out of range")
        return ROCArray(self.dtype, (stop - start,), _buf=self.buf, _offset=self.offset + start * self.itemsize)

    def reinterpret(self, dtype) -> "ROCArray":
        dtype = np.dtype(dtype)
        if self.nbytes % dtype.itemsize:
            raise ValueError("reinterpret: size is not a multiple of the new element size")
        return ROCArray(dtype, (self.nbytes // dtype.itemsize,), _buf=self.buf, _offset=self.offset)

    def fill_(self, value, stream: Stream | None = None) -> "ROCArray":
        """``fill!(A, x)`` as a bit-pattern memset (src/array.jl:253-266)."""
        if self.size:
            bits = int.from_bytes(np.asarray(value, dtype=self.dtype).tobytes().ljust(8, b"\0"), "little")
            check(lib.b200_memset_async(C.c_void_p(self.ptr), bits, self.itemsize, self.size,
                                        (stream or current_stream()).handle))
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
    if dest.size:
        check(lib.b200_memcpy_async(C.c_void_p(dest.ptr), C.c_void_p(src.ptr), src.nbytes,
                                    (stream or current_stream()).handle))
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
