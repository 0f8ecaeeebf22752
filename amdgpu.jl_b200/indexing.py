"""``findall`` / logical indexing and ``reverse``.

Mirrors src/kernels/indexing.jl:8-36 (``findall(bools)`` = cumsum of the mask, read its last
element on the host, scatter the indices; ``xs[bools]``) and src/kernels/reverse.jl:59-122
(``reverse`` / ``reverse!`` along ``dims``).  ``findall`` of an N-d mask returns 1-based LINEAR
indices in column-major order (the reference returns the equivalent ``CartesianIndex`` values).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib
from .accumulate import accumulate_
from .array import ROCArray, copyto_, with_managed
from .broadcast import Broadcasted, materialize_
from .runtime import Stream, current_stream


def _positions(bools: ROCArray, stream: Stream):
    if bools.dtype != np.bool_:
        raise TypeError("the mask must be a Bool array")
    flat = bools.reshape(bools.size)
    # positions fit Int32 below 2^31 entries: half the traffic of the scan and of the compaction
    wide = flat.size >= (1 << 31) - 1
    as_int = ROCArray(np.int64 if wide else np.int32, flat.dims, stream=stream)
    code = bytes((0, 0, 1, 7 if wide else 6))       # LEAF 0, CONVERT -> Int64 / Int32
    leaves = Broadcasted.leaf(flat).flatten()[1]
    t = as_int.tensor()
    with_managed(stream, as_int, flat)
    check(lib.b200_broadcast(stream.handle, C.byref(t), leaves, 1, code, 2))
    idx = accumulate_("+", as_int, as_int, init=None, stream=stream)
    n = int(idx.view(idx.size - 1, idx.size).to_host(stream)[0]) if idx.size else 0     # blocking read, like indices[end]
    return flat, idx, n


def findall(bools: ROCArray, stream: Stream | None = None) -> ROCArray:
    """``findall(bools)`` (src/kernels/indexing.jl:8-36)."""
    st = stream or current_stream()
    flat, idx, n = _positions(bools, st)
    ys = ROCArray(np.int64, (n,), stream=st)
    if n:
        ty, tb, ti = ys.tensor(), flat.tensor(), idx.tensor()
        with_managed(st, ys, flat, idx)
        check(lib.b200_compact(st.handle, C.byref(ty), C.byref(tb), C.byref(ti), None))
    idx.unsafe_free_()
    return ys


def getindex_mask(xs: ROCArray, bools: ROCArray, stream: Stream | None = None) -> ROCArray:
    """``xs[bools]`` (logical indexing, src/kernels/indexing.jl:1-6)."""
    if xs.size != bools.size:
        raise IndexError("mask and array differ in length")
    st = stream or current_stream()
    flat, idx, n = _positions(bools, st)
    ys = ROCArray(xs.dtype, (n,), stream=st)
    if n:
        ty, tb, ti, tv = ys.tensor(), flat.tensor(), idx.tensor(), xs.reshape(xs.size).tensor()
        with_managed(st, ys, flat, idx, xs)
        check(lib.b200_compact(st.handle, C.byref(ty), C.byref(tb), C.byref(ti), C.byref(tv)))
    idx.unsafe_free_()
    return ys


def getindex_mask_dim(xs: ROCArray, bools: ROCArray, dim: int, stream: Stream | None = None) -> ROCArray:
    """``xs[:, ..., bools, ..., :]``: a Bool vector selects along dimension `dim` (1-based), colons
    everywhere else (test/hip_rocarray/indexing.jl:9-18: ``xd[:, md]``, ``xd[:, :, md]``).  The kept
    positions come from ``findall`` (a scan + compaction); the linear indices of all selected
    elements are then formed by one fused broadcast over (leading, selected, trailing) and read
    with the gather kernel - everything stays on the device except the count ``findall`` reads."""
    if not 1 <= dim <= xs.ndim:
        raise IndexError(f"dimension {dim} out of range for an array with {xs.ndim} dimensions")
    if bools.ndim != 1 or bools.size != xs.dims[dim - 1]:
        raise IndexError("the mask must be a vector as long as the dimension it selects from")
    st = stream or current_stream()
    keep = findall(bools, st)                              # 1-based positions along `dim`
    k = keep.size
    lead = int(np.prod(xs.dims[:dim - 1], dtype=np.int64))
    extent = xs.dims[dim - 1]
    trail = int(np.prod(xs.dims[dim:], dtype=np.int64))
    out_dims = xs.dims[:dim - 1] + (k,) + xs.dims[dim:]
    if k == 0 or lead == 0 or trail == 0:
        return ROCArray(xs.dtype, out_dims, stream=st)
    def iota(n):                                           # 1, 2, ..., n as Int64 on the device
        return accumulate_("+", ROCArray(np.int64, (n,), stream=st), ROCArray(np.int64, (n,), stream=st).fill_(1, st), init=None, stream=st)
    a = iota(lead).reshape(lead, 1, 1)
    j = keep.reshape(1, k, 1)
    m = iota(trail).reshape(1, 1, trail)
    # 1-based linear index of element (a, j, m):  a + lead*(j-1) + lead*extent*(m-1)
    expr = a.dot + (j.dot - 1) * lead + (m.dot - 1) * (lead * extent)
    idx = expr.materialize(st)
    xd = xs if xs.is_contiguous else xs.copy(st)
    return getindex(xd, idx.reshape(idx.size), st).reshape(out_dims)


def getindex(xs: ROCArray, ix: ROCArray, stream: Stream | None = None) -> ROCArray:
    """``xs[ix]`` with a device vector of 1-based integer indices (the vectorised ``getindex`` the
    reference's sorting tests use, test/hip_rocarray/sorting.jl:14).  `xs` is indexed linearly;
    an out-of-range index surfaces as an error at the next synchronisation."""
    if ix.dtype not in (np.dtype(np.int64), np.dtype(np.int32)):
        raise ValueError("index vectors must be Int64 or Int32")
    st = stream or current_stream()
    xd = xs if xs.is_contiguous else xs.copy(st)
    ixd = ix if ix.is_contiguous else ix.copy(st)
    out = ROCArray(xs.dtype, ix.dims, stream=st)
    ty, tx, ti = out.tensor(), xd.tensor(), ixd.tensor()
    with_managed(st, out, xd, ixd)
    check(lib.b200_gather(st.handle, C.byref(ty), C.byref(tx), C.byref(ti)))
    return out


def _mask(x: ROCArray, dims) -> int:
    if dims is None:
        dims = range(1, x.ndim + 1)
    elif isinstance(dims, (int, np.integer)):
        dims = (int(dims),)
    m = 0
    for d in dims:
        if not 1 <= d <= max(1, x.ndim):
            raise ValueError(f"dimension out of range: {d}")
        m |= 1 << (d - 1)
    return m


def reverse(x: ROCArray, dims=None, stream: Stream | None = None) -> ROCArray:
    """``reverse(x; dims)`` (src/kernels/reverse.jl:91-100): out of place."""
    st = stream or current_stream()
    y = x.similar(stream=st)
    ty, tx = y.tensor(), x.tensor()
    with_managed(st, y, x)
    check(lib.b200_reverse(st.handle, C.byref(ty), C.byref(tx), _mask(x, dims)))
    return y


def reverse_(x: ROCArray, dims=None, stream: Stream | None = None) -> ROCArray:
    """``reverse!(x; dims)`` (src/kernels/reverse.jl:102-122); goes through a device copy."""
    st = stream or current_stream()
    tmp = x.copy(st)
    tx, tt = x.tensor(), tmp.tensor()
    with_managed(st, x, tmp)
    check(lib.b200_reverse(st.handle, C.byref(tx), C.byref(tt), _mask(x, dims)))
    tmp.unsafe_free_()
    return x
