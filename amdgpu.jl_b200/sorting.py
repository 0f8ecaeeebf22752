"""``sort!`` / ``sort`` / ``sortperm!`` / ``sortperm``.

Mirrors src/kernels/sorting.jl:1-3 of the reference.  The order is ``Base.isless`` (NaN last,
-0.0 before +0.0); ``sortperm`` yields a stable, 1-based ``Int64`` permutation; ``rev=True``
sorts under the reversed ordering, so equal keys keep their input order.  The reference's
tests also pass ``lt`` / ``by`` closures (test/hip_rocarray/sorting.jl:20-26); a radix sort
cannot honour arbitrary closures, so only the defaults are accepted and anything else raises
(no CPU fallback).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib
from .array import ROCArray
from .runtime import Stream, current_stream


def _check_kwargs(lt, by):
    if lt is not None or by is not None:
        raise ValueError("sort on the B200 backend supports the default `lt=isless` and `by=identity` only")


def sort_(x: ROCArray, rev: bool = False, lt=None, by=None, stream: Stream | None = None) -> ROCArray:
    """``Base.sort!(x; rev)`` (src/kernels/sorting.jl:1): in place, returns `x`."""
    _check_kwargs(lt, by)
    if x.ndim != 1:
        raise ValueError("sort! needs a vector")
    t = x.tensor()
    check(lib.b200_sort((stream or current_stream()).handle, C.byref(t), 1 if rev else 0))
    return x


def sort(x: ROCArray, rev: bool = False, lt=None, by=None) -> ROCArray:
    """``Base.sort(x)`` = ``sort!(copy(x))``."""
    return sort_(x.copy(), rev=rev, lt=lt, by=by)


def sortperm_(ix: ROCArray, x: ROCArray, rev: bool = False, lt=None, by=None, stream: Stream | None = None) -> ROCArray:
    """``Base.sortperm!(ix, x; rev)`` (src/kernels/sorting.jl:2); `x` is left untouched."""
    _check_kwargs(lt, by)
    if ix.dtype != np.int64:
        raise ValueError("sortperm! needs an Int64 index vector")
    if x.ndim != 1 or ix.dims != x.dims:
        raise ValueError("sortperm!: index and key vectors must have the same length")
    ti, tx = ix.tensor(), x.tensor()
    check(lib.b200_sortperm((stream or current_stream()).handle, C.byref(ti), C.byref(tx), 1 if rev else 0))
    return ix


def sortperm(x: ROCArray, rev: bool = False, lt=None, by=None) -> ROCArray:
    """``Base.sortperm(x)`` (src/kernels/sorting.jl:3).  The reference uploads ``1:length(x)``;
    here the first radix pass generates the indices on the device."""
    return sortperm_(ROCArray(np.int64, x.dims), x, rev=rev, lt=lt, by=by)
