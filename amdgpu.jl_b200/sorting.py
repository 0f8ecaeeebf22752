"""``sort!`` / ``sort`` / ``sortperm!`` / ``sortperm``.

Mirrors src/kernels/sorting.jl:1-3 of the reference.  The order is ``Base.isless`` (NaN last,
-0.0 before +0.0); ``sortperm`` yields a stable, 1-based ``Int64`` permutation; ``rev=True``
sorts under the reversed ordering, so equal keys keep their input order.

The reference's tests also pass ``lt`` and ``by`` (test/hip_rocarray/sorting.jl:20-26:
``lt=!isless``, ``by=k -> 2k``).  A radix sort cannot call closures, so here

* ``by`` is any function that maps the lazy operand to an expression over the broadcast
  operator set (``lambda k: 2 * k``, ``abs``, ``lambda k: -k`` ...): the keys ``by.(x)`` are
  materialised with one fused kernel, ``sortperm`` runs on them, and the values follow through a
  gather;
* ``lt`` is one of the names ``"isless"`` (default), ``"<"``, ``">"``, ``"!isless"``; the last two
  sort under the reversed ordering (for distinct keys that is what Base produces; ties, where
  ``!isless`` is not a strict order, come out in the stable order of ``rev=true``).

Anything else raises (no CPU fallback).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib
from .array import ROCArray, copyto_, with_managed
from .runtime import Stream, current_stream

_LT_REVERSED = {None: False, "isless": False, "<": False, ">": True, "!isless": True}


def _order(rev: bool, lt) -> bool:
    if callable(lt):
        raise ValueError("sort on the B200 backend takes `lt` by name: 'isless', '<', '>' or '!isless'")
    if lt not in _LT_REVERSED:
        raise ValueError(f"unsupported `lt` {lt!r}: use 'isless', '<', '>' or '!isless'")
    return bool(rev) != _LT_REVERSED[lt]


def _keys(x: ROCArray, by, stream: Stream) -> ROCArray:
    """``by.(x)`` as a dense device vector (`x` itself when `by` is the identity)."""
    if by is None:
        return x if x.is_contiguous else x.copy(stream)
    from .broadcast import Broadcasted
    expr = by(x.dot)
    if not isinstance(expr, Broadcasted):
        raise ValueError("`by` must map the lazy operand to a broadcast expression (e.g. lambda k: 2 * k)")
    return expr.materialize(stream)


def _gather(x: ROCArray, ix: ROCArray, stream: Stream | None = None) -> ROCArray:
    from .indexing import getindex
    return getindex(x, ix, stream)


def sort_(x: ROCArray, rev: bool = False, lt=None, by=None, stream: Stream | None = None) -> ROCArray:
    """``Base.sort!(x; rev, lt, by)`` (src/kernels/sorting.jl:1): in place, returns `x`."""
    if x.ndim != 1:
        raise ValueError("sort! needs a vector")
    rev = _order(rev, lt)
    st = stream or current_stream()
    if by is not None:
        perm = sortperm_(ROCArray(np.int64, x.dims, stream=st), x, rev=rev, by=by, stream=st)
        return copyto_(x, _gather(x if x.is_contiguous else x.copy(st), perm, st), st)
    xd = x if x.is_contiguous else x.copy(st)
    t = xd.tensor()
    with_managed(st, xd)
    check(lib.b200_sort(st.handle, C.byref(t), 1 if rev else 0))
    if xd is not x:
        copyto_(x, xd, st)
    return x


def sort(x: ROCArray, rev: bool = False, lt=None, by=None) -> ROCArray:
    """``Base.sort(x)`` = ``sort!(copy(x))``."""
    return sort_(x.copy(), rev=rev, lt=lt, by=by)


def sortperm_(ix: ROCArray, x: ROCArray, rev: bool = False, lt=None, by=None, stream: Stream | None = None) -> ROCArray:
    """``Base.sortperm!(ix, x; rev, lt, by)`` (src/kernels/sorting.jl:2); `x` is left untouched."""
    if ix.dtype != np.int64:
        raise ValueError("sortperm! needs an Int64 index vector")
    if x.ndim != 1 or ix.dims != x.dims:
        raise ValueError("sortperm!: index and key vectors must have the same length")
    if not ix.is_contiguous:
        raise ValueError("sortperm!: the index vector must be dense")
    rev = _order(rev, lt)
    st = stream or current_stream()
    keys = _keys(x, by, st)
    ti, tx = ix.tensor(), keys.tensor()
    with_managed(st, ix, keys)
    check(lib.b200_sortperm(st.handle, C.byref(ti), C.byref(tx), 1 if rev else 0))
    return ix


def sortperm(x: ROCArray, rev: bool = False, lt=None, by=None) -> ROCArray:
    """``Base.sortperm(x)`` (src/kernels/sorting.jl:3).  The reference uploads ``1:length(x)``;
    here the first radix pass generates the indices on the device."""
    return sortperm_(ROCArray(np.int64, x.dims), x, rev=rev, lt=lt, by=by)
