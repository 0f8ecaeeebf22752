"""``accumulate!`` / ``accumulate`` / ``cumsum`` / ``cumprod``.

Mirrors src/kernels/accumulate.jl:1-8 of the reference: ``accumulate`` defaults to
``init = zero(eltype(A))``, the element type is preserved (no widening, unlike Base's
``cumsum`` on small integers), and the keywords seen in the reference's tests are ``init`` and
``dims`` (test/core/rocarray_base.jl:194-225).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib
from .array import ROCArray, copyto_, with_managed
from .mapreduce import _op_code
from .runtime import Stream, current_stream

_ZERO = object()


def accumulate_(op, B: ROCArray, A: ROCArray, init=_ZERO, dims=None, inclusive: bool = True,
                stream: Stream | None = None) -> ROCArray:
    """``Base.accumulate!(op, B, A; init, dims)``: B[i] = op(B[i-1], A[i]), seeded by `init`.
    `dims` is 1-based; vectors default to their only dimension."""
    if B.dims != A.dims or B.dtype != A.dtype:
        raise ValueError("accumulate!: source and destination must have the same size and element type")
    if dims is None:
        if A.ndim > 1:
            raise ValueError("accumulate over an N-dimensional array needs `dims`")
        dims = 1
    if dims < 1:
        raise ValueError("dims is 1-based")
    if init is _ZERO:
        init = A.dtype.type(0)
    init_buf = None if init is None else np.asarray(init, dtype=A.dtype).tobytes()
    # the scan kernels want dense operands: wrapped ones (views, permuted dims) go through a dense
    # temporary, one strided copy in and one out
    st = stream or current_stream()
    Ad = A if A.is_contiguous else A.copy(st)
    Bd = B if B.is_contiguous else B.similar(stream=st)
    tb, ta = Bd.tensor(), Ad.tensor()
    with_managed(st, Bd, Ad)
    check(lib.b200_accumulate(st.handle, C.byref(tb), C.byref(ta), _op_code(op),
                              init_buf, dims - 1, 1 if inclusive else 0))
    if Bd is not B:
        copyto_(B, Bd, stream)
    return B


def accumulate(op, A: ROCArray, init=_ZERO, dims=None) -> ROCArray:
    """``Base.accumulate(op, A; init, dims)`` (src/kernels/accumulate.jl:4-5)."""
    return accumulate_(op, A.similar(), A, init=init, dims=dims)


def cumsum(A: ROCArray, dims=None) -> ROCArray:
    """``Base.cumsum`` (src/kernels/accumulate.jl:7)."""
    return accumulate_("+", A.similar(), A, init=A.dtype.type(0), dims=dims)


def cumprod(A: ROCArray, dims=None) -> ROCArray:
    """``Base.cumprod`` (src/kernels/accumulate.jl:8)."""
    return accumulate_("*", A.similar(), A, init=A.dtype.type(1), dims=dims)


def prepared(op, B: ROCArray, A: ROCArray, init=_ZERO, dims: int = 1, stream: Stream | None = None):
    """``accumulate!`` with the descriptor work done once; returns a zero-argument callable."""
    if init is _ZERO:
        init = A.dtype.type(0)
    init_buf = None if init is None else np.asarray(init, dtype=A.dtype).tobytes()
    tb, ta = B.tensor(), A.tensor()
    st = stream or current_stream()
    fn, opc = lib.b200_accumulate, _op_code(op)

    def launch(_keep=(A, B, st)):
        with_managed(st, B, A)
        check(fn(st.handle, C.byref(tb), C.byref(ta), opc, init_buf, dims - 1, 1))
    return launch
