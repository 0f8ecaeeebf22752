"""``mapreducedim!`` and the reductions built on it.

Mirrors GPUArrays.mapreducedim! as implemented in src/kernels/mapreduce.jl:86-173 of the
reference: reduced dimensions are those where ``size(R, d) == 1``; `A` may be an array or a
``Broadcasted`` tree (:88); an empty `A` returns `R` untouched (:91); ``init=None`` means `R`
already holds the operator's neutral element (:60); the same `R` object is returned (:93,172).
``mapreduce`` / ``sum`` / ``prod`` / ``maximum`` / ``minimum`` follow Base: small integers
widen to 64 bits under ``+`` and ``*`` (``Base.add_sum``), floats keep their type (16-bit
floats accumulate in Float32 inside the kernel), and reducing an empty collection with
``max`` / ``min`` raises.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, lib
from .array import ROCArray, with_managed
from .broadcast import Broadcasted
from .runtime import Stream, current_stream

_OPS = {"+": _lib.RED_ADD, "add": _lib.RED_ADD, "*": _lib.RED_MUL, "mul": _lib.RED_MUL,
        "max": _lib.RED_MAX, "min": _lib.RED_MIN}


def _op_code(op) -> int:
    if isinstance(op, str) and op in _OPS:
        return _OPS[op]
    import operator
    table = {operator.add: _lib.RED_ADD, operator.mul: _lib.RED_MUL, max: _lib.RED_MAX, min: _lib.RED_MIN,
             np.add: _lib.RED_ADD, np.multiply: _lib.RED_MUL, np.maximum: _lib.RED_MAX, np.minimum: _lib.RED_MIN}
    if op in table:
        return table[op]
    raise ValueError(f"reduction operator {op!r} is not supported (use +, *, max, min); no CPU fallback exists")


def _apply_f(f, A) -> Broadcasted:
    node = Broadcasted.leaf(A)
    if f is None or f == "identity":
        return node
    if isinstance(f, str):
        return Broadcasted.call(f, node)
    if f is abs:
        return Broadcasted.call("abs", node)
    out = f(node)   # a callable written against Broadcasted operands, e.g. lambda x: x * x + 1
    if not isinstance(out, Broadcasted):
        raise TypeError("the mapped function must return a broadcast expression")
    return out


def mapreducedim_(f, op, R: ROCArray, A, init=None, stream: Stream | None = None) -> ROCArray:
    """``GPUArrays.mapreducedim!(f, op, R, A; init)`` (src/kernels/mapreduce.jl:86-173)."""
    expr = _apply_f(f, A)
    shape = expr.shape()
    rdims = R.dims + (1,) * (len(shape) - R.ndim)
    if len(rdims) != len(shape) or any(r != s and r != 1 for r, s in zip(rdims, shape)):
        raise ValueError(f"DimensionMismatch: cannot reduce an array of size {shape} into one of size {R.dims}")
    if int(np.prod(shape, dtype=np.int64)) == 0:
        return R
    code, leaves, nleaves, keep = expr.flatten()
    shp = (C.c_int64 * max(1, len(shape)))(*shape)
    t = R.tensor()
    init_buf = None
    if init is not None:
        init_buf = np.asarray(init, dtype=R.dtype).tobytes()
    st = with_managed(stream or current_stream(), R, *keep)
    check(lib.b200_mapreduce(st.handle, C.byref(t), shp, len(shape), leaves, nleaves,
                             code, len(code) // 2, _op_code(op), init_buf))
    return R


def prepared(f, op, R: ROCArray, A, init=None, stream: Stream | None = None):
    """``mapreducedim!`` with the descriptor work done once; returns a zero-argument callable."""
    expr = _apply_f(f, A)
    shape = expr.shape()
    code, leaves, nleaves, keep = expr.flatten()
    shp = (C.c_int64 * max(1, len(shape)))(*shape)
    t = R.tensor()
    init_buf = None if init is None else np.asarray(init, dtype=R.dtype).tobytes()
    st = stream or current_stream()
    fn, ninstr, opc, nd = lib.b200_mapreduce, len(code) // 2, _op_code(op), len(shape)

    def launch(_keep=(keep, R, st)):
        with_managed(st, R, *keep)
        check(fn(st.handle, C.byref(t), shp, nd, leaves, nleaves, code, ninstr, opc, init_buf))
    return launch


def precompile(f, op, R: ROCArray, A) -> bool:
    """Compiles the kernel ``mapreducedim!(f, op, R, A)`` would need, without launching anything
    (no device needed).  False when the run-time compiler is unavailable."""
    expr = _apply_f(f, A)
    shape = expr.shape()
    code, leaves, nleaves, _keep = expr.flatten()
    shp = (C.c_int64 * max(1, len(shape)))(*shape)
    t = R.tensor()
    return lib.b200_mapreduce_prepare(C.byref(t), shp, len(shape), leaves, nleaves, code, len(code) // 2, _op_code(op)) == 0


def _result_dtype(expr_dtype: int, opc: int) -> np.dtype:
    # Base.add_sum / mul_prod widen small integers; everything else keeps the mapped type.
    if opc in (_lib.RED_ADD, _lib.RED_MUL):
        if expr_dtype in (_lib.I8, _lib.I16, _lib.I32, _lib.BOOL):
            return np.dtype(np.int64)
        if expr_dtype in (_lib.U8, _lib.U16, _lib.U32):
            return np.dtype(np.uint64)
    return _lib.dtype_numpy(expr_dtype)


def _neutral(opc: int, dt: np.dtype):
    if opc == _lib.RED_ADD:
        return dt.type(0)
    if opc == _lib.RED_MUL:
        return dt.type(1)
    if dt.kind == "f" or dt.name == "bfloat16":
        return dt.type(-np.inf if opc == _lib.RED_MAX else np.inf)
    info = np.iinfo(dt)
    return dt.type(info.min if opc == _lib.RED_MAX else info.max)


def mapreduce(f, op, A, dims=None, init=None):
    """``mapreduce(f, op, A; dims, init)``.  Without `dims` the scalar result is copied to the
    host (a blocking read, like ``Array(R)[]`` in the reference, src/array.jl:215-227); with
    `dims` (1-based, int or tuple) a ROCArray with singleton reduced dimensions is returned."""
    opc = _op_code(op)
    expr = _apply_f(f, A)
    shape = expr.shape()
    n = int(np.prod(shape, dtype=np.int64))
    out_dt = _result_dtype(expr.dtype, opc)
    if dims is None:
        rshape = (1,) * len(shape)
    else:
        ds = (dims,) if isinstance(dims, (int, np.integer)) else tuple(dims)
        if any(d < 1 for d in ds):
            raise ValueError("dims are 1-based")
        rshape = tuple(1 if (i + 1) in ds else s for i, s in enumerate(shape))
    if n == 0 and opc in (_lib.RED_MAX, _lib.RED_MIN) and init is None:
        raise ValueError("reducing over an empty collection is not allowed; consider supplying `init`")
    R = ROCArray(out_dt, rshape)
    seed = _neutral(opc, out_dt) if init is None else init
    if n == 0:
        R.fill_(seed)
    else:
        mapreducedim_(lambda _: expr, op, R, A if not isinstance(A, Broadcasted) else A, init=seed)
    if dims is None:
        return R.to_host().reshape(-1)[0]
    return R


def sum(A, dims=None, f=None, init=None):      # noqa: A001 - mirrors Base.sum
    return mapreduce(f, "+", A, dims=dims, init=init)


def prod(A, dims=None, f=None, init=None):
    return mapreduce(f, "*", A, dims=dims, init=init)


def maximum(A, dims=None, f=None, init=None):
    return mapreduce(f, "max", A, dims=dims, init=init)


def minimum(A, dims=None, f=None, init=None):
    return mapreduce(f, "min", A, dims=dims, init=init)
