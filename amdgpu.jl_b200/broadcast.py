"""Lazy fused broadcast: builds a ``Broadcasted`` tree and hands it to the library as one
postfix program.

Mirrors the reference's division of labour: src/broadcast.jl:3-35 only chooses the style,
merges it and allocates the result with ``similar``; the fused kernel is produced elsewhere.
Here the tree is flattened with Julia's promotion rules applied per node (``promote_type``),
so mixed element types compute exactly as ``Base.Broadcast`` would: the operands of a node
are converted to the node's type before the operation.  Supported calls: ``+ - * /``,
``muladd``, ``abs``, ``abs2``, ``exp``, ``max``, ``min``, unary minus; anything else raises
(there is no CPU fallback).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, lib
from .array import ROCArray, with_managed
from .runtime import Stream, current_stream

_FLOATS = (_lib.F16, _lib.BF16, _lib.F32, _lib.F64)
_SIGNED = (_lib.I8, _lib.I16, _lib.I32, _lib.I64)
_UNSIGNED = (_lib.U8, _lib.U16, _lib.U32, _lib.U64)
_BYTES = {_lib.F16: 2, _lib.BF16: 2, _lib.F32: 4, _lib.F64: 8, _lib.I8: 1, _lib.I16: 2, _lib.I32: 4, _lib.I64: 8,
          _lib.U8: 1, _lib.U16: 2, _lib.U32: 4, _lib.U64: 8, _lib.BOOL: 1}


def promote_type(a: int, b: int) -> int:
    """``Base.promote_type`` restricted to the supported element types."""
    if a == b:
        return a
    if a == _lib.BOOL:
        return b
    if b == _lib.BOOL:
        return a
    fa, fb = a in _FLOATS, b in _FLOATS
    if fa and fb:
        if {a, b} == {_lib.F16, _lib.BF16}:
            return _lib.F32
        return a if _BYTES[a] >= _BYTES[b] else b
    if fa:
        return a
    if fb:
        return b
    # integers: the wider one wins; equal widths give the unsigned type
    if _BYTES[a] != _BYTES[b]:
        return a if _BYTES[a] > _BYTES[b] else b
    return a if a in _UNSIGNED else b


def _float_of(dt: int) -> int:
    return dt if dt in _FLOATS else _lib.F64


def _arith_of(dt: int) -> int:
    return _lib.I64 if dt == _lib.BOOL else dt


_UNARY = {"abs": _lib.OP_ABS, "abs2": _lib.OP_ABS2, "exp": _lib.OP_EXP, "neg": _lib.OP_NEG}
_BINARY = {"add": _lib.OP_ADD, "sub": _lib.OP_SUB, "mul": _lib.OP_MUL, "div": _lib.OP_DIV,
           "max": _lib.OP_MAX, "min": _lib.OP_MIN}


class Broadcasted:
    """A node of a lazily fused elementwise expression."""

    __slots__ = ("op", "args", "value", "dtype")
    # NumPy scalars must defer to our reflected operators (np.float32(2.5) * x.dot keeps Float32)
    __array_ufunc__ = None

    def __init__(self, op, args=(), value=None, dtype=None):
        self.op, self.args, self.value, self.dtype = op, args, value, dtype

    # ---- leaves
    @staticmethod
    def leaf(x) -> "Broadcasted":
        if isinstance(x, Broadcasted):
            return x
        if isinstance(x, ROCArray):
            return Broadcasted("array", value=x, dtype=_lib.dtype_code(x.dtype))
        if isinstance(x, (bool, np.bool_)):
            return Broadcasted("scalar", value=np.bool_(x), dtype=_lib.BOOL)
        if isinstance(x, (int,)):
            return Broadcasted("scalar", value=np.int64(x), dtype=_lib.I64)     # Julia Int literal
        if isinstance(x, float):
            return Broadcasted("scalar", value=np.float64(x), dtype=_lib.F64)   # Julia Float64 literal
        if isinstance(x, np.generic):
            return Broadcasted("scalar", value=x, dtype=_lib.dtype_code(x.dtype))
        if isinstance(x, np.ndarray) and x.ndim == 0:
            return Broadcasted.leaf(x[()])
        raise TypeError(f"cannot broadcast over {type(x).__name__}: only ROCArray and scalars are device-compatible")

    # ---- nodes with Julia's result types
    @staticmethod
    def call(name: str, *args) -> "Broadcasted":
        a = [Broadcasted.leaf(x) for x in args]
        if name in _UNARY:
            (x,) = a
            dt = _float_of(_arith_of(x.dtype)) if name == "exp" else _arith_of(x.dtype)
            return Broadcasted(name, (x,), dtype=dt)
        if name in _BINARY:
            x, y = a
            dt = _arith_of(promote_type(x.dtype, y.dtype))
            if name == "div":
                dt = _float_of(dt)
            return Broadcasted(name, (x, y), dtype=dt)
        if name == "muladd":
            x, y, z = a
            dt = _arith_of(promote_type(promote_type(x.dtype, y.dtype), z.dtype))
            return Broadcasted(name, (x, y, z), dtype=dt)
        if name == "identity":
            return a[0]
        raise ValueError(f"function `{name}` is outside the supported broadcast operator set "
                         "(+ - * / muladd abs abs2 exp max min); no CPU fallback exists")

    def __add__(self, o): return Broadcasted.call("add", self, o)
    def __radd__(self, o): return Broadcasted.call("add", o, self)
    def __sub__(self, o): return Broadcasted.call("sub", self, o)
    def __rsub__(self, o): return Broadcasted.call("sub", o, self)
    def __mul__(self, o): return Broadcasted.call("mul", self, o)
    def __rmul__(self, o): return Broadcasted.call("mul", o, self)
    def __truediv__(self, o): return Broadcasted.call("div", self, o)
    def __rtruediv__(self, o): return Broadcasted.call("div", o, self)
    def __neg__(self): return Broadcasted.call("neg", self)
    def __abs__(self): return Broadcasted.call("abs", self)

    # ---- shape
    def shape(self) -> tuple:
        """``Broadcast.combine_axes``: extents must match or be 1."""
        if self.op == "array":
            return self.value.dims
        if self.op == "scalar":
            return ()
        out: list[int] = []
        for a in self.args:
            s = a.shape()
            for d, e in enumerate(s):
                if d >= len(out):
                    out.append(e)
                elif out[d] != e:
                    if out[d] == 1:
                        out[d] = e
                    elif e != 1:
                        raise ValueError(f"DimensionMismatch: arrays could not be broadcast to a common size; "
                                         f"got a dimension with lengths {out[d]} and {e}")
        return tuple(out)

    # ---- flattening
    def flatten(self):
        """Postfix program + leaf table for the C ABI."""
        code: list[int] = []
        leaves: list[Broadcasted] = []

        def leaf_index(n: "Broadcasted") -> int:
            for i, l in enumerate(leaves):
                if l.op == n.op and l.dtype == n.dtype and (
                        l.value is n.value or (n.op == "scalar" and l.value.tobytes() == n.value.tobytes())):
                    return i
            leaves.append(n)
            return len(leaves) - 1

        def emit(n: "Broadcasted", want: int):
            if n.op in ("array", "scalar"):
                code.extend((_lib.OP_LEAF, leaf_index(n)))
            else:
                for a in n.args:
                    emit(a, n.dtype)
                opc = _UNARY.get(n.op) or _BINARY.get(n.op) or _lib.OP_MULADD
                code.extend((opc, n.dtype))
            if n.dtype != want:
                code.extend((_lib.OP_CONVERT, want))

        emit(self, self.dtype)
        if len(leaves) > _lib.MAX_LEAVES:
            raise ValueError(f"broadcast expressions may reference at most {_lib.MAX_LEAVES} distinct operands")
        if len(code) // 2 > _lib.MAX_PROGRAM:
            raise ValueError("broadcast expression too long")
        arr = (_lib.Leaf * max(1, len(leaves)))()
        keep = []
        for i, l in enumerate(leaves):
            if l.op == "array":
                arr[i].t = l.value.tensor()
                arr[i].is_scalar = 0
                keep.append(l.value)
            else:
                arr[i].t.dtype = l.dtype
                arr[i].is_scalar = 1
                arr[i].scalar = int.from_bytes(l.value.tobytes().ljust(8, b"\0"), "little")
        return bytes(code), arr, len(leaves), keep

    def materialize(self, stream: Stream | None = None) -> ROCArray:
        """``Base.materialize(bc)``: allocate with ``similar`` (src/broadcast.jl:26-30), then fill."""
        out = ROCArray(_lib.dtype_numpy(self.dtype), self.shape(), stream=stream)
        return materialize_(out, self, stream)


def materialize_(dest: ROCArray, bc, stream: Stream | None = None) -> ROCArray:
    """``Base.materialize!(dest, bc)`` / ``dest .= bc``: one fused kernel, asynchronous on the
    current stream; returns `dest`."""
    bc = Broadcasted.leaf(bc)
    src_shape = bc.shape()
    if len(src_shape) > dest.ndim or any(
            e != 1 and e != dest.dims[d] for d, e in enumerate(src_shape)):
        raise ValueError(f"DimensionMismatch: destination {dest.dims} cannot hold broadcast of shape {src_shape}")
    code, leaves, nleaves, keep = bc.flatten()
    t = dest.tensor()
    st = with_managed(stream or current_stream(), dest, *keep)
    check(lib.b200_broadcast(st.handle, C.byref(t), leaves, nleaves, code, len(code) // 2))
    return dest


def precompile(dest: ROCArray, bc) -> bool:
    """Compiles the kernel specialised for ``dest .= bc`` without launching anything (the library
    otherwise does it on the first call with a new expression structure, as the reference's JIT
    does).  False when the run-time compiler is unavailable: the expression is then interpreted."""
    bc = Broadcasted.leaf(bc)
    code, leaves, nleaves, _keep = bc.flatten()
    t = dest.tensor()
    return lib.b200_broadcast_prepare(C.byref(t), leaves, nleaves, code, len(code) // 2) == 0


def jit_configure(enable: bool) -> None:
    """Switches run-time specialisation of broadcast expressions on or off (default on)."""
    check(lib.b200_jit_configure(1 if enable else 0))


def jit_stats() -> dict:
    out = (C.c_uint64 * 4)()
    check(lib.b200_jit_stats(out))
    return {"compiled": out[0], "hits": out[1], "failures": out[2], "enabled": bool(out[3])}


def prepared(dest: ROCArray, bc, stream: Stream | None = None):
    """Flattens ``dest .= bc`` once and returns a zero-argument callable that re-issues the same
    launch; for call sites that repeat one expression and want the host cost of a bare C call."""
    bc = Broadcasted.leaf(bc)
    code, leaves, nleaves, keep = bc.flatten()
    t = dest.tensor()
    st = stream or current_stream()
    fn, ninstr = lib.b200_broadcast, len(code) // 2

    def launch(_keep=(keep, dest, st)):
        with_managed(st, dest, *keep)
        check(fn(st.handle, C.byref(t), leaves, nleaves, code, ninstr))
    return launch


# dotted-call helpers: bc.exp(x), bc.abs(x), ...
def exp(x): return Broadcasted.call("exp", x)
def abs_(x): return Broadcasted.call("abs", x)
def abs2(x): return Broadcasted.call("abs2", x)
def neg(x): return Broadcasted.call("neg", x)
def add(x, y): return Broadcasted.call("add", x, y)
def sub(x, y): return Broadcasted.call("sub", x, y)
def mul(x, y): return Broadcasted.call("mul", x, y)
def div(x, y): return Broadcasted.call("div", x, y)
def maximum(x, y): return Broadcasted.call("max", x, y)
def minimum(x, y): return Broadcasted.call("min", x, y)
def muladd(x, y, z): return Broadcasted.call("muladd", x, y, z)
def dot(x): return Broadcasted.leaf(x)
