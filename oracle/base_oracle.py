"""NumPy restatement of what the reference's hot path must compute (checker only).

Sources restated:
* mapreducedim!  - src/kernels/mapreduce.jl:86-173 of the reference: R[Iother] = op over the
  reduced index set of f(A[I]); reduced dimensions are those where size(R, d) == 1; an empty A
  leaves R untouched; `init` is folded in once.
* broadcast      - Base.Broadcast element semantics (the reference only selects the style,
  src/broadcast.jl:3-35; the arithmetic is Julia Base, a dependency that is not in the tree):
  per node, operands are converted to promote_type of their types, + - * round once each,
  muladd may fuse, abs2(x) = x*x, max/min propagate NaN and order -0.0 < +0.0, Float16
  arithmetic computes in Float32 and rounds after every operation, integers wrap.
* accumulate     - src/kernels/accumulate.jl:1-8: B[i] = op(B[i-1], A[i]) seeded by `init`,
  element type preserved.
* sort/sortperm  - src/kernels/sorting.jl:1-3 with Base.isless ordering (NaN last,
  -0.0 < +0.0), stable, `rev` reverses the ordering (ties keep input order), permutation is
  1-based Int64.
Floating-point reductions and scans are evaluated in Float64 here; the tests compare with the
stated relative tolerance.  Integer results are exact (two's-complement wrap).
"""
from __future__ import annotations

import numpy as np

try:
    import ml_dtypes
    _BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    _BF16 = None


def _is_float(dt):
    dt = np.dtype(dt)
    return dt.kind == "f" or dt == _BF16


def promote(a, b):
    """Base.promote_type for the element types in play."""
    a, b = np.dtype(a), np.dtype(b)
    if a == b:
        return a
    if a == np.bool_:
        return b
    if b == np.bool_:
        return a
    fa, fb = _is_float(a), _is_float(b)
    if fa and fb:
        if {a, b} == {np.dtype(np.float16), _BF16}:
            return np.dtype(np.float32)
        return a if a.itemsize >= b.itemsize else b
    if fa:
        return a
    if fb:
        return b
    if a.itemsize != b.itemsize:
        return a if a.itemsize > b.itemsize else b
    return a if a.kind == "u" else b


def _dtype_of(v):
    if isinstance(v, np.ndarray) or isinstance(v, np.generic):
        return v.dtype
    if isinstance(v, bool):
        return np.dtype(np.bool_)
    if isinstance(v, int):
        return np.dtype(np.int64)
    if isinstance(v, float):
        return np.dtype(np.float64)
    raise TypeError(type(v))


def _compute_type(dt):
    dt = np.dtype(dt)
    if dt == np.float16 or dt == _BF16:
        return np.dtype(np.float32)
    return dt


def _jl_max(x, y):
    out = np.where(np.signbit(x - y), y, x)
    return np.where(np.isnan(x) | np.isnan(y), x - y, out) if _is_float(x.dtype) else np.maximum(x, y)


def _jl_min(x, y):
    out = np.where(np.signbit(y - x), y, x)
    return np.where(np.isnan(x) | np.isnan(y), x - y, out) if _is_float(x.dtype) else np.minimum(x, y)


def _eval(node):
    """Returns (values, dtype) of a broadcast tree given as nested tuples (op, args...)."""
    if not isinstance(node, tuple):
        dt = _dtype_of(node)
        return np.asarray(node, dtype=dt), dt
    op, *args = node
    vals = [_eval(a) for a in args]
    dt = vals[0][1]
    for _, d in vals[1:]:
        dt = promote(dt, d)
    if dt == np.bool_:
        dt = np.dtype(np.int64)
    if op == "div" or op == "exp":
        if not _is_float(dt):
            dt = np.dtype(np.float64)
    ct = _compute_type(dt)
    xs = [np.asarray(v).astype(dt).astype(ct) for v, _ in vals]   # convert to the node type first
    with np.errstate(all="ignore"):
        if op == "add": r = xs[0] + xs[1]
        elif op == "sub": r = xs[0] - xs[1]
        elif op == "mul": r = xs[0] * xs[1]
        elif op == "div": r = xs[0] / xs[1]
        elif op == "muladd": r = xs[0] * xs[1] + xs[2]      # unfused variant; tests allow either
        elif op == "abs": r = np.abs(xs[0])
        elif op == "abs2": r = xs[0] * xs[0]
        elif op == "neg": r = -xs[0] if ct.kind != "u" else (np.zeros_like(xs[0]) - xs[0])
        elif op == "exp": r = np.exp(xs[0].astype(np.float64)).astype(ct) if ct != np.float64 else np.exp(xs[0])
        elif op == "max": r = _jl_max(xs[0], xs[1])
        elif op == "min": r = _jl_min(xs[0], xs[1])
        else: raise ValueError(op)
    return np.asarray(r).astype(ct).astype(dt), dt


def broadcast(tree, out_dtype=None):
    """Value of a fused broadcast expression; `tree` = nested tuples ("add", x, ("mul", a, y))..."""
    v, dt = _eval(tree)
    return v.astype(out_dtype) if out_dtype is not None else v


_MAPS = {
    "identity": lambda x: x,
    None: lambda x: x,
    "abs": lambda x: np.abs(x),
    "abs2": lambda x: x * x,
    "neg": lambda x: -x,
    "exp": lambda x: np.exp(x),
}


def _fold(op, x, axis):
    if op in ("+", "add"): return np.add.reduce(x, axis=axis, keepdims=True)
    if op in ("*", "mul"): return np.multiply.reduce(x, axis=axis, keepdims=True)
    if op not in ("max", "min"):
        raise ValueError(op)
    # Base.max / Base.min (base/math.jl): NaN wins, and -0.0 orders below +0.0.  NumPy's max/min
    # propagate NaN as well but leave the sign of a zero result open, so it is fixed here: a zero
    # maximum is +0.0 as soon as one +0.0 takes part, a zero minimum is -0.0 as soon as one -0.0 does.
    r = (np.max if op == "max" else np.min)(x, axis=axis, keepdims=True)
    if _is_float(np.asarray(x).dtype):
        x = np.asarray(x)
        if op == "max":
            has = np.any((x == 0) & ~np.signbit(x), axis=axis, keepdims=True)
            r = np.where(r == 0, np.where(has, x.dtype.type(0.0), x.dtype.type(-0.0)), r)
        else:
            has = np.any((x == 0) & np.signbit(x), axis=axis, keepdims=True)
            r = np.where(r == 0, np.where(has, x.dtype.type(-0.0), x.dtype.type(0.0)), r)
    return r


def _op2(op, a, b):
    if op in ("+", "add"): return a + b
    if op in ("*", "mul"): return a * b
    if op == "max": return _jl_max(np.asarray(a), np.asarray(b))
    return _jl_min(np.asarray(a), np.asarray(b))


def mapreducedim(f, op, r_shape, A, init=None, out_dtype=None):
    """R of shape `r_shape` (1 in reduced dims).  Floats accumulate in Float64 (compare with a
    tolerance); integers accumulate exactly in `out_dtype` (default: Base.add_sum widening)."""
    A = np.asarray(A)
    fx = _MAPS[f](A.astype(_compute_type(A.dtype))) if not callable(f) else f(A)
    r_shape = tuple(r_shape) + (1,) * (A.ndim - len(r_shape))
    axes = tuple(d for d in range(A.ndim) if r_shape[d] == 1 and A.shape[d] != 1)
    if _is_float(fx.dtype):
        acc = fx.astype(np.float64)
    else:
        if out_dtype is None:
            out_dtype = fx.dtype
            if op in ("+", "add", "*", "mul") and fx.dtype.itemsize < 8:
                out_dtype = np.dtype(np.uint64 if fx.dtype.kind == "u" else np.int64)
        acc = fx.astype(out_dtype)
    with np.errstate(all="ignore"):
        r = _fold(op, acc, axes) if axes else acc.copy()
        if init is not None:
            r = _op2(op, np.asarray(init, dtype=r.dtype), r)
    return r.reshape(r_shape)


def mapreduce(f, op, A, init=None):
    """Full reduction to a Python scalar (Float64 for floating-point inputs)."""
    A = np.asarray(A)
    return mapreducedim(f, op, (1,) * A.ndim, A, init=init).reshape(-1)[0]


def accumulate(op, A, init=None, axis=0, exact_dtype=True):
    """Inclusive scan along `axis` (0-based).  Integers: exact, wrapping in A's dtype.  Floats:
    Float64 values (compare with tolerance)."""
    A = np.asarray(A)
    fl = _is_float(A.dtype)
    x = A.astype(np.float64) if fl else A.copy()
    with np.errstate(all="ignore"):
        if op in ("+", "add"): r = np.cumsum(x, axis=axis, dtype=x.dtype)
        elif op in ("*", "mul"): r = np.cumprod(x, axis=axis, dtype=x.dtype)
        elif op == "max": r = np.maximum.accumulate(x, axis=axis)
        elif op == "min": r = np.minimum.accumulate(x, axis=axis)
        else: raise ValueError(op)
        if init is not None:
            r = _op2(op, np.asarray(init, dtype=r.dtype), r).astype(r.dtype)
    return r


def isless_key(x):
    """Integer rank vector r with r[i] < r[j]  <=>  isless(x[i], x[j]) (ties share a rank)."""
    x = np.asarray(x)
    if _is_float(x.dtype):
        xf = x.astype(np.float64)
        isn = np.isnan(xf)
        primary = np.where(isn, np.inf, xf)
        tie = ((xf == 0) & ~np.signbit(xf)).astype(np.int8)     # -0.0 before +0.0
        order = np.lexsort((tie, primary, isn))
        sp, st, si = primary[order], tie[order], isn[order]
        new = np.ones(len(x), dtype=bool)
        new[1:] = (sp[1:] != sp[:-1]) | (st[1:] != st[:-1]) | (si[1:] != si[:-1])
        new[1:] &= ~(si[1:] & si[:-1])                           # all NaNs are equal under isless
        ranks = np.empty(len(x), dtype=np.int64)
        ranks[order] = np.cumsum(new) - 1
        return ranks
    order = np.argsort(x, kind="stable")
    sx = x[order]
    new = np.ones(len(x), dtype=bool)
    new[1:] = sx[1:] != sx[:-1]
    ranks = np.empty(len(x), dtype=np.int64)
    ranks[order] = np.cumsum(new) - 1
    return ranks


def sortperm(x, rev=False):
    """Stable 1-based Int64 permutation under isless (reversed ordering when `rev`)."""
    r = isless_key(x)
    if rev:
        r = -r
    return (np.argsort(r, kind="stable") + 1).astype(np.int64)


def sort(x, rev=False):
    x = np.asarray(x)
    return x[sortperm(x, rev) - 1]
