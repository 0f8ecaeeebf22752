"""Fused broadcast on the device against the CPU oracle (bit-exact except exp)."""
from pathlib import Path

import numpy as np
import pytest

from helpers import SIZES, assert_close, bits_equal

pytestmark = pytest.mark.gpu
G = np.load(Path(__file__).parent / "golden" / "known_answers.npz")
try:
    import ml_dtypes
    BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:
    BF16 = None


def rnd(rng, n, dt):
    dt = np.dtype(dt)
    if dt.kind in "iu":
        return rng.integers(-50 if dt.kind == "i" else 0, 50, n).astype(dt)
    return (rng.random(n) * 4 - 2).astype(dt)


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16, "bf16"])
def test_axpy_all_sizes(gpu, orc, dt):
    if dt == "bf16":
        if BF16 is None:
            pytest.skip("no bfloat16 host type")
        dt = BF16
    dt = np.dtype(dt)
    rng = np.random.default_rng(0)
    a = dt.type(2.5)
    for n in SIZES:
        x, y = rnd(rng, n, dt), rnd(rng, n, dt)
        z = (a * gpu.ROCArray.from_host(x).dot + gpu.ROCArray.from_host(y).dot).materialize()
        assert z.dtype == dt
        assert bits_equal(z.to_host(), orc.broadcast(("add", ("mul", a, x), y))), (dt, n)
    # operands whose pointers are not 16-byte aligned, and in-place destination
    n = 10_001
    x, y = rnd(rng, n + 3, dt), rnd(rng, n + 1, dt)
    xd, yd = gpu.ROCArray.from_host(x).view(3, n + 3), gpu.ROCArray.from_host(y).view(1, n + 1)
    gpu.materialize_(yd, a * xd.dot + yd.dot)
    assert bits_equal(yd.to_host(), orc.broadcast(("add", ("mul", a, x[3:]), y[1:])))


def test_golden_semantics(gpu):
    a, b = gpu.ROCArray.from_host(G["mm_a"]), gpu.ROCArray.from_host(G["mm_b"])
    mx = gpu.broadcast.maximum(a, b).materialize().to_host()
    mn = gpu.broadcast.minimum(a, b).materialize().to_host()
    ok = ~np.isnan(G["mm_max"])
    assert np.array_equal(np.isnan(mx), ~ok) and bits_equal(mx[ok], G["mm_max"][ok])
    assert np.array_equal(np.isnan(mn), ~ok) and bits_equal(mn[ok], G["mm_min"][ok])
    z = (G["axpy_a"][()] * gpu.ROCArray.from_host(G["axpy_x"]).dot + gpu.ROCArray.from_host(G["axpy_y"]).dot).materialize()
    assert bits_equal(z.to_host(), G["axpy_unfused"])      # multiply and add are NOT contracted


def test_fused_exp_expression(gpu, orc):
    rng = np.random.default_rng(4)
    for n in (1, 1000, 4096 * 4, (1 << 20) + 5):
        x, y, z = (rnd(rng, n, np.float32) / 2 for _ in range(3))
        bc = gpu.broadcast
        xd, yd, zd = (gpu.ROCArray.from_host(v) for v in (x, y, z))
        r = (xd.dot * yd.dot + bc.exp(-bc.abs_(zd))).materialize().to_host()
        ref = orc.broadcast(("add", ("mul", x, y), ("exp", ("neg", ("abs", z)))))
        assert np.allclose(r, ref, rtol=1e-6, atol=3e-7), n
        # same tree written the other way round goes through the same kernel
        r2 = (bc.exp(-bc.abs_(zd)) + xd.dot * yd.dot).materialize().to_host()
        assert np.array_equal(r, r2)
    # the evaluator path (a tree the hard-wired kernels do not match) agrees with them
    r3 = (xd.dot * yd.dot + bc.exp(-bc.abs_(zd)) + np.float32(0.0)).materialize().to_host()
    assert np.allclose(r3, r, rtol=0, atol=0) or np.allclose(r3, r, rtol=1e-7)


OPS2 = ["add", "sub", "mul", "div", "max", "min"]
OPS1 = ["abs", "abs2", "neg", "exp"]


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.int32, np.int64, np.float16, np.uint32, np.int16])
def test_every_operator(gpu, orc, dt):
    dt = np.dtype(dt)
    rng = np.random.default_rng(7)
    n = 5003
    x, y, w = rnd(rng, n, dt), rnd(rng, n, dt), rnd(rng, n, dt)
    if dt.kind in "iu":
        y[y == 0] = 3
    xd, yd, wd = (gpu.ROCArray.from_host(v) for v in (x, y, w))
    B = gpu.Broadcasted
    for op in OPS2:
        got = B.call(op, xd, yd).materialize().to_host()
        ref = orc.broadcast((op, x, y))
        assert got.dtype == ref.dtype, (op, got.dtype, ref.dtype)
        assert bits_equal(got, ref), (dt, op)
        s = dt.type(3)
        assert bits_equal(B.call(op, xd, s).materialize().to_host(), orc.broadcast((op, x, s))), (dt, op, "array-scalar")
        assert bits_equal(B.call(op, s, xd).materialize().to_host(), orc.broadcast((op, s, x))), (dt, op, "scalar-array")
    for op in OPS1:
        got = B.call(op, xd).materialize().to_host()
        ref = orc.broadcast((op, x))
        assert got.dtype == ref.dtype, (op, got.dtype, ref.dtype)
        if op == "exp":
            assert np.allclose(got.astype(np.float64), ref.astype(np.float64), rtol=2e-3 if dt.itemsize == 2 else 1e-6), (dt, op)
        else:
            assert bits_equal(got, ref), (dt, op)
    got = B.call("muladd", xd, yd, wd).materialize().to_host()
    ref = orc.broadcast(("muladd", x, y, w))
    if dt.kind in "iu":
        assert bits_equal(got, ref)
    else:
        assert np.allclose(got.astype(np.float64), ref.astype(np.float64), rtol=4e-3 if dt.itemsize == 2 else 1e-6, atol=1e-6)


def test_mixed_types_and_promotion(gpu, orc):
    rng = np.random.default_rng(9)
    n = 777
    i32, f32, f64, i64 = rnd(rng, n, np.int32), rnd(rng, n, np.float32), rnd(rng, n, np.float64), rnd(rng, n, np.int64)
    di32, df32, df64, di64 = (gpu.ROCArray.from_host(v) for v in (i32, f32, f64, i64))
    cases = [
        (di32.dot + df32.dot, ("add", i32, f32)),
        (di64.dot + df64.dot, ("add", i64, f64)),                      # ROCArray([1,2,3]) .+ ROCArray([1.0,2.0,3.0])
        (2 * df32.dot, ("mul", 2, f32)),                                # 2x keeps Float32
        (2.0 * df32.dot, ("mul", 2.0, f32)),                            # Float64 literal widens
        (di32.dot / di32.dot.__add__(101), ("div", i32, ("add", i32, 101))),
        ((di32.dot + di32.dot) * df32.dot, ("mul", ("add", i32, i32), f32)),
        (gpu.broadcast.exp(di32.dot * 0), ("exp", ("mul", i32, 0))),
        (df32.dot + df64.dot * di32.dot, ("add", f32, ("mul", f64, i32))),
    ]
    for bc, tree in cases:
        got, ref = bc.materialize().to_host(), orc.broadcast(tree)
        assert got.dtype == ref.dtype, (tree[0], got.dtype, ref.dtype)
        if tree[0] == "exp":
            assert np.allclose(got, ref, rtol=1e-12)
        else:
            assert bits_equal(got, ref), tree[0]
    # destination type differs from the expression type: converted on store
    dest = gpu.ROCArray(np.float32, n)
    gpu.materialize_(dest, df64.dot * 2.0)
    assert bits_equal(dest.to_host(), (f64 * 2.0).astype(np.float32))


def test_shape_broadcasting(gpu, orc):
    rng = np.random.default_rng(11)
    x, y = rng.random((2, 3)), rng.random((1, 3))
    got = (gpu.ROCArray.from_host(x).dot + gpu.ROCArray.from_host(y).dot).materialize()
    assert got.dims == (2, 3) and bits_equal(got.to_host(), x + y)
    z, a, b = rng.random((2, 3)), rng.random((2, 3)), rng.random(2)
    zd = gpu.ROCArray.from_host(z)
    gpu.materialize_(zd, gpu.ROCArray.from_host(a).dot + gpu.ROCArray.from_host(b).dot)    # z .= x .+ y with y of length 2
    assert bits_equal(zd.to_host(), a + b[:, None])
    p, q, r = rng.random((5, 1, 7)).astype(np.float32), rng.random((1, 6, 1)).astype(np.float32), rng.random((5, 6, 7)).astype(np.float32)
    got = (gpu.ROCArray.from_host(p).dot * gpu.ROCArray.from_host(q).dot - gpu.ROCArray.from_host(r).dot).materialize()
    assert got.dims == (5, 6, 7) and bits_equal(got.to_host(), p * q - r)
    gpu.materialize_(zd, 0.0)                                                              # gpu_mat .= 0f0
    assert not zd.to_host().any()
    with pytest.raises(ValueError):
        (gpu.ROCArray.from_host(x).dot + gpu.ROCArray.from_host(rng.random((3, 3))).dot).materialize()
    e = (gpu.ROCArray(np.float32, 0).dot + 1).materialize()
    assert e.dims == (0,)
