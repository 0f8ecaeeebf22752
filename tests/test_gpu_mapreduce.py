"""mapreducedim! and friends on the device against the CPU oracle.

Tolerances (stated by the workload definition): Float32 <= 1e-5 relative to a Float64
reference, Float16/BFloat16 inputs with Float32 accumulation <= 1e-2, integers bit-exact.
"""
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

RTOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-12, np.dtype(np.float16): 1e-2}
if BF16 is not None:
    RTOL[BF16] = 1e-2


def data(rng, shape, dt):
    dt = np.dtype(dt)
    if dt.kind in "iu":
        return rng.integers(-100 if dt.kind == "i" else 0, 101, shape).astype(dt)
    return rng.random(shape).astype(dt)          # positive: sums are well conditioned


def test_golden(gpu):
    n = int(G["iota_n"])
    x = gpu.ROCArray.from_host(np.arange(1, n + 1, dtype=np.int32))
    s = gpu.sum(x)
    assert s.dtype == np.int64 and s == G["iota_sum"]
    assert gpu.sum(gpu.ROCArray.from_host(G["pow2_in"])) == G["pow2_sum"]
    A = gpu.ROCArray.from_host(G["mat"])
    assert bits_equal(gpu.sum(A, dims=1).to_host(), G["mat_sum_dims1"])
    assert bits_equal(gpu.maximum(A, dims=2).to_host(), G["mat_max_dims2"])
    assert gpu.mapreduce("abs2", "+", A) == G["mat_sumsq"]


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16, "bf16", np.int32, np.int64])
def test_full_reductions_all_sizes(gpu, orc, dt):
    if dt == "bf16":
        if BF16 is None:
            pytest.skip("no bfloat16 host type")
        dt = BF16
    dt = np.dtype(dt)
    rng = np.random.default_rng(1)
    for n in SIZES + ((1 << 22) + 3,):
        if dt.itemsize == 2 and n > 100_003:
            continue                              # the Float16 result itself would overflow
        x = data(rng, n, dt)
        xd = gpu.ROCArray.from_host(x)
        for f, op in (("identity", "+"), ("abs2", "+"), ("abs", "+"), ("identity", "max"), ("identity", "min"), ("abs", "max")):
            got = gpu.mapreduce(f, op, xd)
            ref = orc.mapreduce(f, op, x)
            if dt.kind in "iu":
                assert got == ref, (dt, n, f, op, got, ref)
            else:
                tol = RTOL[dt] if op == "+" else (1e-2 if dt.itemsize == 2 and f != "identity" else 0)
                assert_close(got, ref, tol, (dt, n, f, op))
    # misaligned view and a product
    x = data(rng, 10_007, dt)
    xd = gpu.ROCArray.from_host(x).view(1, 10_007)
    ref = orc.mapreduce("identity", "+", x[1:])
    got = gpu.sum(xd)
    assert (got == ref) if dt.kind in "iu" else abs(float(got) - ref) <= RTOL[dt] * abs(ref)
    small = (rng.random(40) + 0.5).astype(dt) if dt.kind == "f" or dt == BF16 else rng.integers(1, 3, 40).astype(dt)
    got = gpu.prod(gpu.ROCArray.from_host(small))
    ref = orc.mapreduce("identity", "*", small)
    assert (got == ref) if dt.kind in "iu" else abs(float(got) - ref) <= max(RTOL[dt], 1e-6) * abs(ref)


SHAPES = [((3, 100_000), 1), ((3, 100_000), 2), ((512, 1000), 1), ((512, 1000), 2), ((1000, 512), 2),
          ((4096, 64), 1), ((64, 4096), 2), ((1, 777), 1), ((777, 1), 1), ((777, 1), 2), ((2048, 2048), 1),
          ((2048, 2048), 2), ((33, 7, 5), 2), ((33, 7, 5), (1, 2)), ((33, 7, 5), (2, 3)), ((33, 7, 5), (1, 3)),
          ((1, 70, 50, 20), 3), ((16, 16, 16, 16), (2, 3)), ((100_000, 2), 1), ((5, 3), (1, 2))]


@pytest.mark.parametrize("dt", [np.float32, np.float16, np.int32, np.float64])
def test_dims_reductions(gpu, orc, dt):
    dt = np.dtype(dt)
    rng = np.random.default_rng(2)
    for shape, dims in SHAPES:
        A = data(rng, shape, dt)
        Ad = gpu.ROCArray.from_host(A)
        ds = (dims,) if isinstance(dims, int) else dims
        rshape = tuple(1 if (i + 1) in ds else s for i, s in enumerate(shape))
        for f, op in (("identity", "+"), ("identity", "max"), ("abs2", "+"), ("identity", "min")):
            R = gpu.mapreduce(f, op, Ad, dims=dims)
            assert R.dims == rshape, (shape, dims, R.dims)
            ref = orc.mapreducedim(f, op, rshape, A)
            got = R.to_host()
            if dt.kind in "iu":
                assert np.array_equal(got.astype(np.int64), ref.astype(np.int64)), (dt, shape, dims, f, op)
            else:
                tol = RTOL[dt] if op == "+" else 0
                # abs2 of a small Float16 value lands among the Float16 subnormals (quantum 6e-8)
                assert_close(got, ref, tol, (dt, shape, dims, f, op), atol=1e-7 if dt.itemsize == 2 and f == "abs2" else 1e-30)


def test_nan_and_signed_zero(gpu, orc):
    x = np.array([1.0, -3.0, np.nan, 2.0] * 1000, dtype=np.float32)
    xd = gpu.ROCArray.from_host(x)
    assert np.isnan(gpu.maximum(xd)) and np.isnan(gpu.minimum(xd)) and np.isnan(gpu.sum(xd))
    z = gpu.ROCArray.from_host(np.array([-0.0, 0.0, -0.0], dtype=np.float32))
    assert not np.signbit(gpu.maximum(z)) and np.signbit(gpu.minimum(z))
    # against the oracle, bit for bit: zeros of both signs in long vectors and along both dimensions
    rng = np.random.default_rng(12)
    for dt in (np.float32, np.float64, np.float16):
        zeros = np.where(rng.random(70_001) < 0.5, 0.0, -0.0).astype(dt)
        for v in (zeros, np.full(70_001, -0.0, dtype=dt), np.full(33, 0.0, dtype=dt)):
            vd = gpu.ROCArray.from_host(v)
            for op, fn in (("max", gpu.maximum), ("min", gpu.minimum)):
                want = np.asarray(orc.mapreduce("identity", op, v)).astype(dt).reshape(-1)[0]
                got = dt(fn(vd))
                assert got == 0 and np.signbit(got) == np.signbit(want), (dt, op)
        m = np.where(rng.random((300, 70)) < 0.3, 0.0, -0.0).astype(dt)
        md = gpu.ROCArray.from_host(m)
        for dims, rshape in ((1, (1, 70)), (2, (300, 1))):
            for op, fn in (("max", gpu.maximum), ("min", gpu.minimum)):
                want = np.asarray(orc.mapreducedim("identity", op, rshape, m)).astype(dt)
                got = fn(md, dims=dims).to_host()
                assert np.array_equal(np.signbit(got), np.signbit(want)) and not got.any(), (dt, dims, op)
    with pytest.raises(ValueError):
        gpu.maximum(gpu.ROCArray(np.float32, 0))
    assert gpu.sum(gpu.ROCArray(np.float32, 0)) == 0 and gpu.prod(gpu.ROCArray(np.int32, 0)) == 1


def test_mapreducedim_contract(gpu, orc):
    rng = np.random.default_rng(3)
    A = rng.random((3, 2, 10)).astype(np.float32)
    Ad = gpu.ROCArray.from_host(A)
    R = gpu.zeros(np.float32, (3, 2))                     # fewer dims than A: padded with 1
    assert gpu.mapreducedim_("identity", "+", R, Ad) is R   # init=None: R already holds the neutral element
    assert_close(R.to_host(), A.astype(np.float64).sum(axis=2), 1e-5)
    R2 = gpu.fill(np.float32(5.0), (3, 2))
    gpu.mapreducedim_("identity", "+", R2, Ad, init=np.float32(1.0))     # explicit init replaces R's contents
    assert_close(R2.to_host(), A.astype(np.float64).sum(axis=2) + 1.0, 1e-5)
    E = gpu.fill(np.float32(9.0), (1,))
    gpu.mapreducedim_("identity", "+", E, gpu.ROCArray(np.float32, 0))   # empty A: R untouched
    assert E.to_host()[0] == 9.0
    with pytest.raises(ValueError):
        gpu.mapreducedim_("identity", "+", gpu.zeros(np.float32, (2, 2)), Ad)
    # a whole broadcast tree as the mapped function, several operands
    x, y = rng.random(100_001).astype(np.float32), rng.random(100_001).astype(np.float32)
    xd, yd = gpu.ROCArray.from_host(x), gpu.ROCArray.from_host(y)
    got = gpu.mapreduce(None, "+", gpu.broadcast.abs2(xd.dot - yd.dot))
    assert_close(got, ((x.astype(np.float64) - y) ** 2).sum(), 1e-5)
    got = gpu.mapreduce(lambda v: v * v + 1, "+", xd)
    assert_close(got, (orc.broadcast(("add", ("mul", x, x), 1)).astype(np.float64)).sum(), 1e-5)
    M = rng.random((300, 40)).astype(np.float32)
    Md = gpu.ROCArray.from_host(M)
    v = rng.random(300).astype(np.float32)
    got = gpu.mapreduce(None, "max", Md.dot * gpu.ROCArray.from_host(v).dot, dims=1).to_host()
    assert bits_equal(got, (M * v[:, None]).max(axis=0, keepdims=True))


def test_run_to_run_determinism(gpu):
    rng = np.random.default_rng(5)
    x = gpu.ROCArray.from_host(rng.standard_normal(3_000_001).astype(np.float32))
    A = gpu.ROCArray.from_host(rng.standard_normal((4096, 300)).astype(np.float32))
    a = [gpu.sum(x).tobytes() for _ in range(5)]
    assert len(set(a)) == 1
    b = [gpu.sum(A, dims=2).to_host().tobytes() for _ in range(3)]
    assert len(set(b)) == 1


@pytest.mark.parametrize("dt", [np.float16, "bf16"])
def test_packed_extrema_of_16_bit_floats(gpu, dt):
    """maximum / minimum (and their abs forms) of Float16 / BFloat16 fold pairs with one packed
    instruction; the results must be the same bits a widened fold gives: NaN wins wherever one
    occurs, -0.0 is below +0.0, infinities and subnormals pass through - along both dimensions of
    a matrix whose first dimension takes the 16-byte path, and for long vectors."""
    if dt == "bf16":
        if BF16 is None:
            pytest.skip("no bfloat16 host type")
        dt = BF16
    dt = np.dtype(dt)
    rng = np.random.default_rng(21)
    a = rng.standard_normal((512, 300)).astype(np.float32)
    a[rng.random(a.shape) < 0.05] = 0.0
    a[rng.random(a.shape) < 0.05] = -0.0
    a[7, 11] = np.inf
    a[100, 200] = -np.inf
    a[5, :] = np.float32(6e-8)                                   # subnormal in Float16
    a[:, 17] = np.where(np.arange(512) % 2 == 0, 0.0, -0.0)        # a column of zeros of both signs
    a[33, :] = -0.0
    a = a.astype(dt)
    a[200, 3] = np.nan
    a[3, 250] = np.nan
    ad = gpu.ROCArray.from_host(a)
    wide = a.astype(np.float32)

    def fold(x, op, axis):
        nan = np.isnan(x).any(axis=axis, keepdims=True)
        r = (np.max if op == "max" else np.min)(np.where(np.isnan(x), 0, x), axis=axis, keepdims=True)
        # zeros: max is +0.0 if any +0.0 took part, min is -0.0 if any -0.0 did
        pz = ((x == 0) & ~np.signbit(x)).any(axis=axis, keepdims=True)
        nz = ((x == 0) & np.signbit(x)).any(axis=axis, keepdims=True)
        zero = r == 0
        r = np.where(zero & (op == "max"), np.where(pz, 0.0, -0.0), r)
        r = np.where(zero & (op == "min"), np.where(nz, -0.0, 0.0), r)
        return np.where(nan, np.nan, r).astype(np.float32)

    for f, src in ((None, wide), ("abs", np.abs(wide))):
        for op, fn in (("max", gpu.maximum), ("min", gpu.minimum)):
            for dims, axis in ((1, 0), (2, 1)):
                got = (fn(ad, dims=dims) if f is None else gpu.mapreduce(f, op, ad, dims=dims)).to_host().astype(np.float32)
                want = fold(src, op, axis)
                assert np.array_equal(np.isnan(got), np.isnan(want)), (f, op, dims)
                ok = ~np.isnan(want)
                assert np.array_equal(got[ok], want[ok]) and np.array_equal(np.signbit(got[ok]), np.signbit(want[ok])), (f, op, dims)
    v = rng.standard_normal(1_000_003).astype(dt)
    vd = gpu.ROCArray.from_host(v)
    assert dt.type(gpu.maximum(vd)) == v.astype(np.float32).max() and dt.type(gpu.minimum(vd)) == v.astype(np.float32).min()
    v[777_777] = np.nan
    assert np.isnan(gpu.maximum(gpu.ROCArray.from_host(v)))
