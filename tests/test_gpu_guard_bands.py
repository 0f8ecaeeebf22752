"""Every operator with its destination between guard bands (tests/helpers.py: Guarded): results are
right and not one byte outside the destination changes.  Stands in for a device memory checker,
including destinations that start off a 16-byte boundary and ragged sizes around the kernels'
tile sizes."""
import numpy as np
import pytest

from helpers import Guarded

pytestmark = pytest.mark.gpu
SIZES = (1, 3, 31, 1000, 4095, 4097, 8192 * 3 + 5, 262_144 + 4, 1_048_576 + 12)


@pytest.mark.parametrize("misalign", [0, 1])
def test_broadcast_scan_and_fill_stay_inside(gpu, orc, misalign):
    rng = np.random.default_rng(20)
    for n in SIZES:
        x = rng.random(n).astype(np.float32)
        y = rng.random(n).astype(np.float32)
        xd, yd = gpu.ROCArray.from_host(x), gpu.ROCArray.from_host(y)
        g = Guarded(gpu, np.float32, n, misalign)
        gpu.materialize_(g.array, np.float32(2.5) * xd.dot + yd.dot)                 # hard-wired kernel
        assert np.array_equal(g.array.to_host(), np.float32(2.5) * x + y)
        g.check(("axpy", n))
        gpu.materialize_(g.array, gpu.broadcast.maximum(xd.dot, yd.dot) - np.float32(1))   # specialised evaluator
        assert np.array_equal(g.array.to_host(), np.maximum(x, y) - np.float32(1))
        g.check(("tree", n))
        xi = rng.integers(-100, 101, n).astype(np.int32)
        gi = Guarded(gpu, np.int32, n, misalign)
        gpu.accumulate_("+", gi.array, gpu.ROCArray.from_host(xi))
        assert np.array_equal(gi.array.to_host(), np.cumsum(xi, dtype=np.int32))
        gi.check(("cumsum", n))
        gi.array.fill_(7)
        assert (gi.array.to_host() == 7).all()
        gi.check(("fill", n))
        gpu.random.fill_random_(gi.array, gpu.random.INTEGERS, seed=1, lo=-5, hi=5)
        gi.check(("fill_random", n))


def test_reductions_stay_inside(gpu, orc):
    rng = np.random.default_rng(21)
    for shape in ((1000,), (70_001,), (300, 70), (33, 500), (8, 9, 10), (2048, 64)):
        A = rng.random(shape).astype(np.float32)
        Ad = gpu.ROCArray.from_host(A)
        for d in range(len(shape)):
            rshape = tuple(1 if k == d else s for k, s in enumerate(shape))
            g = Guarded(gpu, np.float32, rshape)
            gpu.mapreducedim_("identity", "+", g.array, Ad, init=np.float32(0))
            assert np.allclose(g.array.to_host(), A.sum(axis=d, keepdims=True, dtype=np.float64), rtol=1e-5)
            g.check(("sum", shape, d))
            gpu.mapreducedim_("abs2", "+", g.array, Ad.dot * np.float32(2), init=np.float32(0))    # evaluator path
            assert np.allclose(g.array.to_host(), (4.0 * A.astype(np.float64) ** 2).sum(axis=d, keepdims=True), rtol=1e-5)
            g.check(("evaluator", shape, d))
        g = Guarded(gpu, np.float32, (1,) * len(shape), 1)
        gpu.mapreducedim_("identity", "max", g.array, Ad, init=np.float32(-np.inf))
        assert g.array.to_host().reshape(-1)[0] == A.max()
        g.check(("max", shape))


@pytest.mark.parametrize("misalign", [0, 1])
def test_sort_gather_and_compaction_stay_inside(gpu, misalign):
    rng = np.random.default_rng(22)
    for n in (1, 2, 1000, 8191, 8193, 100_003, 1_000_001):
        k = rng.integers(0, 2**32, n, dtype=np.uint32)
        g = Guarded(gpu, np.uint32, n, misalign)
        g.array.copy_from_host(k)
        gpu.sort_(g.array)
        assert np.array_equal(g.array.to_host(), np.sort(k))
        g.check(("sort", n))
        f = rng.standard_normal(n).astype(np.float32)
        fd = gpu.ROCArray.from_host(f)
        gp = Guarded(gpu, np.int64, n, misalign)
        gpu.sortperm_(gp.array, fd)
        assert np.array_equal(gp.array.to_host(), np.argsort(f, kind="stable") + 1)
        gp.check(("sortperm", n))
        # gather and compaction through the C ABI into guarded destinations
        import ctypes as C
        L = gpu._lib
        gg = Guarded(gpu, np.float32, n, misalign)
        ty, tx, ti = gg.array.tensor(), fd.tensor(), gp.array.tensor()
        assert L.lib.b200_gather(gpu.current_stream().handle, C.byref(ty), C.byref(tx), C.byref(ti)) == L.OK
        assert np.array_equal(gg.array.to_host(), np.sort(f, kind="stable"))
        gg.check(("gather", n))
        m = rng.random(n) < 0.4
        md = gpu.ROCArray.from_host(m)
        pos = gpu.ROCArray.from_host(np.cumsum(m).astype(np.int64))
        cnt = int(m.sum())
        if cnt:
            gc = Guarded(gpu, np.int64, cnt, misalign)
            ty, tb, tp = gc.array.tensor(), md.tensor(), pos.tensor()
            assert L.lib.b200_compact(gpu.current_stream().handle, C.byref(ty), C.byref(tb), C.byref(tp), None) == L.OK
            assert np.array_equal(gc.array.to_host(), np.flatnonzero(m) + 1)
            gc.check(("compact", n))
        y = Guarded(gpu, np.float32, n, misalign)
        gpu._lib.check(L.lib.b200_reverse(gpu.current_stream().handle, C.byref(y.array.tensor()), C.byref(fd.tensor()), 1))
        assert np.array_equal(y.array.to_host(), f[::-1])
        y.check(("reverse", n))
    gpu.synchronize()
