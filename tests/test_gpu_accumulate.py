"""accumulate! / cumsum / cumprod on the device against the CPU oracle."""
from pathlib import Path

import numpy as np
import pytest

from helpers import assert_close, bits_equal

pytestmark = pytest.mark.gpu
G = np.load(Path(__file__).parent / "golden" / "known_answers.npz")
NS = (0, 1, 2, 3, 10, 10_000, 16384, 16384 + 1, 4095, 4096, 4097, 8192 * 3 - 1, 1_000_003,
      1 << 20, (1 << 21) + 32, 3 * (1 << 19) + 4, 5_000_000)     # the last four take the persistent segment kernel


def test_golden(gpu):
    assert bits_equal(gpu.cumsum(gpu.ROCArray.from_host(G["wrap_in"])).to_host(), G["wrap_scan"])
    assert bits_equal(gpu.cumsum(gpu.ROCArray.from_host(G["pow2_in"])).to_host(), G["pow2_scan"])
    n = 100_000
    assert np.array_equal(gpu.cumsum(gpu.ones(np.int64, n)).to_host(), np.arange(1, n + 1))
    alt = np.where(np.arange(n) % 2 == 0, 1, -1).astype(np.int32)
    assert np.array_equal(gpu.cumsum(gpu.ROCArray.from_host(alt)).to_host(), (np.arange(n) % 2 == 0).astype(np.int32))


@pytest.mark.parametrize("dt", [np.float64, np.float32, np.int32, np.int64, np.float16, np.uint32])
def test_vector_scans(gpu, orc, dt):
    dt = np.dtype(dt)
    rng = np.random.default_rng(0)
    for n in NS:
        if dt.itemsize == 2 and n > 20_000:
            continue                              # prefix sums would leave the Float16 range
        x = rng.random(n).astype(dt) if dt.kind == "f" else rng.integers(0 if dt.kind == "u" else -100, 101, n).astype(dt)
        xd = gpu.ROCArray.from_host(x)
        init = dt.type(rng.random()) if dt.kind == "f" else dt.type(7)
        for kw, okw in (({}, {}), ({"init": init}, {"init": init})):
            got = gpu.accumulate("+", xd, **kw).to_host()
            ref = orc.accumulate("+", x, **okw)
            assert got.dtype == dt and got.shape == (n,)
            if dt.kind in "iu":
                assert np.array_equal(got, ref), (dt, n, kw)
            else:
                assert_close(got, ref, {8: 1e-12, 4: 1e-5, 2: 1e-2}[dt.itemsize], (dt, n, kw))
    # in place, specialised forms, other operators
    x = (rng.random(50_001) + 0.5).astype(dt) if dt.kind == "f" else rng.integers(1, 3, 50_001).astype(dt)
    xd = gpu.ROCArray.from_host(x)
    assert gpu.accumulate_("+", xd, xd) is xd
    ref = orc.accumulate("+", x)
    assert np.array_equal(xd.to_host(), ref) if dt.kind in "iu" else np.allclose(xd.to_host(), ref, rtol=1e-2 if dt.itemsize == 2 else 1e-5)
    y = x[:60]
    cp = gpu.cumprod(gpu.ROCArray.from_host(y)).to_host()
    refp = orc.accumulate("*", y)
    assert np.array_equal(cp, refp) if dt.kind in "iu" else np.allclose(cp.astype(np.float64), refp, rtol=2e-2 if dt.itemsize == 2 else 1e-5)
    w = rng.standard_normal(70_001).astype(dt) if dt.kind == "f" else rng.integers(0, 1000, 70_001).astype(dt)
    for op in ("max", "min"):
        got = gpu.accumulate(op, gpu.ROCArray.from_host(w), init=None).to_host()
        assert np.array_equal(got.astype(np.float64), orc.accumulate(op, w).astype(np.float64)), (dt, op)
    # pointer that is not 16-byte aligned
    v = gpu.ROCArray.from_host(x).view(1, 40_000)
    got = gpu.cumsum(v).to_host()
    ref = orc.accumulate("+", x[1:40_000])
    assert np.array_equal(got, ref) if dt.kind in "iu" else np.allclose(got, ref, rtol=1e-2 if dt.itemsize == 2 else 1e-5)


@pytest.mark.parametrize("sizes,dims", [((2,), 2), ((3, 4, 5), 2), ((1, 70, 50, 20), 3), ((3, 100_000), 1),
                                         ((3, 100_000), 2), ((512, 1000), 1), ((512, 1000), 2), ((10_000, 7), 1),
                                         ((7, 9000, 3), 2), ((40, 33), 2), ((5000, 40), 2), ((4, 4, 4), 3)])
def test_multidimensional(gpu, orc, sizes, dims):
    rng = np.random.default_rng(1)
    for dt in (np.int64, np.float32):
        x = rng.integers(-1000, 1000, sizes).astype(dt) if dt == np.int64 else rng.random(sizes).astype(dt)
        xd = gpu.ROCArray.from_host(x)
        got = gpu.accumulate("+", xd, dims=dims).to_host()
        ref = orc.accumulate("+", x, axis=dims - 1) if dims <= x.ndim else x
        if dt == np.int64:
            assert np.array_equal(got, ref), (sizes, dims)
        else:
            assert_close(got, ref, 1e-5, (sizes, dims))
    with pytest.raises(ValueError):
        gpu.accumulate("+", gpu.ROCArray(np.float32, (3, 3)))


def test_int32_scan_is_deterministic_and_exact(gpu, orc):
    rng = np.random.default_rng(2)
    x = rng.integers(-100, 101, (1 << 22) + 11).astype(np.int32)
    xd = gpu.ROCArray.from_host(x)
    outs = [gpu.cumsum(xd).to_host() for _ in range(3)]
    assert np.array_equal(outs[0], orc.accumulate("+", x))
    assert all(np.array_equal(outs[0], o) for o in outs[1:])


def test_segment_kernel_small_types_and_variants(gpu, orc):
    """Long vectors of 16-bit and 64-bit elements, exclusive mode, device-resident carry, max-scan."""
    n = (1 << 21) + 64
    alt = np.where(np.arange(n) % 2 == 0, 1.0, -1.0)
    for dt in (np.float16, np.int64, np.float64):
        x = alt.astype(dt)
        got = gpu.cumsum(gpu.ROCArray.from_host(x)).to_host()
        assert np.array_equal(got, (np.arange(n) % 2 == 0).astype(dt)), dt
    rng = np.random.default_rng(5)
    x = rng.integers(-100, 101, n).astype(np.int32)
    xd = gpu.ROCArray.from_host(x)
    ex = gpu.accumulate_("+", gpu.ROCArray(np.int32, n), xd, init=np.int32(11), inclusive=False).to_host()
    ref = orc.accumulate("+", x, init=np.int32(11))
    assert ex[0] == 11 and np.array_equal(ex[1:], ref[:-1])
    w = rng.standard_normal(n).astype(np.float32)
    assert np.array_equal(gpu.accumulate("max", gpu.ROCArray.from_host(w), init=None).to_host(), np.maximum.accumulate(w))
    # carry in device memory (the sharded scan's second phase)
    import ctypes as C
    L = gpu._lib
    carry = gpu.ROCArray.from_host(np.array([1000], dtype=np.int32))
    out = gpu.ROCArray(np.int32, n)
    tb, ta = out.tensor(), xd.tensor()
    assert L.lib.b200_accumulate_carry(gpu.current_stream().handle, C.byref(tb), C.byref(ta), L.RED_ADD,
                                       C.c_void_p(carry.ptr), 0, 1) == L.OK
    assert np.array_equal(out.to_host(), orc.accumulate("+", x, init=np.int32(1000)))


@pytest.mark.parametrize("sizes", [(33, 500), (64, 300, 5), (128, 65), (1000, 130), (36, 64, 2), (257, 129)])
def test_scans_down_a_strided_dimension(gpu, orc, sizes):
    """accumulate(op, A; dims=2) with at least a warp of columns: the tiled kernel (vector and
    scalar column access, several slabs, ragged edges), all operators, seeds, exclusive form."""
    rng = np.random.default_rng(5)
    for dt in (np.float32, np.float64, np.int32, np.float16):
        dt = np.dtype(dt)
        if dt.kind == "i":
            x = rng.integers(-3, 4, sizes).astype(dt)
        else:
            x = (rng.random(sizes) + 0.5).astype(dt)
        xd = gpu.ROCArray.from_host(x)
        for op in ("+", "max", "min") + (("*",) if dt.kind == "f" and dt.itemsize >= 4 else ()):
            xs = x if op != "*" else (0.9 + 0.2 * rng.random(sizes)).astype(dt)
            xsd = xd if op != "*" else gpu.ROCArray.from_host(xs)
            got = gpu.accumulate(op, xsd, dims=2, init=None).to_host()
            ref = orc.accumulate(op, xs, axis=1)
            if dt.kind == "i" or op in ("max", "min"):
                assert np.array_equal(got.astype(np.float64), np.asarray(ref, dtype=np.float64)), (sizes, dt, op)
            else:
                assert_close(got, ref, 1e-2 if dt.itemsize == 2 else 1e-5, (sizes, dt, op))
        seed = dt.type(2)
        got = gpu.accumulate("+", xd, dims=2, init=seed).to_host()
        ref = orc.accumulate("+", x, axis=1, init=seed)
        if dt.kind == "i":
            assert np.array_equal(got, ref)
        else:
            assert_close(got, ref, 1e-2 if dt.itemsize == 2 else 1e-5, (sizes, dt, "seeded"))
        if dt == np.int32:      # exclusive form: shifted by one row, starting from the seed
            out = gpu.ROCArray(dt, sizes)
            gpu.accumulate_("+", out, xd, dims=2, init=dt.type(0), inclusive=False)
            incl = np.cumsum(x, axis=1, dtype=dt)
            excl = np.concatenate([np.zeros_like(incl[:, :1]), incl[:, :-1]], axis=1)
            assert np.array_equal(out.to_host(), excl)
    # a destination view that starts at an odd element: scalar column access
    big = gpu.zeros(np.float32, sizes[0] * int(np.prod(sizes[1:])) + 1)
    dst = big.view(1, big.size).reshape(sizes)
    src = gpu.ROCArray.from_host(rng.random(sizes).astype(np.float32))
    gpu.accumulate_("+", dst, src, dims=2)
    assert_close(dst.to_host(), orc.accumulate("+", src.to_host(), axis=1), 1e-5)


@pytest.mark.parametrize("sizes", [(3, 1_000_000), (2, 4096), (4, 4097), (3, 100_003), (2, 70_000, 3), (3, 5000, 4), (4, 300_001)])
def test_scans_down_a_few_long_columns(gpu, orc, sizes):
    """accumulate(op, A; dims=2) with two to four interleaved columns (the reference benchmarks
    3 x 1 000 000): the kernel whose tiles hold all columns of a row range.  Every element size,
    all operators, seeded and exclusive forms, several slabs, a ragged last tile, in place, and an
    operand that starts off a 16-byte boundary."""
    rng = np.random.default_rng(6)
    for dt in (np.float32, np.float64, np.int32, np.int64, np.float16):
        dt = np.dtype(dt)
        if dt.kind == "i":
            x = rng.integers(-3, 4, sizes).astype(dt)
        elif dt.itemsize == 2:
            x = np.where(rng.random(sizes) < 0.5, 1.0, -1.0).astype(dt)      # partial sums stay small and exact
        else:
            x = (rng.random(sizes) - 0.25).astype(dt)
        xd = gpu.ROCArray.from_host(x)
        for op in ("+", "max", "min"):
            got = gpu.accumulate(op, xd, dims=2, init=None).to_host()
            ref = orc.accumulate(op, x, axis=1)
            if dt.kind == "i" or op in ("max", "min"):
                assert np.array_equal(got.astype(np.float64), np.asarray(ref, dtype=np.float64)), (sizes, dt, op)
            else:
                wide = np.cumsum(x.astype(np.float64), axis=1)
                tol = 5e-2 if dt.itemsize == 2 else (1e-4 if dt.itemsize == 4 else 1e-11)
                assert np.all(np.abs(got.astype(np.float64) - wide) <= tol * np.maximum(np.abs(wide), 1.0)), (sizes, dt, op)
        if dt.kind == "i":
            seed = dt.type(5)
            assert np.array_equal(gpu.accumulate("+", xd, dims=2, init=seed).to_host(), orc.accumulate("+", x, axis=1, init=seed)), (sizes, dt)
            out = gpu.ROCArray(dt, sizes)
            gpu.accumulate_("+", out, xd, dims=2, init=dt.type(-2), inclusive=False)
            incl = np.cumsum(x, axis=1, dtype=dt)
            excl = np.concatenate([np.zeros_like(incl[:, :1]), incl[:, :-1]], axis=1) - dt.type(2)
            assert np.array_equal(out.to_host(), excl), (sizes, dt)
            assert gpu.accumulate_("+", xd, xd, dims=2, init=None) is xd             # in place
            assert np.array_equal(xd.to_host(), incl), (sizes, dt)
    if len(sizes) == 2:
        # factors spread over a binade (no rounding ties): products of a million Float32 factors
        f = np.exp(rng.uniform(-1e-3, 1e-3, sizes)).astype(np.float32)
        got = gpu.accumulate("*", gpu.ROCArray.from_host(f), dims=2, init=None).to_host()
        assert_close(got, np.cumprod(f.astype(np.float64), axis=1), 1e-3, (sizes, "prod"))
        # an operand one element past a 16-byte boundary: element-wise accesses, same tiles
        n = sizes[0] * sizes[1]
        big = gpu.ROCArray.from_host(rng.integers(-3, 4, n + 1).astype(np.int32))
        src = big.view(1, n + 1).reshape(sizes)
        want = np.cumsum(big.to_host()[1:].reshape(sizes, order="F"), axis=1, dtype=np.int32)
        assert np.array_equal(gpu.accumulate("+", src, dims=2, init=None).to_host(), want), sizes


@pytest.mark.parametrize("sizes", [(512, 1000), (100, 70), (33, 64), (2048, 64), (1030, 65), (8192, 64), (36, 10, 20)])
def test_scans_down_many_contiguous_columns(gpu, orc, sizes):
    """accumulate(op, A; dims=1) with at least 64 columns of 33 elements to 8 KiB (the reference
    benchmarks 512 x 1000): one warp per column; longer columns take the tiled kernel.  Vector and element-wise accesses, ragged last
    steps, all operators, seeded, exclusive and in-place forms."""
    rng = np.random.default_rng(8)
    for dt in (np.float32, np.int64, np.float16, np.int32):
        dt = np.dtype(dt)
        x = rng.integers(-3, 4, sizes).astype(dt) if dt.kind == "i" else (rng.random(sizes) - 0.25).astype(dt)
        xd = gpu.ROCArray.from_host(x)
        for op in ("+", "max", "min"):
            got = gpu.accumulate(op, xd, dims=1, init=None).to_host()
            ref = orc.accumulate(op, x, axis=0)
            if dt.kind == "i" or op in ("max", "min"):
                assert np.array_equal(got.astype(np.float64), np.asarray(ref, dtype=np.float64)), (sizes, dt, op)
            else:
                wide = np.cumsum(x.astype(np.float64), axis=0)
                tol = 2e-2 if dt.itemsize == 2 else 1e-5
                assert np.all(np.abs(got.astype(np.float64) - wide) <= tol * np.maximum(np.abs(wide), 1.0)), (sizes, dt, op)
        if dt.kind == "i":
            seed = dt.type(7)
            assert np.array_equal(gpu.accumulate("+", xd, dims=1, init=seed).to_host(), orc.accumulate("+", x, axis=0, init=seed)), (sizes, dt)
            out = gpu.ROCArray(dt, sizes)
            gpu.accumulate_("+", out, xd, dims=1, init=dt.type(3), inclusive=False)
            incl = np.cumsum(x, axis=0, dtype=dt)
            excl = np.concatenate([np.zeros_like(incl[:1]), incl[:-1]], axis=0) + dt.type(3)
            assert np.array_equal(out.to_host(), excl), (sizes, dt)
            assert gpu.accumulate_("+", xd, xd, dims=1, init=None) is xd
            assert np.array_equal(xd.to_host(), incl), (sizes, dt)
    f = np.exp(rng.uniform(-1e-2, 1e-2, sizes)).astype(np.float32)
    assert_close(gpu.accumulate("*", gpu.ROCArray.from_host(f), dims=1, init=None).to_host(), np.cumprod(f.astype(np.float64), axis=0), 1e-4, (sizes, "prod"))


def test_long_vector_scan_forms(gpu, orc):
    """The persistent kernel for long dense vectors: in place, exclusive, seeded, max/min/prod, 16-bit
    elements, a last segment of every fill level, many launches in a row (descriptor words tagged
    with the launch number, never cleared in between) and a captured launch that is replayed."""
    rng = np.random.default_rng(9)
    tile = 8192                                   # sizes around multiples of 148 blocks x 8192 elements
    for n in (1 << 18, (1 << 18) + 4, 5 * tile - 4, 148 * tile, 149 * tile + 2044, 3 * 148 * tile + 12, (1 << 24) + 8):
        x = rng.integers(-100, 101, n).astype(np.int32)
        xd = gpu.ROCArray.from_host(x)
        ref = np.cumsum(x, dtype=np.int32)
        assert np.array_equal(gpu.cumsum(xd).to_host(), ref), n
        ex = gpu.accumulate_("+", gpu.ROCArray(np.int32, n), xd, init=np.int32(-9), inclusive=False).to_host()
        assert ex[0] == -9 and np.array_equal(ex[1:], (ref[:-1] - 9).astype(np.int32)), n
        assert gpu.accumulate_("+", xd, xd, init=None) is xd            # in place
        assert np.array_equal(xd.to_host(), ref), n
    n = (1 << 21) + 16
    w = rng.standard_normal(n).astype(np.float32)
    wd = gpu.ROCArray.from_host(w)
    assert np.array_equal(gpu.accumulate("max", wd, init=None).to_host(), np.maximum.accumulate(w))
    assert np.array_equal(gpu.accumulate("min", wd, init=np.float32(0.5)).to_host(), np.minimum.accumulate(np.minimum(w, 0.5)))
    # factors spread over a binade (no rounding ties); products of two million Float32 factors
    # carry the rounding of a tree of that depth, hence the wider tolerance
    g = np.exp(rng.uniform(-0.01, 0.01, n)).astype(np.float32)
    assert_close(gpu.cumprod(gpu.ROCArray.from_host(g)).to_host(), np.cumprod(g.astype(np.float64)), 5e-4)
    f = rng.random(n).astype(np.float32)
    assert_close(gpu.cumsum(gpu.ROCArray.from_host(f)).to_host(), np.cumsum(f.astype(np.float64)), 1e-5)
    h = np.where(np.arange(n) % 2 == 0, 1.0, -1.0).astype(np.float16)
    assert np.array_equal(gpu.cumsum(gpu.ROCArray.from_host(h)).to_host(), (np.arange(n) % 2 == 0).astype(np.float16))
    u = rng.integers(0, 1 << 31, n).astype(np.uint32)
    assert np.array_equal(gpu.cumsum(gpu.ROCArray.from_host(u)).to_host(), np.cumsum(u, dtype=np.uint32))
    # many launches back to back, then a captured launch replayed between ordinary ones
    x = rng.integers(-100, 101, 1 << 20).astype(np.int32)
    xd, out = gpu.ROCArray.from_host(x), gpu.ROCArray(np.int32, 1 << 20)
    ref = np.cumsum(x, dtype=np.int32)
    for _ in range(40):
        gpu.accumulate_("+", out, xd, init=None)
    assert np.array_equal(out.to_host(), ref)
    graph = gpu.captured(lambda: gpu.accumulate_("+", out, xd, init=None))
    for k in range(4):
        out.fill_(0)
        gpu.launch(graph)
        assert np.array_equal(out.to_host(), ref), k
        gpu.accumulate_("+", out, xd, init=np.int32(k))                   # ordinary launches in between
        assert np.array_equal(out.to_host(), (ref + k).astype(np.int32)), k
