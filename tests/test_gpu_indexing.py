"""findall / logical indexing / reverse against NumPy (the reference's tests:
test/hip_rocarray/indexing.jl:5-18, test/hip_rocarray/reverse.jl:5-51)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_findall_and_logical_indexing(gpu):
    rng = np.random.default_rng(0)
    for shape in ((0,), (1,), (10,), (4097,), (33, 77), (5, 6, 7), (1_000_003,)):
        b = rng.random(shape) < 0.3
        x = rng.random(shape).astype(np.float32)
        bd, xd = gpu.ROCArray.from_host(b), gpu.ROCArray.from_host(x)
        want = np.flatnonzero(b.reshape(-1, order="F")) + 1
        got = gpu.findall(bd)
        assert got.dtype == np.int64 and np.array_equal(got.to_host(), want), shape
        assert np.array_equal(gpu.getindex_mask(xd, bd).to_host(), x.reshape(-1, order="F")[want - 1]), shape
    assert gpu.findall(gpu.ROCArray.from_host(np.zeros(100, bool))).dims == (0,)
    assert np.array_equal(gpu.findall(gpu.ROCArray.from_host(np.ones(100, bool))).to_host(), np.arange(1, 101))


def test_reverse(gpu):
    rng = np.random.default_rng(1)
    for dt in (np.float32, np.int64, np.float16, np.uint8):
        v = (rng.random(10_001) * 100).astype(dt)
        vd = gpu.ROCArray.from_host(v)
        assert np.array_equal(gpu.reverse(vd).to_host(), v[::-1])
        assert np.array_equal(vd.to_host(), v)
        assert gpu.reverse_(vd) is vd and np.array_equal(vd.to_host(), v[::-1])
    a = rng.random((7, 5, 3)).astype(np.float32)
    ad = gpu.ROCArray.from_host(a)
    assert np.array_equal(gpu.reverse(ad).to_host(), a[::-1, ::-1, ::-1])
    assert np.array_equal(gpu.reverse(ad, dims=1).to_host(), a[::-1])
    assert np.array_equal(gpu.reverse(ad, dims=2).to_host(), a[:, ::-1])
    assert np.array_equal(gpu.reverse(ad, dims=(1, 3)).to_host(), a[::-1, :, ::-1])
    assert np.array_equal(gpu.reverse_(ad, dims=3).to_host(), a[:, :, ::-1])
    with pytest.raises(ValueError):
        gpu.reverse(ad, dims=4)


def test_compaction_checks_its_positions(gpu):
    """Through the C ABI with a destination one element too short and with positions that do not
    belong to the mask: the kernel skips the stores it may not make and the next synchronisation
    reports B200_INVALID_ARG; nothing is written out of bounds, the context stays usable."""
    import ctypes as C
    L = gpu._lib
    mask = np.array([1, 0, 1, 1, 0, 1], dtype=bool)
    pos = np.cumsum(mask).astype(np.int64)
    md, pd_ = gpu.ROCArray.from_host(mask), gpu.ROCArray.from_host(pos)
    guard = gpu.ROCArray(np.int64, 8).fill_(-7)
    short = guard.view(0, 3)                       # 4 true entries, room for 3
    ty, tb, ti = short.tensor(), md.tensor(), pd_.tensor()
    assert L.lib.b200_compact(gpu.current_stream().handle, C.byref(ty), C.byref(tb), C.byref(ti), None) == L.OK
    with pytest.raises(gpu.B200Error) as ei:
        gpu.synchronize()
    assert ei.value.code == L.INVALID_ARG
    assert np.array_equal(guard.to_host(), [1, 3, 4, -7, -7, -7, -7, -7])
    bad = gpu.ROCArray.from_host(np.array([0, 0, -3, 99, 0, 2], dtype=np.int64))
    full = gpu.ROCArray(np.int64, 4).fill_(-7)
    ty, ti = full.tensor(), bad.tensor()
    assert L.lib.b200_compact(gpu.current_stream().handle, C.byref(ty), C.byref(tb), C.byref(ti), None) == L.OK
    with pytest.raises(gpu.B200Error):
        gpu.synchronize()
    assert np.array_equal(full.to_host(), [-7, 6, -7, -7])
    assert np.array_equal(gpu.findall(md).to_host(), [1, 3, 4, 6])


def test_mask_along_one_dimension(gpu):
    """xd[:, md] and xd[:, :, md] (test/hip_rocarray/indexing.jl:9-18), plus a mask in the middle."""
    rng = np.random.default_rng(2)
    for shape, dim in (((1, 16), 2), ((3, 1, 16), 3), ((5, 300), 2), ((40, 7, 9), 2), ((33, 4), 1), ((6,), 1)):
        x = rng.integers(-1000, 1000, shape).astype(np.int32)
        m = rng.random(shape[dim - 1]) < 0.5
        xd, md = gpu.ROCArray.from_host(x), gpu.ROCArray.from_host(m)
        want = np.compress(m, x, axis=dim - 1)
        got = gpu.getindex_mask_dim(xd, md, dim)
        assert got.dims == want.shape and np.array_equal(got.to_host(), want), (shape, dim)
    none = gpu.getindex_mask_dim(gpu.ROCArray.from_host(np.ones((3, 4), np.float32)), gpu.ROCArray.from_host(np.zeros(4, bool)), 2)
    assert none.dims == (3, 0)
    with pytest.raises(IndexError):
        gpu.getindex_mask_dim(gpu.ROCArray(np.float32, (3, 4)), gpu.ROCArray.from_host(np.zeros(3, bool)), 2)


def test_vector_paths_and_their_edges(gpu):
    """The 16-byte forms of reverse, gather and compaction and the shapes that fall back to the
    element-wise forms: first dimensions that hold a whole number of vectors or not, every
    element size, flips of several dimensions at once, operands that start off a 16-byte boundary
    (views), lengths that are not a multiple of four, Int32 index vectors."""
    rng = np.random.default_rng(3)
    for dt in (np.uint8, np.float16, np.float32, np.float64):
        for shape in ((64, 9, 5), (48,), (16, 3), (20, 6), (4096, 33)):
            a = (rng.random(shape) * 200).astype(dt)
            ad = gpu.ROCArray.from_host(a)
            nd = len(shape)
            for dims in [None] + list(range(1, nd + 1)) + ([(1, nd)] if nd > 1 else []):
                sl = tuple(slice(None, None, -1) if (dims is None or d + 1 == dims or (isinstance(dims, tuple) and d + 1 in dims))
                           else slice(None) for d in range(nd))
                assert np.array_equal(gpu.reverse(ad, dims=dims).to_host(), a[sl]), (dt, shape, dims)
    v = rng.integers(-1000, 1000, 10_003).astype(np.int32)
    vd = gpu.ROCArray.from_host(v)
    off = vd.view(1, 10_001)                                   # starts 4 bytes past a 16-byte boundary
    assert np.array_equal(gpu.reverse(off).to_host(), v[1:10_001][::-1])
    # gather: lengths around multiples of four, both index types, an index vector off the boundary
    x = rng.standard_normal(5000).astype(np.float32)
    xd = gpu.ROCArray.from_host(x)
    for n in (1, 3, 4, 5, 1023, 1024, 4099):
        for it in (np.int64, np.int32):
            ix = rng.integers(1, 5001, n).astype(it)
            assert np.array_equal(gpu.getindex(xd, gpu.ROCArray.from_host(ix)).to_host(), x[ix - 1]), (n, it)
    ix = rng.integers(1, 5001, 2002).astype(np.int64)
    ixd = gpu.ROCArray.from_host(ix)
    assert np.array_equal(gpu.getindex(xd, ixd.view(1, 2002)).to_host(), x[ix[1:2002] - 1])
    for dt in (np.uint8, np.float16, np.float64):
        y = (rng.random(777) * 100).astype(dt)
        ix = rng.integers(1, 778, 1001).astype(np.int64)
        assert np.array_equal(gpu.getindex(gpu.ROCArray.from_host(y), gpu.ROCArray.from_host(ix)).to_host(), y[ix - 1])
    # compaction: a mask that starts off the boundary, all element sizes, sparse and dense masks
    for n in (5, 4096, 100_003):
        for p in (0.01, 0.5, 0.99):
            m = rng.random(n) < p
            md = gpu.ROCArray.from_host(m)
            want = np.flatnonzero(m) + 1
            assert np.array_equal(gpu.findall(md).to_host(), want), (n, p)
            if n > 8:
                assert np.array_equal(gpu.findall(md.view(3, n)).to_host(), np.flatnonzero(m[3:]) + 1), (n, p)
            for dt in (np.uint8, np.int16, np.float32, np.float64):
                xs = (rng.random(n) * 100).astype(dt)
                assert np.array_equal(gpu.getindex_mask(gpu.ROCArray.from_host(xs), md).to_host(), xs[m]), (n, p, dt)
