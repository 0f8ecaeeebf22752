"""Host-side logic of the operator mirror: promotion, program flattening, limits, shards."""
import numpy as np
import pytest


class FakeArray:
    pass


def test_promote_type_matches_oracle(pkg, orc):
    L = pkg._lib
    dts = [np.float16, np.float32, np.float64, np.int8, np.int16, np.int32, np.int64,
           np.uint8, np.uint16, np.uint32, np.uint64, np.bool_]
    for a in dts:
        for b in dts:
            got = L.dtype_numpy(pkg.promote_type(L.dtype_code(a), L.dtype_code(b)))
            assert got == orc.promote(a, b), (a, b)
    assert pkg.promote_type(L.F16, L.BF16) == L.F32


def test_parse_memory_limit(pkg):
    total = 180 * 1024**3
    assert pkg.parse_memory_limit("none", total) == (1 << 64) - 1
    assert pkg.parse_memory_limit("8 GiB", total) == 8 * 1024**3
    assert pkg.parse_memory_limit("512 MiB", total) == 512 * 1024**2
    assert pkg.parse_memory_limit("50 %", total) == total // 2
    for bad in ("8GiB", "8 GB", "0 %", "101 %", "400 GiB"):
        with pytest.raises(ValueError):
            pkg.parse_memory_limit(bad, total)


def test_shard_range_partitions(pkg):
    sr = pkg.sharded.shard_range
    for n in (0, 1, 5, 1000, 2**20 + 3, 2**33):
        for world in (1, 2, 4, 8):
            spans = [sr(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b
            assert all(lo % 4 == 0 for lo, hi in spans if hi > lo)
    assert sr(2**33, 3, 8) == (3 * 2**30, 4 * 2**30)


def test_scalar_leaf_types(pkg):
    B, L = pkg.Broadcasted, pkg._lib
    assert B.leaf(2).dtype == L.I64 and B.leaf(2.5).dtype == L.F64
    assert B.leaf(np.float32(2.5)).dtype == L.F32 and B.leaf(True).dtype == L.BOOL
    with pytest.raises(TypeError):
        B.leaf([1, 2, 3])
    with pytest.raises(ValueError):
        B.call("sin", 1.0)


def test_sort_order_keywords(pkg):
    order = pkg.sorting._order
    assert order(False, None) is False and order(True, None) is True
    assert order(False, "<") is False and order(False, ">") is True and order(False, "!isless") is True
    assert order(True, ">") is False                  # reversed twice
    with pytest.raises(ValueError):
        order(False, lambda a, b: a > b)              # closures cannot run inside a radix sort
    with pytest.raises(ValueError):
        order(False, ">=")


class _FakeBuffer:
    """Stands in for pool memory so that view geometry can be checked without a device."""
    ptr, freed, stream = 1 << 20, False, None


def test_view_geometry_matches_numpy(pkg):
    shape = (6, 5, 4)
    host = np.asfortranarray(np.arange(np.prod(shape), dtype=np.float32).reshape(shape, order="F"))
    A = pkg.ROCArray(np.float32, shape, _buf=_FakeBuffer())
    assert A.is_contiguous and A.strides == (1, 6, 30)

    def same(view, ref):
        assert view.dims == ref.shape
        assert view.strides == tuple(s // 4 for s in ref.strides)
        assert view.ptr - A.ptr == ref.__array_interface__["data"][0] - host.__array_interface__["data"][0]

    same(A.subview(slice(1, 5), slice(None), slice(None)), host[1:5])
    same(A.subview(slice(0, 6, 2), 3, slice(1, 4)), host[0:6:2, 3, 1:4])
    same(A.subview(2, slice(None), 1), host[2, :, 1])
    same(A.permuteddims((3, 1, 2)), host.transpose(2, 0, 1))
    M = A.subview(slice(None), slice(None), 0)
    same(M.transpose(), host[:, :, 0].T)
    assert not M.transpose().is_contiguous and M.is_contiguous
    assert A.subview(slice(None), slice(None), slice(0, 1)).is_contiguous       # extent-1 dims do not matter
    row = pkg.ROCArray(np.float32, (7,), _buf=_FakeBuffer()).transpose()
    assert row.dims == (1, 7) and row.is_contiguous
    with pytest.raises(ValueError):
        A.subview(slice(0, 6, 2), slice(None), slice(None)).reshape(60)
    with pytest.raises(IndexError):
        A.subview(6, slice(None), slice(None))
    with pytest.raises(ValueError):
        A.permuteddims((1, 1, 2))


def test_alloc_cache_reuses_buffers(pkg, monkeypatch):
    """GPUArrays.@cached semantics with the allocator faked: the second pass through a cached
    block makes no allocator call, frees inside the block are no-ops, unsafe_free_ returns all."""
    import sys
    arr = sys.modules[pkg.ROCArray.__module__]
    mem = sys.modules[pkg.AllocCache.__module__]
    calls = {"alloc": 0, "free": []}

    def fake_alloc(nbytes, stream=None):
        calls["alloc"] += 1
        return 0x1000 * calls["alloc"]

    monkeypatch.setattr(arr, "pool_alloc", fake_alloc)
    monkeypatch.setattr(arr, "pool_free", lambda ptr, stream=None: calls["free"].append(ptr))
    monkeypatch.setattr(mem, "pool_free", lambda ptr, stream=None: calls["free"].append(ptr))

    class FakeStream:
        device, handle = 0, 1

    def block():
        a = pkg.ROCArray(np.float32, (4, 4), stream=FakeStream())
        b = pkg.ROCArray(np.float32, (4, 4), stream=FakeStream())
        c = pkg.ROCArray(np.int64, 3, stream=FakeStream())
        ptrs = (a.ptr, b.ptr, c.ptr)
        a.unsafe_free_()                      # no-op: the cache owns it
        return ptrs

    cache = pkg.AllocCache()
    with pkg.cached(cache):
        first = block()
    assert calls["alloc"] == 3 and calls["free"] == []
    assert cache.sizeof() == 64 + 64 + 24
    with pkg.cached(cache):
        second = block()
    assert calls["alloc"] == 3                # everything came back from the cache
    assert sorted(second) == sorted(first)
    outside = pkg.ROCArray(np.float32, (4, 4), stream=FakeStream())      # not cached
    assert calls["alloc"] == 4
    outside.unsafe_free_()
    assert calls["free"] == [outside.buf.ptr]
    cache.unsafe_free_()
    assert sorted(calls["free"][1:]) == sorted(first) and cache.sizeof() == 0


def test_pool_cleanup_policy(pkg):
    """pool_cleanup (src/memory.jl:289-321): trim a device's pool after five idle looks in a row."""
    counts = {0: 10, 1: 5}
    trimmed = []
    pc = pkg.PoolCleanup(lambda: [0, 1], lambda d: counts[d], trimmed.append, interval=3600, idle_periods=5)
    assert pc.step() == []                    # first look only records the counters
    for i in range(4):
        counts[1] += 1                        # device 1 stays busy
        assert pc.step() == []
    assert pc.step() == [0] and trimmed == [0]
    counts[0] += 1                            # activity resets the idle count
    assert pc.step() == []
    assert pc.step() == [] and pc.step() == []
    assert pc.step() == [1] and trimmed == [0, 1]     # device 1 has now been idle five looks in a row
