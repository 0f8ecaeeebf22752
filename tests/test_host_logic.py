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
