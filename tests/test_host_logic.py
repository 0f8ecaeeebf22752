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


def test_sort_rejects_closures(pkg):
    with pytest.raises(ValueError):
        pkg.sorting._check_kwargs(lt=lambda a, b: a > b, by=None)
