"""The allocation-free scan entry point against the regular one, through the C ABI.

Who needs it: callers that cannot allocate while they run - a process that handed the whole
device to its own arena, a plug-in under a host that forbids allocations after start-up, a loop
with a fixed latency budget.  `b200_accumulate_noalloc` keeps the scan's tile descriptors in an
array built into the library instead of pool memory.  The file name sorts last so that a run
stopping at the first failure has already executed every other test; the test also passes alone
in a fresh process (it sets up everything it uses).
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _scan(gpu, fn, out, src, op, init, dim=0, inclusive=1):
    L = gpu._lib
    tb, ta = out.tensor(), src.tensor()
    ib = None if init is None else np.asarray(init, dtype=src.dtype).tobytes()
    return fn(gpu.current_stream().handle, C.byref(tb), C.byref(ta), op, ib, dim, inclusive)


def test_noalloc_scan_matches_regular_entry_point(gpu):
    L = gpu._lib
    regular, noalloc = L.lib.b200_accumulate, L.lib.b200_accumulate_noalloc
    rng = np.random.default_rng(0)
    live_before = None
    # two calls in a row (different sizes and types: the second call sees the first one's leftovers)
    for round_ in range(2):
        for dt, n, init in ((np.int32, 1_000_003, np.int32(7)), (np.float32, 300_001, None),
                            (np.int64, 50_000, np.int64(-3)), (np.int32, 4097, None)):
            x = rng.integers(-100, 101, n).astype(dt) if np.dtype(dt).kind == "i" else rng.random(n).astype(dt)
            src = gpu.ROCArray.from_host(x)
            a, b = gpu.ROCArray(dt, n), gpu.ROCArray(dt, n)
            gpu.synchronize()
            if live_before is None:
                live_before = gpu.pool_stats()["alloc_count"]
            assert _scan(gpu, regular, a, src, L.RED_ADD, init) == L.OK, L.last_error()
            allocs = gpu.pool_stats()["alloc_count"]
            assert _scan(gpu, noalloc, b, src, L.RED_ADD, init) == L.OK, L.last_error()
            assert gpu.pool_stats()["alloc_count"] == allocs          # the variant took nothing from the pool
            gpu.synchronize()
            ha, hb = a.to_host(), b.to_host()
            if np.dtype(dt).kind == "i":
                assert np.array_equal(ha, hb), (round_, dt, n)
            else:   # look-back order may differ between two runs: same tolerance as the scan tests
                ref = np.cumsum(x, dtype=np.float64)
                assert np.all(np.abs(hb - ref) <= 1e-5 * np.abs(ref) + 1e-6) and np.allclose(ha, hb, rtol=1e-5)
    # matrices: along the contiguous and the strided dimension
    m = rng.integers(-9, 10, (300, 70)).astype(np.int64)
    src = gpu.ROCArray.from_host(m)
    for dim in (0, 1):
        a, b = gpu.ROCArray(np.int64, m.shape), gpu.ROCArray(np.int64, m.shape)
        assert _scan(gpu, regular, a, src, L.RED_ADD, None, dim) == L.OK
        assert _scan(gpu, noalloc, b, src, L.RED_ADD, None, dim) == L.OK
        assert np.array_equal(a.to_host(), b.to_host()) and np.array_equal(b.to_host(), np.cumsum(m, axis=dim))


def test_noalloc_scan_other_forms(gpu):
    """Exclusive scans, a max-scan, Float16 elements (tiles of 8192) and the shape that needs no
    bookkeeping at all (columns of at most 32 elements, one thread per column)."""
    L = gpu._lib
    regular, noalloc = L.lib.b200_accumulate, L.lib.b200_accumulate_noalloc
    rng = np.random.default_rng(1)
    cases = (
        (rng.integers(-100, 101, 200_003).astype(np.int32), L.RED_ADD, np.int32(5), 0, 0),      # exclusive
        (rng.standard_normal(100_001).astype(np.float32), L.RED_MAX, None, 0, 1),                # max-scan
        (np.where(np.arange(70_000) % 2 == 0, 1, -1).astype(np.float16), L.RED_ADD, None, 0, 1),  # 16-bit tiles
        (rng.integers(-9, 10, (20, 2048)).astype(np.int64), L.RED_ADD, None, 0, 1),              # short columns
        (rng.integers(-9, 10, (20, 2048)).astype(np.int64), L.RED_ADD, np.int64(3), 0, 0),
    )
    for x, op, init, dim, inclusive in cases:
        src = gpu.ROCArray.from_host(x)
        a, b = gpu.ROCArray(x.dtype, x.shape), gpu.ROCArray(x.dtype, x.shape)
        assert _scan(gpu, regular, a, src, op, init, dim, inclusive) == L.OK, L.last_error()
        allocs = gpu.pool_stats()["alloc_count"]
        assert _scan(gpu, noalloc, b, src, op, init, dim, inclusive) == L.OK, L.last_error()
        assert gpu.pool_stats()["alloc_count"] == allocs
        assert np.array_equal(a.to_host(), b.to_host()), (x.dtype, x.shape, op, inclusive)


def test_noalloc_scan_refuses_oversized_input(gpu):
    L = gpu._lib
    # 33 x 150000: every column takes a tile of its own, more tiles than the built-in array holds
    src = gpu.zeros(np.float32, (33, 150_000))
    out = gpu.ROCArray(np.float32, (33, 150_000))
    st = _scan(gpu, L.lib.b200_accumulate_noalloc, out, src, L.RED_ADD, None, 0)
    assert st == L.TOO_LARGE and "built-in" in L.last_error()
    assert _scan(gpu, L.lib.b200_accumulate, out, src, L.RED_ADD, None, 0) == L.OK      # the regular entry point takes it
    gpu.synchronize()
