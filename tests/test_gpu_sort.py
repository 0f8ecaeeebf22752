"""sort! / sortperm on the device: bit-exact against the stable isless oracle."""
from pathlib import Path

import numpy as np
import pytest

from helpers import bits_equal

pytestmark = pytest.mark.gpu
G = np.load(Path(__file__).parent / "golden" / "known_answers.npz")
SZ = (1, 2, 3, 4, 33, 333, 3333, 4096, 8191, 8192, 8193, 100_003)
try:
    import ml_dtypes
    BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:
    BF16 = None


def keys(rng, n, dt):
    dt = np.dtype(dt)
    if dt.kind == "u":
        return rng.integers(0, np.iinfo(dt).max, n, dtype=dt, endpoint=True)
    if dt.kind == "i":
        return rng.integers(np.iinfo(dt).min, np.iinfo(dt).max, n, dtype=dt, endpoint=True)
    return rng.standard_normal(n).astype(dt)


def test_golden_order(gpu):
    x = gpu.ROCArray.from_host(G["order_in"])
    s = gpu.sort(x).to_host()
    assert bits_equal(s[:-1], G["order_sorted"][:-1]) and np.isnan(s[-1])
    assert np.array_equal(gpu.sortperm(x).to_host(), G["order_perm"])
    assert np.array_equal(gpu.sortperm(x, rev=True).to_host(), G["order_perm_rev"])
    assert bits_equal(x.to_host()[:3], G["order_in"][:3])          # sortperm leaves the keys alone
    r = gpu.ROCArray.from_host(np.arange(100_000, 0, -1, dtype=np.int32))
    assert np.array_equal(gpu.sort_(r).to_host(), np.arange(1, 100_001, dtype=np.int32))
    e = gpu.ROCArray.from_host(np.full(10_001, 4.0, np.float32))
    assert np.array_equal(gpu.sortperm(e).to_host(), np.arange(1, 10_002))
    assert np.array_equal(gpu.sortperm(e, rev=True).to_host(), np.arange(1, 10_002))
    assert gpu.sort(gpu.ROCArray(np.float32, 0)).dims == (0,)


@pytest.mark.parametrize("dt", [np.float16, np.float32, np.float64, np.int16, np.int32, np.int64, np.uint16, np.uint32, np.uint64, "bf16"])
def test_sort_and_sortperm(gpu, orc, dt):
    if dt == "bf16":
        if BF16 is None:
            pytest.skip("no bfloat16 host type")
        dt = BF16
    dt = np.dtype(dt)
    rng = np.random.default_rng(3)
    for n in SZ:
        x = keys(rng, n, dt)
        if n > 100:
            x[:: max(2, n // 50)] = x[1]              # duplicates: stability is observable
        xd = gpu.ROCArray.from_host(x)
        for rev in (False, True):
            assert bits_equal(gpu.sort(xd, rev=rev).to_host(), orc.sort(x, rev=rev)), (dt, n, rev)
            p = gpu.sortperm(xd, rev=rev)
            assert p.dtype == np.int64
            assert np.array_equal(p.to_host(), orc.sortperm(x, rev=rev)), (dt, n, rev)
        assert bits_equal(xd.to_host(), x)
    if dt.kind == "f" or dt == BF16:
        x = keys(rng, 5000, dt)
        x[::7] = np.nan
        x[1::11] = -0.0
        x[2::13] = 0.0
        x[3::17] = np.inf
        x[4::19] = -np.inf
        xd = gpu.ROCArray.from_host(x)
        assert np.array_equal(gpu.sortperm(xd).to_host(), orc.sortperm(x))
        s, ref = gpu.sort(xd).to_host(), orc.sort(x)
        m = ~np.isnan(ref.astype(np.float64))
        assert np.array_equal(np.isnan(s.astype(np.float64)), ~m) and bits_equal(s[m], ref[m])


def test_low_entropy_and_in_place(gpu, orc):
    rng = np.random.default_rng(4)
    x = rng.integers(0, 4, 300_000).astype(np.uint32)          # most digits identical
    assert np.array_equal(gpu.sort(gpu.ROCArray.from_host(x)).to_host(), np.sort(x))
    assert np.array_equal(gpu.sortperm(gpu.ROCArray.from_host(x)).to_host(), orc.sortperm(x))
    xd = gpu.ROCArray.from_host(x)
    assert gpu.sort_(xd) is xd and np.array_equal(xd.to_host(), np.sort(x))
    outs = [gpu.sortperm(gpu.ROCArray.from_host(x)).to_host() for _ in range(3)]
    assert all(np.array_equal(outs[0], o) for o in outs)
