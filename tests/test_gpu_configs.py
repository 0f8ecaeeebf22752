"""The five benchmark configurations at their full sizes, checked through properties that do
not need a full-size CPU recomputation where that would take minutes (sortedness, checksums,
permutation validity, stability), and against the oracle where NumPy finishes in seconds.
Inputs are generated on the device by the counter-based generator (synthetic stand-ins for
the seeded arrays of the workload definition)."""
import numpy as np
import pytest

from helpers import assert_close

pytestmark = pytest.mark.gpu


def test_config1_vectors_2p24(gpu, orc):
    R, n = gpu.random, 1 << 24
    x = R.fill_random_(gpu.ROCArray(np.float32, n), R.UNIFORM01, seed=0, stream_id=0)
    y = R.fill_random_(gpu.ROCArray(np.float32, n), R.UNIFORM01, seed=0, stream_id=1)
    xh, yh = x.to_host(), y.to_host()
    assert np.array_equal(xh, R.host_uniform01(0, 0, 0, n))
    a = np.float32(2.5)
    z = gpu.ROCArray(np.float32, n)
    gpu.materialize_(z, a * x.dot + y.dot)
    assert np.array_equal(z.to_host(), a * xh + yh)
    assert_close(gpu.sum(x), xh.astype(np.float64).sum(), 1e-5)
    assert_close(gpu.cumsum(x).to_host(), np.cumsum(xh, dtype=np.float64), 1e-5)


@pytest.mark.parametrize("dt", ["float32", "float16", "bfloat16"])
def test_config2_matrix_8192(gpu, dt):
    import ml_dtypes
    dt = np.dtype(ml_dtypes.bfloat16) if dt == "bfloat16" else np.dtype(dt)
    R, m = gpu.random, 8192
    A = R.fill_random_(gpu.ROCArray(dt, (m, m)), R.NORMAL, seed=1)
    Ah = A.to_host().astype(np.float64)
    tol = 1e-5 if dt == np.float32 else 1e-2
    # sums of N(0,1) columns cancel: compare against the Float64 sum with the tolerance scaled
    # by the sum of magnitudes (the conditioning of the problem), as for any summation bound
    s1 = gpu.ROCArray(np.float32, (1, m))
    gpu.mapreducedim_("identity", "+", s1, A, init=np.float32(0))
    ref = Ah.sum(axis=0, keepdims=True)
    mag = np.abs(Ah).sum(axis=0, keepdims=True)
    assert np.all(np.abs(s1.to_host() - ref) <= tol * mag)
    mx = gpu.maximum(A, dims=2)
    assert mx.dims == (m, 1) and np.array_equal(mx.to_host().astype(np.float64), Ah.max(axis=1, keepdims=True))
    sq = gpu.ROCArray(np.float32, (1, 1))
    gpu.mapreducedim_("abs2", "+", sq, A, init=np.float32(0))
    assert_close(sq.to_host(), (Ah * Ah).sum().reshape(1, 1), tol)


def test_config3_scans_2p28(gpu):
    R, n = gpu.random, 1 << 28
    v = R.fill_random_(gpu.ROCArray(np.int32, n), R.INTEGERS, seed=2, lo=-100, hi=100)
    vh = v.to_host()
    out = gpu.accumulate("+", v).to_host()
    assert np.array_equal(out, np.cumsum(vh, dtype=np.int32))
    del out, vh
    f = R.fill_random_(gpu.ROCArray(np.float32, n), R.UNIFORM01, seed=2, stream_id=1)
    fh = f.to_host()
    got = gpu.accumulate("+", f).to_host()
    ref = np.cumsum(fh, dtype=np.float64)
    step = 1 << 26                           # bounded temporaries
    for s in range(0, n, step):
        assert np.all(np.abs(got[s:s + step] - ref[s:s + step]) <= 1e-5 * ref[s:s + step] + 1e-6)


def test_config4_sort_2p28_and_sortperm_2p26(gpu):
    R, n = gpu.random, 1 << 28
    k = R.fill_random_(gpu.ROCArray(np.uint32, n), R.RAWBITS, seed=3)
    kh = k.to_host()
    sums = (int(kh.sum(dtype=np.uint64)), int(np.bitwise_xor.reduce(kh)),
            int((kh.astype(np.uint64) * kh.astype(np.uint64)).sum(dtype=np.uint64)))
    gpu.sort_(k)
    sh = k.to_host()
    assert np.all(sh[1:] >= sh[:-1])                                    # sorted
    assert sums == (int(sh.sum(dtype=np.uint64)), int(np.bitwise_xor.reduce(sh)),
                    int((sh.astype(np.uint64) * sh.astype(np.uint64)).sum(dtype=np.uint64)))   # same multiset (checksums)
    q = np.linspace(0, n - 1, 1001).astype(np.int64)
    assert np.array_equal(sh[q], np.partition(kh, q)[q])                # order statistics agree
    del kh, sh
    m = 1 << 26
    f = R.fill_random_(gpu.ROCArray(np.float32, m), R.NORMAL_DUP1PCT, seed=3, hi=m)
    fh = f.to_host()
    p = gpu.sortperm(f).to_host()
    assert p.dtype == np.int64 and p.min() == 1 and p.max() == m
    seen = np.zeros(m, dtype=bool)
    seen[p - 1] = True
    assert seen.all()                                                    # a permutation
    g = fh[p - 1]
    assert np.all(g[1:] >= g[:-1])                                       # keys ascend
    ties = g[1:] == g[:-1]
    assert ties.sum() > m // 400 and np.all(p[1:][ties] > p[:-1][ties])  # stable among equal keys
    assert np.array_equal(f.to_host(), fh)


def test_config5_shard_2p30(gpu, orc):
    R, n = gpu.random, 1 << 30                        # the per-GPU shard of the 2^33 / 8-GPU workload
    x, y, z = (R.fill_random_(gpu.ROCArray(np.float32, n), R.UNIFORM11, seed=4, stream_id=s) for s in range(3))
    r = gpu.ROCArray(np.float32, n)
    bc = gpu.broadcast
    gpu.materialize_(r, x.dot * y.dot + bc.exp(-bc.abs_(z)))
    total = gpu.sum(r, f="abs2")
    ref_total = 0.0
    chunk = 1 << 26
    for s in (0, 5 * chunk, n - chunk):              # spot-checked chunks
        xs, ys, zs = (R.host_uniform11(4, k, s, chunk) for k in range(3))
        want = orc.broadcast(("add", ("mul", xs, ys), ("exp", ("neg", ("abs", zs)))))
        got = r.view(s, s + chunk).to_host()
        assert np.allclose(got, want, rtol=1e-6, atol=3e-7)
    # the reduction against a Float64 sum of the device's own r, streamed in chunks
    for s in range(0, n, chunk):
        c = r.view(s, s + chunk).to_host().astype(np.float64)
        ref_total += float((c * c).sum())
    assert_close(total, ref_total, 1e-5)


def test_more_than_2p32_elements_on_one_gpu(gpu, orc):
    """Config 5 on a single GPU holds 2^33 elements per array; here broadcast and reduction run
    over 2^32 + 5 Float32 elements (index arithmetic beyond 32 bits, ragged tail).  Checked at the
    2^32 boundary and at the tail against the host, and through linearity: the sum over the whole
    array equals the sum of the sums over two parts that each stay below 2^32 elements."""
    R, n = gpu.random, (1 << 32) + 5
    free, _ = gpu.mem_info()
    if free < 40 << 30:
        pytest.skip("needs 40 GiB of free device memory")
    x = R.fill_random_(gpu.ROCArray(np.float32, n), R.UNIFORM11, seed=4, stream_id=0)
    r = gpu.ROCArray(np.float32, n)
    bc = gpu.broadcast
    gpu.materialize_(r, x.dot * x.dot + bc.exp(-bc.abs_(x)))
    for s, e in ((0, 4096), ((1 << 31) - 2048, (1 << 31) + 2048), ((1 << 32) - 4096, n)):
        xs = R.host_uniform11(4, 0, s, e - s)
        assert np.array_equal(x.view(s, e).to_host(), xs)
        want = orc.broadcast(("add", ("mul", xs, xs), ("exp", ("neg", ("abs", xs)))))
        assert np.allclose(r.view(s, e).to_host(), want, rtol=1e-6, atol=3e-7), (s, e)
    total = float(gpu.sum(r, f="abs2"))
    cut = (1 << 31) + 12
    parts = float(gpu.sum(r.view(0, cut), f="abs2")) + float(gpu.sum(r.view(cut, n), f="abs2"))
    assert abs(total - parts) <= 1e-5 * parts
    # U[-1,1): E[(x^2 + exp(-|x|))^2] = 1/5 + 2(2 - 5/e) + (1 - e^-2)/2 = 0.95344...
    assert abs(total / n - (0.2 + 2 * (2 - 5 / np.e) + (1 - np.exp(-2.0)) / 2)) < 1e-3
