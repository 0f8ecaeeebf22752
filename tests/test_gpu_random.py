"""Device generator against its NumPy restatement."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_draws_match_host(gpu):
    R = gpu.random
    n = 100_003
    u = R.fill_random_(gpu.ROCArray(np.float32, n), R.UNIFORM01, seed=0, stream_id=1).to_host()
    assert np.array_equal(u, R.host_uniform01(0, 1, 0, n))
    s = R.fill_random_(gpu.ROCArray(np.float32, 1000), R.UNIFORM11, seed=4, stream_id=2, first_index=5000).to_host()
    assert np.array_equal(s, R.host_uniform11(4, 2, 5000, 1000)) and s.min() >= -1 and s.max() < 1
    i = R.fill_random_(gpu.ROCArray(np.int32, n), R.INTEGERS, seed=2, lo=-100, hi=100).to_host()
    assert np.array_equal(i, R.host_integers(2, 0, 0, n, -100, 100))
    k = R.fill_random_(gpu.ROCArray(np.uint32, n), R.RAWBITS, seed=3).to_host()
    assert np.array_equal(k, R.host_rawbits(3, 0, 0, n))
    g = R.fill_random_(gpu.ROCArray(np.float32, 1 << 20), R.NORMAL, seed=1).to_host()
    assert abs(g.mean()) < 0.01 and abs(g.std() - 1) < 0.01 and np.isfinite(g).all()
    d = R.fill_random_(gpu.ROCArray(np.float32, 1 << 20), R.NORMAL_DUP1PCT, seed=3, hi=1 << 20).to_host()
    dup = (1 << 20) - len(np.unique(d))
    assert 0.005 * (1 << 20) < dup < 0.02 * (1 << 20)
    h = R.fill_random_(gpu.ROCArray(np.float16, 1000), R.NORMAL, seed=1).to_host()
    assert np.allclose(h.astype(np.float32), g[:1000], rtol=1e-3, atol=1e-3)
