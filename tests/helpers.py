import numpy as np

SIZES = (1, 2, 3, 10, 33, 333, 3333, 4096, 4097, 10_000, 16384, 16385, 100_003, (1 << 20) + 7)


def assert_close(got, ref64, rtol, what="", atol=1e-30):
    got = np.asarray(got, dtype=np.float64)
    ref64 = np.asarray(ref64, dtype=np.float64)
    assert got.shape == ref64.shape, (what, got.shape, ref64.shape)
    nan_ok = np.isnan(got) == np.isnan(ref64)
    assert nan_ok.all(), (what, "NaN pattern differs")
    m = ~np.isnan(ref64)
    err = np.abs(got[m] - ref64[m])
    tol = rtol * np.abs(ref64[m]) + atol
    inf = np.isinf(ref64[m])
    bad = (err > tol) & ~inf
    assert not bad.any(), (what, "max rel err", float((err[~inf] / (np.abs(ref64[m][~inf]) + 1e-300)).max()), "rtol", rtol)
    assert np.array_equal(got[m][inf], ref64[m][inf]), (what, "infinities differ")


def bits_equal(a, b):
    a, b = np.asarray(a), np.asarray(b)
    return a.dtype == b.dtype and a.shape == b.shape and a.tobytes() == b.tobytes()


class Guarded:
    """A destination array with guard bands: the array is a view into a larger buffer whose 4 KiB
    before and after it hold a known byte pattern.  `check()` verifies that an operator wrote
    nothing outside its destination - the stand-in for a memory checker on the device."""
    BAND = 4096
    PATTERN = 0xA5

    def __init__(self, gpu, dtype, dims, misalign: int = 0):
        dtype = np.dtype(dtype)
        n = int(np.prod(dims, dtype=np.int64)) if not isinstance(dims, (int, np.integer)) else int(dims)
        self.gpu, self.nbytes = gpu, n * dtype.itemsize
        pad = misalign * dtype.itemsize                       # start the array off a 16-byte boundary
        self.raw = gpu.ROCArray(np.uint8, self.BAND + pad + self.nbytes + self.BAND).fill_(self.PATTERN)
        self.lo = self.BAND + pad
        self.array = self.raw.view(self.lo, self.lo + self.nbytes).reinterpret(dtype).reshape(dims)

    def check(self, what=""):
        h = self.raw.to_host()
        assert (h[:self.lo] == self.PATTERN).all(), (what, "wrote before its destination")
        assert (h[self.lo + self.nbytes:] == self.PATTERN).all(), (what, "wrote past its destination")
