"""Run-time specialised broadcast kernels against the interpreter: the two run the same evaluator
source, so their results must agree bit for bit, whatever the element types, layout or tail."""
import numpy as np
import pytest

from helpers import bits_equal

pytestmark = pytest.mark.gpu


def _both(gpu, build, dest_dtype, shape):
    """Evaluates the expression with the specialised kernel and with the interpreter."""
    B = gpu.broadcast
    outs = []
    for jit in (True, False):
        B.jit_configure(jit)
        try:
            d = gpu.ROCArray(dest_dtype, shape).fill_(0)
            gpu.materialize_(d, build())
            outs.append(d.to_host())
        finally:
            B.jit_configure(True)
    return outs


def test_specialised_kernels_match_the_interpreter(gpu):
    B = gpu.broadcast
    rng = np.random.default_rng(21)
    before = B.jit_stats()
    assert before["enabled"]
    for n in (1, 3, 4, 1023, 100_003, 1 << 20):
        xs = [rng.standard_normal(n).astype(np.float32) for _ in range(3)]
        xi = rng.integers(-100, 100, n).astype(np.int32)
        xh = rng.standard_normal(n).astype(np.float16)
        d = [gpu.ROCArray.from_host(a) for a in xs]
        di, dh = gpu.ROCArray.from_host(xi), gpu.ROCArray.from_host(xh)
        cases = [
            (lambda: d[0].dot * d[1].dot + B.exp(-B.abs_(d[2].dot)) + np.float32(0.25), np.float32),
            (lambda: B.maximum(d[0].dot - d[1].dot, d[2].dot * np.float32(2)), np.float32),
            (lambda: di.dot * d[0].dot * 1.5, np.float64),                    # Int32 * Float32 * Float64
            (lambda: B.muladd(dh.dot, dh.dot, d[0].dot) / np.float32(3), np.float32),
            (lambda: B.abs2(dh.dot) + dh.dot, np.float16),                    # narrow type re-rounded per operator
            (lambda: B.minimum(di.dot, 7) - di.dot * di.dot, np.int64),
        ]
        for build, dt in cases:
            a, b = _both(gpu, build, dt, n)
            assert bits_equal(a, b), (n, dt)
    after = B.jit_stats()
    if after["failures"] > before["failures"] and after["compiled"] == before["compiled"]:
        pytest.skip("no run-time compiler on this machine: the interpreter ran both times")
    # 36 evaluations went through the specialised path: each either compiled a kernel or found one
    # (other tests of the same process may have compiled some of these structures already)
    assert after["compiled"] + after["hits"] >= before["compiled"] + before["hits"] + 36
    assert after["hits"] > before["hits"]


def test_specialised_kernels_on_strided_and_broadcast_operands(gpu):
    B = gpu.broadcast
    rng = np.random.default_rng(22)
    H = np.asfortranarray(rng.standard_normal((96, 40)).astype(np.float32))
    col = rng.standard_normal((96, 1)).astype(np.float32)
    A, c = gpu.ROCArray.from_host(H), gpu.ROCArray.from_host(col)
    At = gpu.ROCArray.from_host(np.asfortranarray(H.T))
    a, b = _both(gpu, lambda: A.dot * c.dot + B.exp(At.transpose().dot) - np.float32(1), np.float32, (96, 40))
    assert bits_equal(a, b)
    ref = H.astype(np.float64) * col + np.exp(H.astype(np.float64)) - 1.0
    assert np.allclose(a, ref, rtol=1e-5, atol=1e-5)     # expf differs from libm by an ulp or two
    # the same structure with other sizes and scalar values reuses the compiled kernel
    s0 = B.jit_stats()
    x = gpu.ROCArray.from_host(rng.standard_normal(777).astype(np.float32))
    for k in (2.0, 3.0, 4.0):
        out = (x.dot * np.float32(k) + B.abs_(x.dot) * B.abs_(x.dot)).materialize().to_host()
        ref = x.to_host() * np.float32(k) + np.abs(x.to_host()) * np.abs(x.to_host())
        assert bits_equal(out, ref.astype(np.float32))
    s1 = B.jit_stats()
    if s1["compiled"] > s0["compiled"]:
        assert s1["compiled"] == s0["compiled"] + 1 and s1["hits"] >= s0["hits"] + 2
    assert B.precompile(gpu.ROCArray(np.float32, 10), x.dot * np.float32(5) + B.abs_(x.dot) * B.abs_(x.dot)) in (True, False)


def test_specialised_reductions_match_the_interpreter(gpu):
    """mapreduce over a map expression with several operands (dot products, distances ...)."""
    B = gpu.broadcast
    rng = np.random.default_rng(23)
    H, K = rng.standard_normal((300, 41, 7)).astype(np.float32), rng.standard_normal((300, 41, 7)).astype(np.float32)
    Hd, Kd = gpu.ROCArray.from_host(np.asfortranarray(H)), gpu.ROCArray.from_host(np.asfortranarray(K))
    ints = gpu.ROCArray.from_host(rng.integers(-9, 9, 100_003).astype(np.int32))
    half = gpu.ROCArray.from_host(rng.standard_normal(100_003).astype(np.float16))
    cases = [
        (lambda: gpu.mapreduce(None, "+", Hd.dot * Kd.dot), None),                         # dot product
        (lambda: gpu.mapreduce(None, "+", B.abs2(Hd.dot - Kd.dot), dims=1), None),
        (lambda: gpu.mapreduce(None, "max", B.abs_(Hd.dot - Kd.dot), dims=(1, 3)), None),
        (lambda: gpu.mapreduce(None, "min", Hd.dot * np.float32(2) + Kd.dot, dims=2), None),
        (lambda: gpu.mapreduce(None, "+", ints.dot * ints.dot - 3), None),
        (lambda: gpu.mapreduce(None, "+", half.dot * half.dot + ints.dot), None),
    ]
    before = B.jit_stats()
    for build, _ in cases:
        outs = []
        for jit in (True, False):
            B.jit_configure(jit)
            try:
                r = build()
                outs.append(r.to_host() if hasattr(r, "to_host") else np.asarray(r))
            finally:
                B.jit_configure(True)
        assert bits_equal(outs[0], outs[1])
    ref = (H.astype(np.float64) * K).sum()
    assert abs(float(gpu.mapreduce(None, "+", Hd.dot * Kd.dot)) - ref) <= 1e-5 * abs(ref) + 1e-3
    after = B.jit_stats()
    if after["compiled"] == before["compiled"] and after["failures"] > before["failures"]:
        pytest.skip("no run-time compiler on this machine")
    assert after["compiled"] + after["hits"] >= before["compiled"] + before["hits"] + 6
