"""The oracle against closed-form known answers and against its own C restatement (CPU only)."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

G = np.load(Path(__file__).parent / "golden" / "known_answers.npz")


def test_closed_form_reductions(orc):
    n = int(G["iota_n"])
    x = np.arange(1, n + 1, dtype=np.int32)
    assert orc.mapreduce("identity", "+", x) == G["iota_sum"]
    assert orc.mapreduce("identity", "+", G["pow2_in"]) == np.float64(G["pow2_sum"])
    assert np.array_equal(orc.mapreducedim("identity", "+", (1, 4), G["mat"]), G["mat_sum_dims1"].astype(np.float64))
    assert np.array_equal(orc.mapreducedim("identity", "max", (3, 1), G["mat"]), G["mat_max_dims2"].astype(np.float64))
    assert orc.mapreduce("abs2", "+", G["mat"]) == np.float64(G["mat_sumsq"])


def test_closed_form_scans(orc):
    n = 1000
    assert np.array_equal(orc.accumulate("+", np.ones(n, dtype=np.int64)), np.arange(1, n + 1))
    alt = np.where(np.arange(8) % 2 == 0, 1, -1).astype(np.int32)
    assert np.array_equal(orc.accumulate("+", alt), G["alt_scan_first8"])
    assert np.array_equal(orc.accumulate("+", G["wrap_in"]), G["wrap_scan"])
    assert np.array_equal(orc.accumulate("+", G["pow2_in"]), G["pow2_scan"].astype(np.float64))
    assert np.array_equal(orc.accumulate("+", np.ones(4, np.int32), init=np.int32(5)), np.array([6, 7, 8, 9], np.int32))


def test_isless_ordering(orc):
    x = G["order_in"]
    s = orc.sort(x)
    assert np.array_equal(s.view(np.uint32)[:-1], G["order_sorted"].view(np.uint32)[:-1]) and np.isnan(s[-1])
    assert np.array_equal(orc.sortperm(x), G["order_perm"])
    assert np.array_equal(orc.sortperm(x, rev=True), G["order_perm_rev"])
    assert np.array_equal(orc.sort(np.arange(100, 0, -1, dtype=np.int32)), np.arange(1, 101, dtype=np.int32))
    assert np.array_equal(orc.sortperm(np.full(17, 4.0, np.float32)), np.arange(1, 18))
    assert np.array_equal(orc.sortperm(np.full(17, 4.0, np.float32), rev=True), np.arange(1, 18))


def test_broadcast_semantics(orc):
    mx = orc.broadcast(("max", G["mm_a"], G["mm_b"]))
    mn = orc.broadcast(("min", G["mm_a"], G["mm_b"]))
    ok = ~np.isnan(G["mm_max"])
    assert np.array_equal(np.isnan(mx), ~ok) and np.array_equal(mx[ok].view(np.uint32), G["mm_max"][ok].view(np.uint32))
    assert np.array_equal(np.isnan(mn), ~ok) and np.array_equal(mn[ok].view(np.uint32), G["mm_min"][ok].view(np.uint32))
    z = orc.broadcast(("add", ("mul", G["axpy_a"][()], G["axpy_x"]), G["axpy_y"]))
    assert z.dtype == np.float32 and np.array_equal(z, G["axpy_unfused"])
    # promotion: Int64 literal * Float32 array stays Float32; Float64 literal widens
    assert orc.broadcast(("mul", 2, np.ones(3, np.float32))).dtype == np.float32
    assert orc.broadcast(("mul", 2.0, np.ones(3, np.float32))).dtype == np.float64
    assert orc.broadcast(("div", np.ones(3, np.int32), np.full(3, 2, np.int32))).dtype == np.float64
    assert orc.broadcast(("add", np.array([1, 2, 3]), np.array([1.0, 2.0, 3.0]))).tolist() == [2.0, 4.0, 6.0]
    # Float16 arithmetic rounds after every operation
    h = np.array([2049.0], dtype=np.float16)   # rounds to 2048
    assert orc.broadcast(("add", h, np.float16(1.0)))[0] == np.float16(2048.0)


def test_c_restatement_matches_numpy(orc):
    import b200_oracle.c_oracle as co
    lib = co.load()
    rng = np.random.default_rng(1)
    n = 200_003
    x, y, z = (rng.random(n, dtype=np.float32) * 2 - 1 for _ in range(3))
    out = np.empty_like(x)
    lib.ora_axpy_f32(2.5, co.ptr(x, C.c_float), co.ptr(y, C.c_float), co.ptr(out, C.c_float), n, 4)
    assert np.array_equal(out, orc.broadcast(("add", ("mul", np.float32(2.5), x), y)))
    lib.ora_muladd_exp_f32(co.ptr(x, C.c_float), co.ptr(y, C.c_float), co.ptr(z, C.c_float), co.ptr(out, C.c_float), n, 4)
    ref = orc.broadcast(("add", ("mul", x, y), ("exp", ("neg", ("abs", z)))))
    assert np.allclose(out, ref, rtol=1e-6, atol=2e-7)   # expf of libm vs NumPy: last-bit differences
    for sq in (0, 1):
        want = orc.mapreduce("abs2" if sq else "identity", "+", x)
        for th in (1, 4):
            got = lib.ora_sum_f32(co.ptr(x, C.c_float), n, sq, th)
            assert abs(got - want) <= 1e-5 * max(1.0, abs(want))
    iv = rng.integers(-100, 101, n, dtype=np.int32)
    o1, o2 = np.empty_like(iv), np.empty_like(iv)
    lib.ora_cumsum_i32(co.ptr(iv, C.c_int32), co.ptr(o1, C.c_int32), n)
    lib.ora_cumsum_i32_mt(co.ptr(iv, C.c_int32), co.ptr(o2, C.c_int32), n, 4)
    assert np.array_equal(o1, orc.accumulate("+", iv)) and np.array_equal(o2, o1)
    k = rng.integers(0, 2**32, n, dtype=np.uint32)
    ks = k.copy()
    lib.ora_sort_u32(co.ptr(ks, C.c_uint32), n)
    assert np.array_equal(ks, orc.sort(k))
    f = rng.standard_normal(n).astype(np.float32)
    f[::50] = f[7]
    f[3], f[4], f[5] = np.nan, -0.0, 0.0
    p = np.empty(n, dtype=np.int64)
    lib.ora_sortperm_f32(co.ptr(f, C.c_float), co.ptr(p, C.c_int64), n)
    assert np.array_equal(p, orc.sortperm(f))


def test_generator_pin(pkg):
    assert np.array_equal(pkg.random.host_draw(0, 0, 0, 8), G["draws_seed0_stream0"])
    assert np.array_equal(pkg.random.host_draw(3, 1, 1000, 4), G["draws_seed3_stream1_at1000"])
    # slices of one stream agree with the whole
    a = pkg.random.host_uniform01(5, 2, 0, 100)
    b = pkg.random.host_uniform01(5, 2, 40, 10)
    assert np.array_equal(a[40:50], b) and a.min() >= 0 and a.max() < 1
    i = pkg.random.host_integers(2, 0, 0, 10_000, -100, 100)
    assert i.min() >= -100 and i.max() <= 100 and i.dtype == np.int32


def test_signed_zero_in_max_min_reductions(orc):
    """Base.max/min order -0.0 below +0.0; the oracle's reductions must say which zero comes out."""
    pz, nz = np.float32(0.0), np.float32(-0.0)
    sign = lambda v: bool(np.signbit(np.asarray(v).reshape(-1)[0]))
    assert not sign(orc.mapreduce("identity", "max", np.array([nz, pz, nz], np.float32)))
    assert sign(orc.mapreduce("identity", "max", np.array([nz, nz], np.float32)))
    assert sign(orc.mapreduce("identity", "min", np.array([pz, nz, pz], np.float32)))
    assert not sign(orc.mapreduce("identity", "min", np.array([pz, pz], np.float32)))
    m = np.array([[nz, pz], [nz, nz]], np.float32)
    assert [bool(s) for s in np.signbit(orc.mapreducedim("identity", "max", (2, 1), m)).reshape(-1)] == [False, True]
    assert np.isnan(orc.mapreduce("identity", "max", np.array([1.0, np.nan, 0.0], np.float32)))


def test_torch_cpu_is_a_third_opinion(orc):
    """torch's CPU kernels (Float64 sum and cumsum, stable sort) as an implementation that shares no
    code with the oracle or with NumPy's reductions."""
    import torch
    rng = np.random.default_rng(3)
    x = (rng.random(300_007) * 2 - 1).astype(np.float32)
    tx = torch.from_numpy(x).double()
    assert abs(orc.mapreduce("identity", "+", x) - float(tx.sum())) <= 1e-9 * float(tx.abs().sum())
    assert abs(orc.mapreduce("abs2", "+", x) - float((tx * tx).sum())) <= 1e-9 * float((tx * tx).sum())
    assert np.allclose(orc.accumulate("+", x), torch.cumsum(tx, 0).numpy(), rtol=1e-12, atol=1e-9)
    iv = rng.integers(-100, 101, 100_003).astype(np.int32)
    assert np.array_equal(orc.accumulate("+", iv), torch.cumsum(torch.from_numpy(iv), 0, dtype=torch.int32).numpy())
    k = rng.integers(0, 1000, 50_001).astype(np.int64)             # many ties: stability matters
    vals, idx = torch.sort(torch.from_numpy(k), stable=True)
    assert np.array_equal(orc.sort(k), vals.numpy()) and np.array_equal(orc.sortperm(k), idx.numpy() + 1)
    f = rng.standard_normal(20_001).astype(np.float32)
    f[::40] = f[3]
    vals, idx = torch.sort(torch.from_numpy(f), stable=True)
    assert np.array_equal(orc.sort(f), vals.numpy()) and np.array_equal(orc.sortperm(f), idx.numpy() + 1)
    vals, idx = torch.sort(torch.from_numpy(f), stable=True, descending=True)
    assert np.array_equal(orc.sort(f, rev=True), vals.numpy()) and np.array_equal(orc.sortperm(f, rev=True), idx.numpy() + 1)
