"""Runtime layer on a real device: streams, events, pool accounting, limits, copies, fills."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_device_and_versions(gpu):
    p = gpu.device_properties()
    assert p["cc"][0] == 10 and p["sm_count"] >= 100, p
    v = gpu.versioninfo()
    assert v["cuda_runtime"] >= 12000
    assert gpu.ndevices() >= 1 and gpu.current_device() == 0


def test_streams_events_priorities(gpu):
    for prio in (-1, 0, 1):
        st = gpu.Stream(0, prio)
        with gpu.using_stream(st):
            x = gpu.ROCArray(np.float32, 1 << 20).fill_(1.5)
            a, b = gpu.Event(timing=True).record(), None
            y = (x.dot * 2).materialize()
            b = gpu.Event(timing=True).record()
            b.synchronize()
            assert gpu.elapsed_ms(a, b) >= 0.0
            assert y.to_host()[123] == 3.0
        st.synchronize()
        assert st.isdone()
    with pytest.raises(gpu.B200Error):
        gpu.Stream(0, 5)
    with gpu.elapsed() as t:
        gpu.ROCArray(np.float32, 1 << 22).fill_(0)
    assert t() > 0


def test_copy_fill_views(gpu):
    rng = np.random.default_rng(0)
    for dt in (np.uint8, np.int16, np.float16, np.int32, np.float32, np.float64, np.int64):
        a = (rng.random(1001) * 100).astype(dt)
        d = gpu.ROCArray.from_host(a)
        assert np.array_equal(d.to_host(), a)
        assert np.array_equal(d.copy().to_host(), a)
        v = d.view(3, 500)                      # pointer not 16-byte aligned
        assert np.array_equal(v.to_host(), a[3:500])
        v.fill_(dt(7))
        a[3:500] = 7
        assert np.array_equal(d.to_host(), a)
    m = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    d = gpu.ROCArray.from_host(m)
    assert np.array_equal(d.to_host(), m)
    assert np.array_equal(d.reshape(6, 4).to_host(), m.reshape(6, 4, order="F"))
    assert gpu.zeros(np.int32, (3, 3)).to_host().sum() == 0 and gpu.ones(np.float64, 5).to_host().sum() == 5
    assert gpu.ROCArray(np.float32, 0).to_host().shape == (0,)


def test_pool_accounting_and_limits(gpu):
    gpu.synchronize()
    s0 = gpu.pool_stats()
    x = gpu.ROCArray(np.uint8, 10 << 20)
    s1 = gpu.pool_stats()
    assert s1["alloc_count"] == s0["alloc_count"] + 1 and s1["live_bytes"] == s0["live_bytes"] + (10 << 20)
    x.unsafe_free_()
    s2 = gpu.pool_stats()
    assert s2["free_count"] == s0["free_count"] + 1 and s2["live_bytes"] == s0["live_bytes"]
    with pytest.raises(RuntimeError):
        x.ptr
    # out-of-memory injected through the host-side budget: nothing on the GPU faults.  (The retry
    # ladder ends with reclaim, which also hands back operator scratch: do that first, so that the
    # limit is set against what the arrays themselves hold.)
    gpu.reclaim()
    live = gpu.pool_stats()["live_bytes"]
    gpu.configure(hard=f"{(live >> 20) + 64} MiB")
    try:
        with pytest.raises(gpu.OutOfMemoryError):
            gpu.ROCArray(np.uint8, 256 << 20)
        small = gpu.ROCArray(np.uint8, 1 << 20)      # still fine below the limit
        small.unsafe_free_()
    finally:
        gpu.configure(hard="none")
    big = gpu.ROCArray(np.uint8, 256 << 20)
    big.unsafe_free_()
    gpu.synchronize()
    gpu.reclaim()
    free, total = gpu.mem_info()
    assert 0 < free <= total


def test_errors_are_reported_not_fatal(gpu):
    x = gpu.ROCArray.from_host(np.ones(8, np.float32))
    with pytest.raises(ValueError):
        gpu.broadcast.Broadcasted.call("sin", x)
    with pytest.raises(ValueError):
        gpu.materialize_(gpu.ROCArray(np.float32, 7), x.dot + 1)
    with pytest.raises(ValueError):
        gpu.sort_(x, lt=lambda a, b: a > b)
    bad = gpu._lib.Tensor()
    bad.dtype, bad.ndim = 99, 1
    bad.shape[0] = 4
    import ctypes as C
    st = gpu._lib.lib.b200_sort(gpu.current_stream().handle, C.byref(bad), 0)
    assert st == gpu._lib.UNSUPPORTED
    # the context is still usable afterwards
    assert float(gpu.sum(x)) == 8.0


def test_bounded_wait_reports_timeout_and_context_survives(gpu):
    """A device-side wait that can never be satisfied (its flag is never set) runs out of its
    small poll budget, the kernel returns, and the error surfaces from the next synchronisation
    as a status - the way the reference surfaces device exceptions at synchronize
    (src/highlevel.jl:40).  Nothing traps or hangs; later work on the same context is fine."""
    L = gpu._lib
    st = gpu.current_stream()
    assert L.lib.b200_selftest_wait_timeout(st.handle, 2000) == L.OK
    with pytest.raises(gpu.B200Error) as ei:
        st.synchronize()
    assert ei.value.code == L.LOOKBACK_TIMEOUT
    st.synchronize()                                    # the latched word was cleared by the report
    x = gpu.ROCArray.from_host(np.arange(100_000, dtype=np.int32))
    assert np.array_equal(gpu.cumsum(x).to_host(), np.cumsum(np.arange(100_000, dtype=np.int32), dtype=np.int32))
    assert gpu.sum(x) == 100_000 * 99_999 // 2


def test_buffer_moves_between_streams_in_order(gpu, orc):
    """An array written on one stream and read on another needs no explicit synchronisation: the
    operator hands the buffer over (event on the old stream, wait on the new one), which is what
    take_ownership! does in the reference (src/memory.jl:431-446) with a host-side sync."""
    a, b = gpu.Stream(0), gpu.Stream(0)
    n = 1 << 24
    ref = None
    for it in range(100):
        x = gpu.ROCArray(np.float32, n, stream=a)
        x.fill_(np.float32(1.0 + it), a)                         # long fill on stream a
        gpu.materialize_(x, x.dot * np.float32(0.5), a)          # and a dependent kernel behind it
        r = gpu.ROCArray(np.float32, 1, stream=b)
        gpu.mapreducedim_("identity", "+", r, x, init=np.float32(0), stream=b)     # read on stream b, no sync
        assert x.buf.stream is b
        got = float(r.to_host(b)[0])
        ref = n * (1.0 + it) * 0.5
        assert got == ref, (it, got, ref)
    # free follows the last user: drop on b while b still reads, reallocate on a, contents intact
    y = gpu.ROCArray(np.float32, n, stream=a).fill_(np.float32(3), a)
    total = gpu.ROCArray(np.float32, 1, stream=b)
    gpu.mapreducedim_("identity", "+", total, y, init=np.float32(0), stream=b)
    del y                                                        # stream-ordered free on b, behind the reduction
    z = gpu.ROCArray(np.float32, n, stream=a).fill_(np.float32(-1), a)
    assert float(total.to_host(b)[0]) == 3.0 * n
    assert float(gpu.sum(z)) == -1.0 * n
    a.synchronize(); b.synchronize()


def test_reclaim_returns_operator_scratch(gpu):
    """Operator scratch (radix double buffers, scan descriptors) belongs to the stream; reclaim
    hands it back, and live bytes return to what the arrays themselves hold."""
    gpu.synchronize()
    gpu.reclaim()
    base = gpu.pool_stats()["live_bytes"]
    n = 1 << 26
    keys = gpu.random.fill_random_(gpu.ROCArray(np.uint32, n), gpu.random.RAWBITS, seed=3)
    gpu.sort_(keys)
    gpu.cumsum(gpu.ROCArray(np.int32, 1 << 22).fill_(1)).unsafe_free_()
    gpu.synchronize()
    assert gpu.pool_stats()["live_bytes"] >= base + 4 * n + 4 * n      # the keys and the sort's second buffer
    keys.unsafe_free_()
    gpu.reclaim()
    assert gpu.pool_stats()["live_bytes"] == base
    # scratch comes back on demand
    x = gpu.ROCArray.from_host(np.arange(1 << 21, dtype=np.int32))
    assert int(gpu.cumsum(x).to_host()[-1]) == int(np.int64((1 << 21) * ((1 << 21) - 1) // 2).astype(np.int32))   # Int32 wraps


def test_dependent_small_kernels_back_to_back(gpu):
    """Kernels that may overlap the tail of their predecessor on the stream still see everything
    it wrote: a long chain of small dependent operators (in-place update, scan of the result,
    reduction of the scan) with no host synchronisation in between, checked exactly in Int32."""
    rng = np.random.default_rng(5)
    n = 1 << 19                                    # 2 MiB: the streaming, segment-scan and block-reduction kernels
    x = rng.integers(-3, 4, n).astype(np.int32)
    y = rng.integers(-3, 4, n).astype(np.int32)
    xd, yd = gpu.ROCArray.from_host(x), gpu.ROCArray.from_host(y)
    scan = gpu.ROCArray(np.int32, n)
    tot = gpu.ROCArray(np.int32, 1)
    totals = []
    for k in range(60):
        gpu.broadcast.materialize_(xd, xd.dot + yd.dot)            # x .+= y
        gpu.accumulate_("+", scan, xd, init=None)
        gpu.mapreducedim_("identity", "+", tot, scan, init=np.int32(0))
        gpu.broadcast.materialize_(yd, yd.dot * np.int32(-1))      # y .= -y, read by the next round
        totals.append(tot.copy())
    ref_x, ref_y = x.copy(), y.copy()
    for k in range(60):
        ref_x = ref_x + ref_y
        want = np.cumsum(ref_x, dtype=np.int32).sum(dtype=np.int32)
        ref_y = -ref_y
        assert int(totals[k].to_host()[0]) == int(want), k
    assert np.array_equal(xd.to_host(), ref_x)
