"""Graph capture and replay, following test/core/graph_tests.jl of the reference (+1, malloc/free
inside the capture, allocation cache, update), plus the library-specific rule about scratch."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_plus_one(gpu):
    z = gpu.zeros(np.int64, (4, 4))
    graph = gpu.captured(lambda: gpu.materialize_(z, z.dot + 1))
    assert gpu.sum(z) == 16
    gpu.launch(graph)
    assert gpu.sum(z) == 32
    gpu.launch(graph)
    assert gpu.sum(z) == 48
    assert not gpu.is_capturing()


def test_malloc_and_free_inside_capture(gpu):
    z = gpu.zeros(np.int64, (4, 4))

    def f():
        x = gpu.ones(np.int64, (4, 4))
        gpu.materialize_(z, z.dot + (x.dot + 1))
        x.unsafe_free_()

    graph = gpu.captured(f)
    assert gpu.sum(z) == 32
    gpu.launch(graph)
    assert gpu.sum(z) == 64
    gpu.launch(graph)
    assert gpu.sum(z) == 96


def test_alloc_cache_inside_capture(gpu):
    z = gpu.zeros(np.int64, (4, 4))

    def f():
        x = gpu.ones(np.int64, (4, 4))
        y = gpu.ones(np.int64, (4, 4))
        gpu.materialize_(z, z.dot + (x.dot * y.dot + 1))

    cache = gpu.AllocCache()
    with gpu.cached(cache):          # pre-populate: no allocator call during the capture
        f()
    before = gpu.pool_stats()["alloc_count"]
    with gpu.cached(cache):
        graph = gpu.captured(f)
    assert gpu.pool_stats()["alloc_count"] == before
    assert gpu.sum(z) == 16 * 2 * 2
    gpu.launch(graph)
    assert gpu.sum(z) == 16 * 2 * 3
    gpu.launch(graph)
    assert gpu.sum(z) == 16 * 2 * 4
    gpu.synchronize()
    cache.unsafe_free_()


def test_update(gpu):
    z = gpu.zeros(np.int64, (4, 4))
    graph = gpu.captured(lambda: gpu.materialize_(z, z.dot + 1))
    assert gpu.sum(z) == 16
    g_new = gpu.capture(lambda: gpu.materialize_(z, z.dot + 2))
    assert gpu.update(graph, g_new)
    gpu.launch(graph)
    assert gpu.sum(z) == 48
    two_nodes = gpu.capture(lambda: (gpu.materialize_(z, z.dot + 2), gpu.materialize_(z, z.dot + 2)))
    assert gpu.update(graph, two_nodes, throw_error=False) is False      # different topology
    with pytest.raises(RuntimeError):
        gpu.update(graph, two_nodes)
    gpu.launch(graph)                                                    # still the old executable
    assert gpu.sum(z) == 80


def test_operators_replay_and_scratch_rule(gpu):
    """A scan, a dims reduction and a sort replayed from one graph on a fresh stream: the first
    capture is refused (the stream has no scratch yet), `captured` runs the function once and
    captures again; replays give the same results on new input."""
    st = gpu.Stream()
    with gpu.using_stream(st):
        n = 50_000
        x = gpu.ROCArray.from_host(np.arange(n, dtype=np.int32))
        c = gpu.ROCArray(np.int32, n)
        keys = gpu.ROCArray(np.uint32, n)
        A = gpu.ROCArray.from_host(np.ones((256, 64), np.float32))
        R = gpu.ROCArray(np.float32, (1, 64))

        def f():
            gpu.accumulate_("+", c, x)
            gpu.mapreducedim_("identity", "+", R, A, init=np.float32(0))
            gpu.materialize_(keys, c.dot * np.uint32(2654435761))     # scrambles the order (wraps in UInt32)
            gpu.sort_(keys)

        assert gpu.capture(f, throw_error=False) is None               # scratch would have to grow
        assert not gpu.is_capturing()
        graph = gpu.captured(f)

        def check():
            h = x.to_host()
            cs = np.cumsum(h, dtype=np.int32)
            assert np.array_equal(c.to_host(), cs)
            assert np.array_equal(R.to_host(), A.to_host().sum(axis=0, keepdims=True))
            k = cs.astype(np.uint32) * np.uint32(2654435761)
            assert np.array_equal(keys.to_host(), np.sort(k))

        check()
        x.copy_from_host(np.arange(n, dtype=np.int32)[::-1].copy())
        A.copy_from_host(np.full((256, 64), 2.0, np.float32))
        gpu.launch(graph)
        check()
        gpu.launch(graph)
        check()
        st.synchronize()
