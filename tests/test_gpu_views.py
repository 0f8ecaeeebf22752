"""Wrapped operands (views, permuted dimensions, transposes), the sort keywords and integer-vector
indexing, against NumPy on the same data.  These are the shapes the reference's own unit tests
use: test/core/rocarray_base.jl:55-62 (offset views), :263-267 (reduction into a transpose),
test/core/rocarray_broadcast.jl:19-20 (broadcast over views), test/hip_rocarray/sorting.jl:12-26
(``xd[sortperm(xd)]``, ``lt=!isless``, ``by=k -> 2k``)."""
import numpy as np
import pytest

from helpers import assert_close, bits_equal

pytestmark = pytest.mark.gpu


def fa(rng, shape, dt=np.float32):
    return np.asfortranarray(rng.standard_normal(shape).astype(dt))


def test_strided_views_round_trip(gpu):
    rng = np.random.default_rng(11)
    H = fa(rng, (37, 29, 5))
    A = gpu.ROCArray.from_host(H)
    cases = [
        (A.subview(slice(3, 30), slice(None), slice(None)), H[3:30]),
        (A.subview(slice(0, 37, 3), 4, slice(1, 5)), H[0:37:3, 4, 1:5]),
        (A.subview(5, slice(None), 2), H[5, :, 2]),
        (A.permuteddims((3, 1, 2)), H.transpose(2, 0, 1)),
        (A.subview(slice(None), slice(None), 1).transpose(), H[:, :, 1].T),
    ]
    for view, ref in cases:
        assert bits_equal(view.to_host(), np.asfortranarray(ref))
        assert bits_equal(view.copy().to_host(), np.asfortranarray(ref))
    assert bits_equal(A.permutedims((2, 3, 1)).to_host(), np.asfortranarray(H.transpose(1, 2, 0)))
    # writes through a view land in the parent
    B = gpu.ROCArray.from_host(H)
    B.subview(slice(0, 37, 2), slice(None), 3).fill_(7.0)
    ref = H.copy()
    ref[0:37:2, :, 3] = 7.0
    assert bits_equal(B.to_host(), ref)
    patch = fa(rng, (10, 29))
    B.subview(slice(20, 30), slice(None), 0).copy_from_host(patch)
    ref[20:30, :, 0] = patch
    assert bits_equal(B.to_host(), ref)


def test_broadcast_and_reduce_over_views(gpu, orc):
    rng = np.random.default_rng(12)
    H, K = fa(rng, (64, 48)), fa(rng, (48, 64))
    A, B = gpu.ROCArray.from_host(H), gpu.ROCArray.from_host(K)
    out = (A.dot * B.transpose().dot + np.float32(1.5)).materialize().to_host()
    assert bits_equal(out, (H * K.T + np.float32(1.5)).astype(np.float32))
    # destination is a view: dest .= expr
    D = gpu.zeros(np.float32, (64, 48))
    gpu.materialize_(D.subview(slice(8, 24), slice(None)), A.subview(slice(0, 16), slice(None)).dot * np.float32(2))
    ref = np.zeros((64, 48), np.float32)
    ref[8:24] = H[0:16] * np.float32(2)
    assert bits_equal(D.to_host(), ref)
    # reductions with a strided source, and into a transposed destination (rocarray_base.jl:263-267)
    v = A.subview(slice(1, 64, 2), slice(None))
    assert_close(gpu.sum(v, dims=1).to_host(), H[1:64:2].astype(np.float64).sum(axis=0, keepdims=True), 1e-5)
    assert bits_equal(gpu.maximum(B.transpose(), dims=2).to_host(), K.T.max(axis=1, keepdims=True))
    assert_close(gpu.sum(v), H[1:64:2].astype(np.float64).sum(), 1e-5)
    T3 = fa(rng, (3, 2, 10))
    R = gpu.zeros(np.float32, (2, 3)).transpose()
    assert gpu.mapreducedim_("identity", "+", R, gpu.ROCArray.from_host(T3), init=np.float32(0)) is R
    assert_close(R.to_host(), T3.astype(np.float64).sum(axis=2), 1e-5)


def test_accumulate_and_sort_on_views(gpu):
    rng = np.random.default_rng(13)
    H = np.asfortranarray(rng.integers(-50, 50, (40, 33)).astype(np.int64))
    A = gpu.ROCArray.from_host(H)
    row = A.subview(7, slice(None))                         # stride 40
    assert np.array_equal(gpu.cumsum(row).to_host(), np.cumsum(H[7]))
    assert np.array_equal(gpu.cumsum(A.transpose(), dims=1).to_host(), np.cumsum(H.T, axis=0))
    out = gpu.zeros(np.int64, (40, 33))
    gpu.accumulate_("+", out.subview(slice(None), 2), A.subview(slice(None), 5))
    assert np.array_equal(out.to_host()[:, 2], np.cumsum(H[:, 5])) and not out.to_host()[:, 3].any()
    # sort! of a strided row sorts the parent's elements in place and touches nothing else
    S = gpu.ROCArray.from_host(H)
    gpu.sort_(S.subview(3, slice(None)))
    ref = H.copy()
    ref[3] = np.sort(H[3], kind="stable")
    assert np.array_equal(S.to_host(), ref)
    assert np.array_equal(gpu.sortperm(A.subview(9, slice(None))).to_host(), np.argsort(H[9], kind="stable") + 1)


@pytest.mark.parametrize("dt", [np.float16, np.float32, np.float64, np.int16, np.int32, np.int64])
def test_sort_keywords_like_the_reference_tests(gpu, dt):
    rng = np.random.default_rng(14)
    dt = np.dtype(dt)
    for n in (1, 2, 3, 4, 33, 333, 3333, 4096):
        if dt.kind == "f":
            x = rng.random(n).astype(dt)
        else:   # rand(Int) spans the whole range; halve it so that 2k does not wrap differently on the host
            x = rng.integers(np.iinfo(dt).min // 2, np.iinfo(dt).max // 2, n, dtype=dt)
        xd = gpu.ROCArray.from_host(x)
        y = np.sort(x, kind="stable")
        assert bits_equal(gpu.sort(xd).to_host(), y)
        assert bits_equal(gpu.getindex(xd, gpu.sortperm(xd)).to_host(), y)
        assert bits_equal(gpu.sort(xd, rev=True).to_host(), y[::-1])
        assert bits_equal(gpu.getindex(xd, gpu.sortperm(xd, rev=True)).to_host(), y[::-1])
        assert bits_equal(gpu.sort(xd, lt="!isless").to_host(), y[::-1])
        assert bits_equal(gpu.getindex(xd, gpu.sortperm(xd, lt="!isless")).to_host(), y[::-1])
        assert bits_equal(gpu.sort(xd, by=lambda k: 2 * k).to_host(), y)
        assert bits_equal(gpu.getindex(xd, gpu.sortperm(xd, by=lambda k: 2 * k)).to_host(), y)
    # `by` that changes the order: |k| ascending, stable among equal magnitudes
    v = np.array([3, -1, 2, -3, 1, -2, 0, 3], dtype=dt)
    vd = gpu.ROCArray.from_host(v)
    perm = np.argsort(np.abs(v), kind="stable")
    assert np.array_equal(gpu.sortperm(vd, by=abs).to_host(), perm + 1)
    assert bits_equal(gpu.sort(vd, by=abs).to_host(), v[perm])
    assert bits_equal(gpu.sort(vd, by=lambda k: -k).to_host(), v[np.argsort(-v, kind="stable")])
    with pytest.raises(ValueError):
        gpu.sort(vd, lt=lambda a, b: a > b)


def test_integer_vector_indexing(gpu):
    rng = np.random.default_rng(15)
    for dt in (np.int8, np.float16, np.float32, np.float64):
        x = (rng.standard_normal(10_007) * 50).astype(dt)
        for it in (np.int64, np.int32):
            ix = rng.integers(1, x.size, 33_333, endpoint=True).astype(it)
            got = gpu.getindex(gpu.ROCArray.from_host(x), gpu.ROCArray.from_host(ix)).to_host()
            assert bits_equal(got, x[ix.astype(np.int64) - 1])
    M = np.asfortranarray(rng.standard_normal((17, 9)).astype(np.float32))
    ix = np.array([1, 17, 18, 153], dtype=np.int64)                     # linear, column-major
    assert bits_equal(gpu.getindex(gpu.ROCArray.from_host(M), gpu.ROCArray.from_host(ix)).to_host(),
                      M.reshape(-1, order="F")[ix - 1])
    assert gpu.getindex(gpu.ROCArray.from_host(x), gpu.ROCArray(np.int64, 0)).dims == (0,)
    # an index outside 1:length(x) is reported at the next synchronisation; the context stays usable
    bad = gpu.ROCArray.from_host(np.array([1, 0, 5], dtype=np.int64))
    small = gpu.ROCArray.from_host(np.arange(5, dtype=np.float32))
    out = gpu.getindex(small, bad)
    with pytest.raises(gpu.B200Error):
        gpu.synchronize()
    gpu.synchronize()
    assert gpu.sum(small) == 10.0
    del out


def test_large_transposed_operands_go_through_tiles(gpu):
    """Transposed matrices above 2^14 elements are copied into dense form through shared-memory
    tiles before the expression runs (or straight into a dense destination for a plain copy):
    every element size, extents that are not multiples of the tile, the transpose of a view with
    a leading dimension, several transposed operands at once, a destination that aliases the
    source, and a dimension of extent one between the two."""
    rng = np.random.default_rng(13)
    for dt in (np.uint8, np.float16, np.float32, np.int64):
        for shape in ((200, 300), (129, 257), (1024, 64), (64, 1024), (131, 128)):
            K = np.asfortranarray((rng.random(shape[::-1]) * 100).astype(dt))        # K.T has `shape`
            Kd = gpu.ROCArray.from_host(K)
            assert bits_equal(Kd.transpose().copy().to_host(), np.asfortranarray(K.T)), (dt, shape)
            assert bits_equal(Kd.permutedims((2, 1)).to_host(), np.asfortranarray(K.T)), (dt, shape)
    H, K, L = fa(rng, (300, 200)), fa(rng, (200, 300)), fa(rng, (200, 300))
    A, B, Cc = gpu.ROCArray.from_host(H), gpu.ROCArray.from_host(K), gpu.ROCArray.from_host(L)
    out = (A.dot + B.transpose().dot).materialize().to_host()
    assert bits_equal(out, H + K.T)
    out = (B.transpose().dot * Cc.transpose().dot + np.float32(0.5)).materialize().to_host()
    assert bits_equal(out, (K.T * L.T + np.float32(0.5)).astype(np.float32))
    # the transpose of a window of a larger matrix
    Big = fa(rng, (400, 500))
    Bd = gpu.ROCArray.from_host(Big)
    win = Bd.subview(slice(10, 210), slice(5, 305))                               # 200 x 300, leading dimension 400
    assert bits_equal(win.transpose().copy().to_host(), np.asfortranarray(Big[10:210, 5:305].T))
    assert bits_equal((A.dot - win.transpose().dot).materialize().to_host(), H - Big[10:210, 5:305].T)
    # A .= A' on a square matrix: the source is copied before the destination is written
    S = fa(rng, (256, 256))
    Sd = gpu.ROCArray.from_host(S)
    gpu.materialize_(Sd, Sd.transpose().dot)
    assert bits_equal(Sd.to_host(), np.asfortranarray(S.T))
    # 3-d operand whose middle dimension has extent one
    T = fa(rng, (150, 1, 180))
    Td = gpu.ROCArray.from_host(T)
    assert bits_equal(Td.permuteddims((3, 2, 1)).copy().to_host(), np.asfortranarray(T.transpose(2, 1, 0)))
    # mixed element types still take the evaluator after the copy
    I = np.asfortranarray(rng.integers(-50, 50, (200, 300)).astype(np.int32))
    out = (gpu.ROCArray.from_host(I).transpose().dot * A.dot).materialize().to_host()
    assert bits_equal(out, (I.T.astype(np.float32) * H).astype(np.float32))


def test_permuted_operands_of_higher_rank(gpu):
    """PermutedDimsArray operands whose unit-stride dimension is not the first one take the tiled
    copy with the remaining dimensions as batch: every permutation of a 3-d array, a 4-d case,
    extents that are not multiples of the tile, 2- and 8-byte elements, and use inside a fused
    expression next to a dense operand."""
    import itertools
    rng = np.random.default_rng(14)
    H = fa(rng, (40, 50, 60))
    A = gpu.ROCArray.from_host(H)
    for perm in itertools.permutations((1, 2, 3)):
        ref = np.asfortranarray(H.transpose(tuple(p - 1 for p in perm)))
        assert bits_equal(A.permuteddims(perm).copy().to_host(), ref), perm
        D = gpu.ROCArray.from_host(np.asfortranarray(ref * np.float32(0.5)))
        out = (A.permuteddims(perm).dot + D.dot).materialize().to_host()
        assert bits_equal(out, ref + ref * np.float32(0.5)), perm
    for dt in (np.float16, np.int64):
        K = np.asfortranarray((rng.random((33, 70, 9, 21)) * 100).astype(dt))
        Kd = gpu.ROCArray.from_host(K)
        for perm in ((2, 1, 3, 4), (4, 3, 2, 1), (3, 4, 1, 2), (2, 4, 1, 3)):
            ref = np.asfortranarray(K.transpose(tuple(p - 1 for p in perm)))
            assert bits_equal(Kd.permutedims(perm).to_host(), ref), (dt, perm)
    # short first dimension: stays on the strided path and must still be right
    S = fa(rng, (3000, 5))
    assert bits_equal(gpu.ROCArray.from_host(S).transpose().copy().to_host(), np.asfortranarray(S.T))


def test_reductions_over_permuted_operands(gpu, orc):
    """mapreduce whose operand is a large transposed / permuted view: the view is copied into dense
    form first (a pool temporary that is freed on the stream), then the ordinary kernels run."""
    rng = np.random.default_rng(15)

    def fp(shape):                                   # positive data: the sums are well conditioned
        return np.asfortranarray(rng.random(shape).astype(np.float32))
    K = fp((300, 200))
    Kd = gpu.ROCArray.from_host(K)
    gpu.synchronize()
    live = gpu.pool_stats()["live_bytes"]
    T = Kd.transpose()                                            # 200 x 300
    assert_close(gpu.sum(T, dims=1).to_host(), K.T.astype(np.float64).sum(axis=0, keepdims=True), 1e-5)
    assert_close(gpu.sum(T, dims=2).to_host(), K.T.astype(np.float64).sum(axis=1, keepdims=True), 1e-5)
    assert bits_equal(gpu.maximum(T, dims=2).to_host(), K.T.max(axis=1, keepdims=True))
    assert_close(gpu.sum(T), K.astype(np.float64).sum(), 1e-5)
    H = fp((200, 300))
    Hd = gpu.ROCArray.from_host(H)
    got = gpu.mapreduce(None, "+", Hd.dot * T.dot)
    assert_close(got, (H.astype(np.float64) * K.T).sum(), 1e-5)
    got = gpu.mapreduce(None, "max", gpu.broadcast.abs_(Hd.dot - T.dot), dims=1).to_host()
    assert bits_equal(got, np.abs(H - K.T).max(axis=0, keepdims=True))
    P3 = fp((30, 40, 50))
    Pd = gpu.ROCArray.from_host(P3).permuteddims((3, 1, 2))      # 50 x 30 x 40
    ref = P3.transpose(2, 0, 1).astype(np.float64)
    assert_close(gpu.sum(Pd, dims=(1, 3)).to_host(), ref.sum(axis=(0, 2), keepdims=True), 1e-5)
    gpu.synchronize()
    assert gpu.pool_stats()["live_bytes"] == live + Hd.nbytes + P3.nbytes      # the temporaries are gone
