// Consumers of the scan and their sibling: findall / logical indexing (stream compaction after a
// cumsum) and reverse.  They take the place of src/kernels/indexing.jl:8-36 and
// src/kernels/reverse.jl:59-122 of the reference.  Both are pure HBM-bound element movers.
#include "program.cuh"

namespace b200 {

// Four consecutive indices starting at element i0 (16-byte accesses when `vec`).
template <typename IT>
__device__ __forceinline__ void load_index4(const IT* p, int64_t i0, int64_t n, bool vec, int64_t out[4]) {
    if (vec && i0 + 4 <= n) {
        if constexpr (sizeof(IT) == 8) {
            const longlong2 a = *reinterpret_cast<const longlong2*>(p + i0), b = *reinterpret_cast<const longlong2*>(p + i0 + 2);
            out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
        } else {
            const int4 a = *reinterpret_cast<const int4*>(p + i0);
            out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
        }
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) out[k] = (i0 + k < n) ? (int64_t)p[i0 + k] : 0;
    }
}

// ys[indices[i] - 1] = i + 1 (linear, 1-based) for every i with bools[i]; with `values` given,
// the selected VALUES are gathered instead (xs[bools]).  Four mask bytes per thread and step in
// one load; the positions of a group are read only when one of its entries is selected.  A
// position outside 1..ny (positions that are not the cumsum of this mask, or a destination that
// is too short) latches B200_INVALID_ARG in the device's error word and skips that store, as
// the gather kernel below does.  `vec`: mask and positions are 16-byte aligned.
template <int BYTES, typename IT>
__global__ void __launch_bounds__(256)
compact_kernel(void* ys, const uint8_t* bools, const IT* indices, const void* values, int64_t n,
               int64_t ny, int32_t* err_word, int vec) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t groups = (n + 3) / 4;
    for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
        const int64_t i0 = g * 4;
        uint32_t m = 0;
        if (vec && i0 + 4 <= n) {
            m = *reinterpret_cast<const uint32_t*>(bools + i0);
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) if (i0 + k < n && bools[i0 + k]) m |= 0xffu << (8 * k);
        }
        if (m == 0) continue;
        int64_t pos[4];
        load_index4<IT>(indices, i0, n, vec != 0, pos);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (((m >> (8 * k)) & 0xffu) == 0) continue;
            const int64_t b = pos[k] - 1;
            if (b < 0 || b >= ny) { latch_error(err_word, B200_INVALID_ARG); continue; }
            if (values == nullptr) reinterpret_cast<int64_t*>(ys)[b] = i0 + k + 1;
            else store_bits(ys, BYTES, b, load_bits(values, BYTES, i0 + k));
        }
    }
}

struct FlipPlan {
    int32_t ndim;
    uint32_t flip_mask;
    int64_t shape[B200_MAX_DIMS];
};

// y[flipped index] = x[i]; element size BYTES.  Reads are linear, writes are linear runs in
// reverse wherever dimension 1 is flipped.  (Shapes and alignments the vector kernel below does
// not take.)
template <int BYTES>
__global__ void __launch_bounds__(256) reverse_kernel(void* y, const void* x, FlipPlan pl, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t rem = i, out = 0, mult = 1;
        for (int d = 0; d < pl.ndim; ++d) {
            const int64_t e = pl.shape[d];
            const int64_t q = rem / e;
            int64_t c = rem - q * e;
            if ((pl.flip_mask >> d) & 1u) c = e - 1 - c;
            out += c * mult;
            mult *= e;
            rem = q;
        }
        store_bits(y, BYTES, out, load_bits(x, BYTES, i));
    }
}

// The elements of a 16-byte vector in reverse order.
template <int BYTES>
__device__ __forceinline__ uint4 reverse_lanes(uint4 v) {
    if constexpr (BYTES == 8) return make_uint4(v.z, v.w, v.x, v.y);
    else if constexpr (BYTES == 4) return make_uint4(v.w, v.z, v.y, v.x);
    else if constexpr (BYTES == 2)
        return make_uint4(__byte_perm(v.w, 0, 0x1032), __byte_perm(v.z, 0, 0x1032), __byte_perm(v.y, 0, 0x1032), __byte_perm(v.x, 0, 0x1032));
    else
        return make_uint4(__byte_perm(v.w, 0, 0x0123), __byte_perm(v.z, 0, 0x0123), __byte_perm(v.y, 0, 0x0123), __byte_perm(v.x, 0, 0x0123));
}

// The same flip with 16-byte accesses: the first dimension holds a whole number of vectors and
// both arrays are 16-byte aligned.  A thread moves four vectors of one output tile; with the
// first dimension flipped a source vector comes from the mirrored place of its row with its
// elements reversed, other flipped dimensions only permute whole rows.
constexpr int kFlipUnroll = 4;
template <int BYTES>
__global__ void __launch_bounds__(256) reverse_vec_kernel(uint4* y, const uint4* x, FlipPlan pl, int64_t nvec, int64_t row_vecs) {
    const bool flip0 = (pl.flip_mask & 1u) != 0;
    const int64_t tile = (int64_t)blockDim.x * kFlipUnroll;
    for (int64_t base = (int64_t)blockIdx.x * tile; base < nvec; base += (int64_t)gridDim.x * tile) {
        uint4 v[kFlipUnroll];
        bool on[kFlipUnroll];
#pragma unroll
        for (int u = 0; u < kFlipUnroll; ++u) {
            const int64_t o = base + (int64_t)u * blockDim.x + threadIdx.x;      // output vector
            on[u] = o < nvec;
            if (!on[u]) continue;
            const int64_t row = o / row_vecs;
            const int64_t cv = o - row * row_vecs;
            int64_t rem = row, src_row = 0, mult = 1;
            for (int d = 1; d < pl.ndim; ++d) {
                const int64_t e = pl.shape[d];
                const int64_t q = rem / e;
                int64_t c = rem - q * e;
                if ((pl.flip_mask >> d) & 1u) c = e - 1 - c;
                src_row += c * mult;
                mult *= e;
                rem = q;
            }
            v[u] = __ldcs(x + src_row * row_vecs + (flip0 ? row_vecs - 1 - cv : cv));
        }
#pragma unroll
        for (int u = 0; u < kFlipUnroll; ++u) {
            if (!on[u]) continue;
            const int64_t o = base + (int64_t)u * blockDim.x + threadIdx.x;
            __stcs(y + o, flip0 ? reverse_lanes<BYTES>(v[u]) : v[u]);
        }
    }
}

// y[i] = x[ix[i]] with 1-based indices (Int64 or Int32).  An index outside 1..nx latches
// B200_INVALID_ARG in the device's error word (reported by the next synchronisation, like the
// reference's asynchronous BoundsError) and leaves that output element untouched.  A thread takes
// four consecutive indices in one load and has its four (random) reads out together.
template <int BYTES, typename IT>
__global__ void __launch_bounds__(256)
gather_kernel(void* y, const void* x, const IT* ix, int64_t n, int64_t nx, int32_t* err_word, int vec) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t groups = (n + 3) / 4;
    for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
        const int64_t i0 = g * 4;
        int64_t j[4];
        load_index4<IT>(ix, i0, n, vec != 0, j);
        uint64_t val[4];
        bool ok[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            ok[k] = i0 + k < n && j[k] >= 1 && j[k] <= nx;
            if (ok[k]) val[k] = load_bits(x, BYTES, j[k] - 1);
            else if (i0 + k < n) latch_error(err_word, B200_INVALID_ARG);
        }
        if (BYTES == 4 && vec && ok[0] && ok[1] && ok[2] && ok[3]) {
            *reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(y) + i0) =
                make_uint4((uint32_t)val[0], (uint32_t)val[1], (uint32_t)val[2], (uint32_t)val[3]);
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) if (ok[k]) store_bits(y, BYTES, i0 + k, val[k]);
        }
    }
}

// Grid of the index kernels: one resident wave over groups of four elements.
static unsigned index_grid(b200_stream_t st, int64_t n) {
    return balanced_grid(((n + 3) / 4 + 255) / 256, (int64_t)sm_count(st->dev) * 8);
}

static bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

template <typename IT>
static void launch_gather(b200_stream_t st, const b200_tensor* y, const b200_tensor* x, const b200_tensor* ix, int64_t n) {
    const unsigned grid = index_grid(st, n);
    const IT* idx = reinterpret_cast<const IT*>(ix->ptr);
    const int64_t nx = tensor_numel(x);
    int32_t* err = device_error_word(st->dev);
    const int vec = aligned16(ix->ptr) && aligned16(y->ptr);
    switch (dtype_size(x->dtype)) {
        case 1: gather_kernel<1, IT><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, idx, n, nx, err, vec); break;
        case 2: gather_kernel<2, IT><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, idx, n, nx, err, vec); break;
        case 4: gather_kernel<4, IT><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, idx, n, nx, err, vec); break;
        default: gather_kernel<8, IT><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, idx, n, nx, err, vec); break;
    }
}

template <typename IT>
static void launch_compact(b200_stream_t st, const b200_tensor* ys, const b200_tensor* bools, const b200_tensor* indices,
                           const void* vals, int bytes, int64_t n) {
    const unsigned grid = index_grid(st, n);
    const uint8_t* m = reinterpret_cast<const uint8_t*>(bools->ptr);
    const IT* idx = reinterpret_cast<const IT*>(indices->ptr);
    const int64_t ny = tensor_numel(ys);
    int32_t* err = device_error_word(st->dev);
    const int vec = aligned16(bools->ptr) && aligned16(indices->ptr);
    switch (bytes) {
        case 1: compact_kernel<1, IT><<<grid, 256, 0, st->s>>>(ys->ptr, m, idx, vals, n, ny, err, vec); break;
        case 2: compact_kernel<2, IT><<<grid, 256, 0, st->s>>>(ys->ptr, m, idx, vals, n, ny, err, vec); break;
        case 4: compact_kernel<4, IT><<<grid, 256, 0, st->s>>>(ys->ptr, m, idx, vals, n, ny, err, vec); break;
        default: compact_kernel<8, IT><<<grid, 256, 0, st->s>>>(ys->ptr, m, idx, vals, n, ny, err, vec); break;
    }
}

}  // namespace b200

using namespace b200;

extern "C" int32_t b200_gather(b200_stream_t st, const b200_tensor* y, const b200_tensor* x, const b200_tensor* ix) {
    B200_TRY(enter(st));
    B200_TRY(check_tensor(y, "gather destination"));
    B200_TRY(check_tensor(x, "gather source"));
    B200_TRY(check_tensor(ix, "gather indices"));
    if (x->dtype != y->dtype) return fail(B200_INVALID_ARG, "gather: source and destination differ in element type");
    if (ix->dtype != B200_I64 && ix->dtype != B200_I32) return fail(B200_UNSUPPORTED, "gather: indices must be Int64 or Int32");
    if (!tensor_is_contiguous(x) || !tensor_is_contiguous(y) || !tensor_is_contiguous(ix))
        return fail(B200_UNSUPPORTED, "gather: operands must be dense");
    const int64_t n = tensor_numel(ix);
    if (tensor_numel(y) != n) return fail(B200_INVALID_ARG, "gather: destination and indices differ in length");
    if (n == 0) return B200_OK;
    if (tensor_numel(x) == 0) return fail(B200_INVALID_ARG, "gather: indexing into an empty array");
    if (ix->dtype == B200_I64) launch_gather<int64_t>(st, y, x, ix, n);
    else launch_gather<int32_t>(st, y, x, ix, n);
    return finish(st, "b200_gather");
}

extern "C" int32_t b200_compact(b200_stream_t st, const b200_tensor* ys, const b200_tensor* bools,
                                const b200_tensor* indices, const b200_tensor* values) {
    B200_TRY(enter(st));
    B200_TRY(check_tensor(ys, "compaction destination"));
    B200_TRY(check_tensor(bools, "compaction mask"));
    B200_TRY(check_tensor(indices, "compaction positions"));
    if (bools->dtype != B200_BOOL && bools->dtype != B200_U8) return fail(B200_UNSUPPORTED, "the mask must be Bool");
    if (indices->dtype != B200_I64 && indices->dtype != B200_I32)
        return fail(B200_UNSUPPORTED, "positions must be Int64 or Int32 (cumsum of the mask)");
    const int64_t n = tensor_numel(bools);
    if (tensor_numel(indices) != n) return fail(B200_INVALID_ARG, "mask and positions differ in length");
    if (!tensor_is_contiguous(bools) || !tensor_is_contiguous(indices) || !tensor_is_contiguous(ys))
        return fail(B200_UNSUPPORTED, "compaction operands must be dense");
    int bytes = 8;
    const void* vals = nullptr;
    if (values) {
        B200_TRY(check_tensor(values, "compaction values"));
        if (tensor_numel(values) != n || !tensor_is_contiguous(values)) return fail(B200_INVALID_ARG, "values and mask differ in length");
        if (values->dtype != ys->dtype) return fail(B200_INVALID_ARG, "values and destination differ in element type");
        bytes = (int)dtype_size(values->dtype);
        vals = values->ptr;
    } else if (ys->dtype != B200_I64) {
        return fail(B200_UNSUPPORTED, "findall writes Int64 indices");
    }
    if (n == 0 || tensor_numel(ys) == 0) return B200_OK;
    if (indices->dtype == B200_I64) launch_compact<int64_t>(st, ys, bools, indices, vals, bytes, n);
    else launch_compact<int32_t>(st, ys, bools, indices, vals, bytes, n);
    return finish(st, "b200_compact");
}

extern "C" int32_t b200_reverse(b200_stream_t st, const b200_tensor* y, const b200_tensor* x, uint32_t dims_mask) {
    B200_TRY(enter(st));
    B200_TRY(check_tensor(y, "reverse destination"));
    B200_TRY(check_tensor(x, "reverse source"));
    if (x->dtype != y->dtype || x->ndim != y->ndim) return fail(B200_INVALID_ARG, "reverse: source and destination differ");
    for (int d = 0; d < x->ndim; ++d)
        if (x->shape[d] != y->shape[d]) return fail(B200_INVALID_ARG, "reverse: input and output arrays must equal in size");
    if (!tensor_is_contiguous(x) || !tensor_is_contiguous(y)) return fail(B200_UNSUPPORTED, "reverse: operands must be dense");
    if (x->ptr == y->ptr) return fail(B200_INVALID_ARG, "reverse: source and destination must not alias (reverse! goes through a copy)");
    const int64_t n = tensor_numel(x);
    if (n == 0) return B200_OK;
    FlipPlan pl{};
    pl.ndim = x->ndim;
    for (int d = 0; d < x->ndim; ++d) {
        pl.shape[d] = x->shape[d];
        if (((dims_mask >> d) & 1u) && x->shape[d] > 1) pl.flip_mask |= 1u << d;
    }
    const int bytes = (int)dtype_size(x->dtype);
    const int64_t row_bytes = (x->ndim > 0 ? x->shape[0] : 1) * bytes;
    if (row_bytes % 16 == 0 && aligned16(x->ptr) && aligned16(y->ptr)) {
        const int64_t nvec = n * bytes / 16, row_vecs = row_bytes / 16;
        const int64_t tiles = (nvec + 256 * kFlipUnroll - 1) / (256 * kFlipUnroll);
        const unsigned grid = (unsigned)(tiles > 0x7fffffff ? 0x7fffffff : tiles);      // one tile per block
        uint4* yo = reinterpret_cast<uint4*>(y->ptr);
        const uint4* xi = reinterpret_cast<const uint4*>(x->ptr);
        switch (bytes) {
            case 1: reverse_vec_kernel<1><<<grid, 256, 0, st->s>>>(yo, xi, pl, nvec, row_vecs); break;
            case 2: reverse_vec_kernel<2><<<grid, 256, 0, st->s>>>(yo, xi, pl, nvec, row_vecs); break;
            case 4: reverse_vec_kernel<4><<<grid, 256, 0, st->s>>>(yo, xi, pl, nvec, row_vecs); break;
            default: reverse_vec_kernel<8><<<grid, 256, 0, st->s>>>(yo, xi, pl, nvec, row_vecs); break;
        }
        return finish(st, "b200_reverse");
    }
    const unsigned grid = balanced_grid((n + 255) / 256, (int64_t)sm_count(st->dev) * 8);
    switch (bytes) {
        case 1: reverse_kernel<1><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, pl, n); break;
        case 2: reverse_kernel<2><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, pl, n); break;
        case 4: reverse_kernel<4><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, pl, n); break;
        default: reverse_kernel<8><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, pl, n); break;
    }
    return finish(st, "b200_reverse");
}
