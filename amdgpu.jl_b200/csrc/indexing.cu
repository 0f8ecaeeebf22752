// Consumers of the scan and their sibling: findall / logical indexing (stream compaction after a
// cumsum) and reverse.  They take the place of src/kernels/indexing.jl:8-36 and
// src/kernels/reverse.jl:59-122 of the reference.  Both are pure HBM-bound element movers.
#include "program.cuh"

namespace b200 {

// ys[indices[i] - 1] = i + 1 (linear, 1-based) for every i with bools[i]; with `values` given,
// the selected VALUES are gathered instead (xs[bools]).  A position outside 1..ny (positions that
// are not the cumsum of this mask, or a destination that is too short) latches B200_INVALID_ARG
// in the device's error word and skips that store, as the gather kernel below does.
template <int BYTES>
__global__ void __launch_bounds__(256)
compact_kernel(void* ys, const uint8_t* bools, const int64_t* indices, const void* values, int64_t n,
               int64_t ny, int32_t* err_word) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        if (bools[i]) {
            const int64_t b = indices[i] - 1;
            if (b < 0 || b >= ny) { latch_error(err_word, B200_INVALID_ARG); continue; }
            if (values == nullptr) reinterpret_cast<int64_t*>(ys)[b] = i + 1;
            else store_bits(ys, BYTES, b, load_bits(values, BYTES, i));
        }
    }
}

struct FlipPlan {
    int32_t ndim;
    uint32_t flip_mask;
    int64_t shape[B200_MAX_DIMS];
};

// y[flipped index] = x[i]; element size BYTES.  Reads are linear, writes are linear runs in
// reverse wherever dimension 1 is flipped.
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

// y[i] = x[ix[i]] with 1-based indices (Int64 or Int32).  An index outside 1..nx latches
// B200_INVALID_ARG in the device's error word (reported by the next synchronisation, like the
// reference's asynchronous BoundsError) and leaves that output element untouched.
template <int BYTES, typename IT>
__global__ void __launch_bounds__(256)
gather_kernel(void* y, const void* x, const IT* ix, int64_t n, int64_t nx, int32_t* err_word) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t j = (int64_t)ix[i] - 1;
        if (j < 0 || j >= nx) { latch_error(err_word, B200_INVALID_ARG); continue; }
        store_bits(y, BYTES, i, load_bits(x, BYTES, j));
    }
}

template <typename IT>
static void launch_gather(b200_stream_t st, const b200_tensor* y, const b200_tensor* x, const b200_tensor* ix, int64_t n) {
    const unsigned grid = balanced_grid((n + 255) / 256, (int64_t)sm_count(st->dev) * 8);
    const IT* idx = reinterpret_cast<const IT*>(ix->ptr);
    const int64_t nx = tensor_numel(x);
    int32_t* err = device_error_word(st->dev);
    switch (dtype_size(x->dtype)) {
        case 1: gather_kernel<1, IT><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, idx, n, nx, err); break;
        case 2: gather_kernel<2, IT><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, idx, n, nx, err); break;
        case 4: gather_kernel<4, IT><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, idx, n, nx, err); break;
        default: gather_kernel<8, IT><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, idx, n, nx, err); break;
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
    if (indices->dtype != B200_I64) return fail(B200_UNSUPPORTED, "positions must be Int64 (cumsum of the mask)");
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
    const unsigned grid = balanced_grid((n + 255) / 256, (int64_t)sm_count(st->dev) * 8);
    const uint8_t* m = reinterpret_cast<const uint8_t*>(bools->ptr);
    const int64_t* idx = reinterpret_cast<const int64_t*>(indices->ptr);
    const int64_t ny = tensor_numel(ys);
    int32_t* err = device_error_word(st->dev);
    switch (bytes) {
        case 1: compact_kernel<1><<<grid, 256, 0, st->s>>>(ys->ptr, m, idx, vals, n, ny, err); break;
        case 2: compact_kernel<2><<<grid, 256, 0, st->s>>>(ys->ptr, m, idx, vals, n, ny, err); break;
        case 4: compact_kernel<4><<<grid, 256, 0, st->s>>>(ys->ptr, m, idx, vals, n, ny, err); break;
        default: compact_kernel<8><<<grid, 256, 0, st->s>>>(ys->ptr, m, idx, vals, n, ny, err); break;
    }
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
    const unsigned grid = balanced_grid((n + 255) / 256, (int64_t)sm_count(st->dev) * 8);
    switch (dtype_size(x->dtype)) {
        case 1: reverse_kernel<1><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, pl, n); break;
        case 2: reverse_kernel<2><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, pl, n); break;
        case 4: reverse_kernel<4><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, pl, n); break;
        default: reverse_kernel<8><<<grid, 256, 0, st->s>>>(y->ptr, x->ptr, pl, n); break;
    }
    return finish(st, "b200_reverse");
}
