/*
 * C restatement of the CPU algorithms the array hot path is compared and timed against.
 * TEST INFRASTRUCTURE ONLY (checker and CPU-baseline timing); the product never calls it.
 * PARITY UNPINNED: the reference (Julia, AMD GPUs) ships no golden vectors for this path and
 * cannot run here; these functions restate the specification its tests use - Julia Base on
 * Array - and are pinned by closed-form known answers only.
 *
 * What is restated:
 *  - fused elementwise loops of Base.Broadcast for  z .= a .* x .+ y  and
 *    r .= x .* y .+ exp.(-abs.(z))  (multiply and add rounded separately, -ffp-contract=off);
 *  - Base's pairwise reduction (base/reduce.jl, mapreduce_impl with 1024-element blocks), which
 *    is what sum / mapreduce(abs2, +, .) run on a Vector{Float32};
 *  - the inclusive scan loop of Base.accumulate! (src/kernels/accumulate.jl:1-8 of the
 *    reference forwards to an external package; Base's sequential definition is the oracle);
 *  - a stable least-significant-digit radix sort under Base.isless for sort!/sortperm
 *    (src/kernels/sorting.jl:1-3), index payload Int64 1-based.
 * Threaded variants split the index range over OpenMP threads (Base's own multi-threading
 * for these calls would be a user-written @threads loop over chunks).
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

API int ora_max_threads(void) { return omp_get_max_threads(); }

API void ora_axpy_f32(float a, const float* x, const float* y, float* z, int64_t n, int threads) {
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float p = a * x[i];
        z[i] = p + y[i];
    }
}

API void ora_muladd_exp_f32(const float* x, const float* y, const float* z, float* r, int64_t n, int threads) {
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float p = x[i] * y[i];
        r[i] = p + expf(-fabsf(z[i]));
    }
}

/* Base.mapreduce_impl: sequential below the block size, otherwise split in the middle. */
static float pairwise_f32(const float* a, int64_t lo, int64_t hi, int sq) {
    if (hi - lo < 1024) {
        float v = sq ? a[lo] * a[lo] : a[lo];
        for (int64_t i = lo + 1; i <= hi; ++i) v += sq ? a[i] * a[i] : a[i];
        return v;
    }
    int64_t mid = lo + ((hi - lo) >> 1);
    return pairwise_f32(a, lo, mid, sq) + pairwise_f32(a, mid + 1, hi, sq);
}

/* sum(x) (sq = 0) or mapreduce(abs2, +, x) (sq = 1); threads > 1 reduces chunks in parallel and
 * adds the chunk results in order. */
API float ora_sum_f32(const float* x, int64_t n, int sq, int threads) {
    if (n == 0) return 0.0f;
    if (threads <= 1) return pairwise_f32(x, 0, n - 1, sq);
    float* part = (float*)calloc((size_t)threads, sizeof(float));
    int used = 0;
#pragma omp parallel num_threads(threads)
    {
        int t = omp_get_thread_num(), nt = omp_get_num_threads();
        int64_t per = (n + nt - 1) / nt, lo = t * per, hi = lo + per;
        if (hi > n) hi = n;
        if (lo < hi) part[t] = pairwise_f32(x, lo, hi - 1, sq);
#pragma omp single
        used = nt;
    }
    float s = 0.0f;
    for (int t = 0; t < used; ++t) s += part[t];
    free(part);
    return s;
}

API double ora_sum_f64acc(const float* x, int64_t n, int sq, int threads) {
    double s = 0.0;
#pragma omp parallel for num_threads(threads) reduction(+ : s) schedule(static)
    for (int64_t i = 0; i < n; ++i) s += sq ? (double)x[i] * (double)x[i] : (double)x[i];
    return s;
}

API void ora_cumsum_f32(const float* x, float* out, int64_t n) {
    float acc = 0.0f;
    for (int64_t i = 0; i < n; ++i) { acc = acc + x[i]; out[i] = acc; }
}

API void ora_cumsum_i32(const int32_t* x, int32_t* out, int64_t n) {
    uint32_t acc = 0;
    for (int64_t i = 0; i < n; ++i) { acc += (uint32_t)x[i]; out[i] = (int32_t)acc; }
}

/* two-pass threaded scan: per-thread block totals, then offsets */
API void ora_cumsum_i32_mt(const int32_t* x, int32_t* out, int64_t n, int threads) {
    uint32_t* tot = (uint32_t*)calloc((size_t)threads + 1, sizeof(uint32_t));
#pragma omp parallel num_threads(threads)
    {
        int t = omp_get_thread_num(), nt = omp_get_num_threads();
        int64_t per = (n + nt - 1) / nt, lo = t * per, hi = lo + per;
        if (hi > n) hi = n;
        uint32_t acc = 0;
        for (int64_t i = lo; i < hi; ++i) { acc += (uint32_t)x[i]; out[i] = (int32_t)acc; }
        tot[t + 1] = acc;
#pragma omp barrier
#pragma omp single
        for (int k = 1; k <= nt; ++k) tot[k] += tot[k - 1];
        uint32_t off = tot[t];
        if (off) for (int64_t i = lo; i < hi; ++i) out[i] = (int32_t)((uint32_t)out[i] + off);
    }
    free(tot);
}

static inline uint32_t f32_key(uint32_t b) {
    int nan = (b & 0x7fffffffu) > 0x7f800000u;
    return ((b & 0x80000000u) && !nan) ? ~b : (b | 0x80000000u);
}

/* stable LSD radix sort of u32 keys, 8-bit digits */
API void ora_sort_u32(uint32_t* keys, int64_t n) {
    uint32_t* tmp = (uint32_t*)malloc((size_t)n * 4);
    uint32_t *src = keys, *dst = tmp;
    for (int p = 0; p < 4; ++p) {
        int64_t cnt[257] = {0};
        for (int64_t i = 0; i < n; ++i) cnt[((src[i] >> (8 * p)) & 255) + 1]++;
        for (int d = 0; d < 256; ++d) cnt[d + 1] += cnt[d];
        for (int64_t i = 0; i < n; ++i) dst[cnt[(src[i] >> (8 * p)) & 255]++] = src[i];
        uint32_t* t = src; src = dst; dst = t;
    }
    free(tmp);
}

/* sortperm of Float32 keys under isless: stable, 1-based Int64 result */
API void ora_sortperm_f32(const float* x, int64_t* perm, int64_t n) {
    uint32_t* k0 = (uint32_t*)malloc((size_t)n * 4);
    uint32_t* k1 = (uint32_t*)malloc((size_t)n * 4);
    int64_t* p1 = (int64_t*)malloc((size_t)n * 8);
    for (int64_t i = 0; i < n; ++i) { uint32_t b; memcpy(&b, &x[i], 4); k0[i] = f32_key(b); perm[i] = i + 1; }
    uint32_t *ks = k0, *kd = k1;
    int64_t *ps = perm, *pd = p1;
    for (int p = 0; p < 4; ++p) {
        int64_t cnt[257] = {0};
        for (int64_t i = 0; i < n; ++i) cnt[((ks[i] >> (8 * p)) & 255) + 1]++;
        for (int d = 0; d < 256; ++d) cnt[d + 1] += cnt[d];
        for (int64_t i = 0; i < n; ++i) { int64_t o = cnt[(ks[i] >> (8 * p)) & 255]++; kd[o] = ks[i]; pd[o] = ps[i]; }
        uint32_t* t = ks; ks = kd; kd = t;
        int64_t* q = ps; ps = pd; pd = q;
    }
    free(k0); free(k1); free(p1);
}
