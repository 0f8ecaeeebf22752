// Counter-based synthetic data: element i of an array is a pure function of (seed, stream_id, i),
// so shards can be generated in place on any device and any slice can be regenerated for a
// check.  Stands in for AMDGPU.rand!/randn! (src/random.jl:30-70 of the reference) for the
// synthetic workloads; the integer, raw and uniform distributions are bit-identical to the
// NumPy restatement used by the tests, the normal ones only statistically (device libm).
#include "program.cuh"

namespace b200 {

__host__ __device__ inline uint64_t mix64(uint64_t z) {
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}
__host__ __device__ inline uint64_t counter_key(uint64_t seed, uint64_t stream_id) {
    return mix64(seed + 0x9E3779B97F4A7C15ull * (stream_id + 1));
}
__host__ __device__ inline uint64_t counter_draw(uint64_t key, uint64_t index) {
    return mix64(key + (index + 1) * 0x9E3779B97F4A7C15ull);
}

__device__ __forceinline__ double normal_from(uint64_t r) {
    const float u1 = (float)((r >> 40) + 1) * 5.9604644775390625e-8f;          // (0,1]
    const float u2 = (float)((r >> 8) & 0xffffffull) * 5.9604644775390625e-8f; // [0,1)
    return (double)(sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2));
}

struct GenArgs {
    void*    out;
    int32_t  dtype, dist;
    uint64_t key, first, n;
    int64_t  lo, hi;
};

__global__ void __launch_bounds__(256) fill_random_kernel(GenArgs a) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const int bytes = dtype_bytes(a.dtype);
    const int cls = dtype_class(a.dtype);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
        uint64_t idx = a.first + i;
        uint64_t r = counter_draw(a.key, idx);
        if (a.dist == 5) {
            // about 1 % of the positions repeat the value of another position
            if (mix64(r ^ 0xA5A5A5A5A5A5A5A5ull) % 100 == 0) {
                idx = mix64(r ^ 0x5A5A5A5A5A5A5A5Aull) % (uint64_t)a.hi;
                r = counter_draw(a.key, idx);
            }
        }
        double f = 0.0;
        uint64_t raw = 0;
        bool is_float_value = true;
        switch (a.dist) {
            case 0: f = (cls == CF64) ? (double)(r >> 11) * 1.1102230246251565e-16 : (double)((float)(r >> 40) * 5.9604644775390625e-8f); break;
            case 1: f = (cls == CF64) ? 2.0 * ((double)(r >> 11) * 1.1102230246251565e-16) - 1.0
                                      : (double)(2.0f * ((float)(r >> 40) * 5.9604644775390625e-8f) - 1.0f); break;
            case 2: case 5: f = normal_from(r); break;
            case 3: raw = (uint64_t)(a.lo + (int64_t)(r % (uint64_t)(a.hi - a.lo + 1))); is_float_value = false; break;
            default: raw = r; is_float_value = false; break;
        }
        uint64_t bits;
        if (cls == CF32 || cls == CF64) {
            const double v = is_float_value ? f : (double)(int64_t)raw;
            if (cls == CF64) bits = (uint64_t)__double_as_longlong(v);
            else bits = encode<uint64_t>(a.dtype, (uint64_t)__float_as_uint((float)v));
        } else {
            bits = is_float_value ? (uint64_t)(int64_t)f : raw;
        }
        store_bits(a.out, bytes, (int64_t)i, bits);
    }
}

}  // namespace b200

using namespace b200;

extern "C" int32_t b200_fill_random(b200_stream_t st, const b200_tensor* out, int32_t dist, uint64_t seed,
                                    uint64_t stream_id, uint64_t first_index, int64_t lo, int64_t hi) {
    B200_TRY(enter(st));
    B200_TRY(check_tensor(out, "fill_random destination"));
    if (!tensor_is_contiguous(out)) return fail(B200_UNSUPPORTED, "fill_random: destination must be dense");
    if (dist < 0 || dist > 5) return fail(B200_INVALID_ARG, "fill_random: unknown distribution %d", dist);
    if (dist == 3 && hi < lo) return fail(B200_INVALID_ARG, "fill_random: empty integer range");
    if (dist == 5 && hi <= 0) return fail(B200_INVALID_ARG, "fill_random: distribution 5 needs the array length in `hi`");
    const int64_t n = tensor_numel(out);
    if (n == 0) return B200_OK;
    GenArgs a{out->ptr, out->dtype, dist, counter_key(seed, stream_id), first_index, (uint64_t)n, lo, hi};
    int64_t blocks = (n + 256 * 8 - 1) / (256 * 8);
    const int64_t cap = (int64_t)sm_count(st->dev) * 16;
    if (blocks > cap) blocks = cap;
    fill_random_kernel<<<(unsigned)blocks, 256, 0, st->s>>>(a);
    return finish(st, "b200_fill_random");
}
