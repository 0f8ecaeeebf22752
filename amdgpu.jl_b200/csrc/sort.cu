// sort! and sortperm: onesweep least-significant-digit radix sort, 8-bit digits.
//
// Takes the place of AK.sort! / AK.sortperm! as called from src/kernels/sorting.jl:1-3 of the
// reference (a comparison merge sort there).  Keys are mapped to unsigned integers whose
// natural order is Base.isless (sign flip for signed integers; for floats negative values
// are complemented and positive ones get the top bit, so -0.0 < +0.0 and NaNs come last;
// `rev` complements the mapped key, which keeps equal keys in input order as a stable sort
// under the reversed ordering does).  One upfront kernel builds the histograms of all digits;
// then each digit takes ONE pass over the data: a tile ranks its keys with warp-wide matching,
// publishes its 256 digit counts, resolves the counts of all earlier tiles by decoupled
// look-back (bounded waits, as in the scan) and scatters through shared memory so that global
// writes go out in runs per digit.  Traffic for 4-byte keys: 4 B (histogram) + 4 x 8 B.
#include "common.cuh"

#include <cstring>

namespace b200 {

constexpr int kSortThreads = 512;
constexpr int kSortWarps = kSortThreads / 32;
constexpr uint32_t kFlagShift = 30;
constexpr uint32_t kValueMask = (1u << kFlagShift) - 1;
constexpr uint32_t kFlagAggregate = 1u << kFlagShift;
constexpr uint32_t kFlagPrefix = 2u << kFlagShift;

enum { KIND_UNSIGNED = 0, KIND_SIGNED = 1, KIND_FLOAT = 2 };

template <typename UK>
__device__ __forceinline__ UK to_radix(UK bits, int kind, int rev, UK expmask) {
    constexpr UK TOP = UK(UK(1) << (8 * sizeof(UK) - 1));
    UK r;
    if (kind == KIND_UNSIGNED) r = bits;
    else if (kind == KIND_SIGNED) r = bits ^ TOP;
    else {
        const bool nan = UK(bits & UK(~TOP)) > expmask;
        r = ((bits & TOP) && !nan) ? UK(~bits) : UK(bits | TOP);
    }
    return rev ? UK(~r) : r;
}
template <typename UK>
__device__ __forceinline__ UK from_radix(UK r, int kind, int rev) {
    constexpr UK TOP = UK(UK(1) << (8 * sizeof(UK) - 1));
    if (rev) r = UK(~r);
    if (kind == KIND_UNSIGNED) return r;
    if (kind == KIND_SIGNED) return r ^ TOP;
    return (r & TOP) ? UK(r ^ TOP) : UK(~r);
}

// ---- all digit histograms in one pass over the keys ---------------------------------------------------
template <typename UK>
__global__ void __launch_bounds__(kSortThreads)
sort_histogram_kernel(const UK* keys, uint32_t n, int kind, int rev, UK expmask, uint32_t* ghist) {
    constexpr int P = sizeof(UK);
    constexpr int V = 16 / sizeof(UK);
    __shared__ uint32_t h[P * 256];
    for (int i = threadIdx.x; i < P * 256; i += blockDim.x) h[i] = 0;
    __syncthreads();
    const bool aligned = reinterpret_cast<uintptr_t>(keys) % 16 == 0;
    const uint32_t nvec = aligned ? n / V : 0;
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        Vec<UK, V> v = __builtin_bit_cast(Vec<UK, V>, __ldcs(reinterpret_cast<const uint4*>(keys) + i));
#pragma unroll
        for (int q = 0; q < V; ++q) {
            const UK r = to_radix<UK>(v.v[q], kind, rev, expmask);
#pragma unroll
            for (int p = 0; p < P; ++p) atomicAdd(&h[p * 256 + (int)((r >> (8 * p)) & 0xff)], 1u);
        }
    }
    for (uint32_t i = nvec * V + blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const UK r = to_radix<UK>(keys[i], kind, rev, expmask);
#pragma unroll
        for (int p = 0; p < P; ++p) atomicAdd(&h[p * 256 + (int)((r >> (8 * p)) & 0xff)], 1u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < P * 256; i += blockDim.x)
        if (h[i]) atomicAdd(&ghist[i], h[i]);
}

// exclusive scan of each digit histogram: block p handles pass p (256 threads)
__global__ void __launch_bounds__(256) sort_scan_histogram_kernel(const uint32_t* ghist, uint32_t* bin_base) {
    __shared__ uint32_t s[8];
    const int d = threadIdx.x, lane = d & 31, warp = d >> 5;
    const uint32_t c = ghist[blockIdx.x * 256 + d];
    uint32_t inc = c;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        uint32_t o = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += o;
    }
    if (lane == 31) s[warp] = inc;
    __syncthreads();
    uint32_t wp = 0;
    for (int w = 0; w < warp; ++w) wp += s[w];
    bin_base[blockIdx.x * 256 + d] = wp + inc - c;
}

struct SweepArgs {
    const void* keys_in;
    void*       keys_out;
    const uint32_t* vals_in;
    uint32_t*   vals_out;
    int64_t*    perm_out;      // last pass of sortperm: 1-based Int64 permutation, no key output
    uint32_t    n, ntiles;
    int32_t     shift;
    int32_t     first;         // keys_in holds raw keys: map them
    int32_t     last;          // keys_out receives raw keys: map back
    int32_t     gen_index;     // values are the global positions (first pass of sortperm)
    int32_t     kind, rev;
    uint64_t    expmask;
    const uint32_t* bin_base;  // [256] exclusive digit offsets of this pass
    uint32_t*   state;         // [ntiles][256] look-back words of this pass
    unsigned int* ticket;
    int32_t*    err_word;
    uint32_t    max_polls;
};

template <typename UK, int KPT, bool PAIRS>
__global__ void __launch_bounds__(kSortThreads)
onesweep_kernel(const __grid_constant__ SweepArgs a) {
    constexpr int TILE = kSortThreads * KPT;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint32_t* whist = reinterpret_cast<uint32_t*>(smem_raw);            // [warps][256]
    uint32_t* s_binstart = whist + kSortWarps * 256;                     // [256]
    uint32_t* s_goff = s_binstart + 256;                                 // [256]
    UK* exch = reinterpret_cast<UK*>(s_goff + 256);                      // [TILE]
    uint32_t* vexch = reinterpret_cast<uint32_t*>(exch + TILE);          // [TILE] when PAIRS
    __shared__ uint32_t s_tile;
    __shared__ uint32_t s_wsum[8];
    __shared__ int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        const unsigned int t = atomicAdd(a.ticket, 1u);
        if (t == a.ntiles - 1) *a.ticket = 0;
        s_tile = t;
        s_abort = 0;
    }
    for (int i = tid; i < kSortWarps * 256; i += kSortThreads) whist[i] = 0;
    __syncthreads();
    const uint32_t tile = s_tile;
    const uint32_t tile_base = tile * (uint32_t)TILE;
    const uint32_t left = a.n - tile_base;
    const uint32_t count = left < (uint32_t)TILE ? left : (uint32_t)TILE;
    const UK expmask = (UK)a.expmask;

    // ---- load, warp-striped: item i of lane l is element warp_base + i*32 + l
    UK key[KPT];
    uint32_t val[KPT];
    const uint32_t warp_off = (uint32_t)warp * 32u * KPT;
    const UK* kin = reinterpret_cast<const UK*>(a.keys_in);
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const uint32_t local = warp_off + (uint32_t)i * 32u + lane;
        if (local < count) {
            const UK raw = kin[tile_base + local];
            key[i] = a.first ? to_radix<UK>(raw, a.kind, a.rev, expmask) : raw;
            if (PAIRS) val[i] = a.gen_index ? tile_base + local : a.vals_in[tile_base + local];
        } else {
            key[i] = UK(~UK(0));
            if (PAIRS) val[i] = 0;
        }
    }

    // ---- rank inside the warp: keys with equal digits get consecutive ranks in element order
    uint32_t rank[KPT];
    uint32_t* myhist = whist + warp * 256;
    const uint32_t lt_mask = (1u << lane) - 1u;
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const uint32_t d = (uint32_t)((key[i] >> a.shift) & 0xff);
        // lanes holding the same digit: eight ballots, one per digit bit (measured far cheaper
        // on this part than one match.any per key)
        uint32_t peers = 0xffffffffu;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const bool bit = (d >> b) & 1u;
            const uint32_t m = __ballot_sync(0xffffffffu, bit);
            peers &= bit ? m : ~m;
        }
        const int leader = __ffs(peers) - 1;
        uint32_t base = 0;
        if (lane == leader) {
            base = myhist[d];
            myhist[d] = base + __popc(peers);
        }
        __syncwarp();
        base = __shfl_sync(0xffffffffu, base, leader);
        rank[i] = base + __popc(peers & lt_mask);
    }
    __syncthreads();

    // ---- per digit: offsets of each warp inside the digit, tile count, publish
    uint32_t c = 0;
    if (tid < 256) {
        uint32_t run = 0;
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w) {
            const uint32_t t = whist[w * 256 + tid];
            whist[w * 256 + tid] = run;
            run += t;
        }
        c = run;
        if (tid == 255) c -= (uint32_t)TILE - count;    // padding keys carry digit 255 and come last
        *reinterpret_cast<volatile uint32_t*>(a.state + (size_t)tile * 256 + tid) =
            (tile == 0 ? kFlagPrefix : kFlagAggregate) | c;
        // tile-local exclusive scan over the 256 digits
        uint32_t inc = c;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            uint32_t o = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= off) inc += o;
        }
        if (lane == 31) s_wsum[warp] = inc;
        c = c;   // keep
        s_binstart[tid] = inc;   // inclusive inside the warp for now
    }
    __syncthreads();
    if (tid < 256) {
        uint32_t wp = 0;
        for (int w = 0; w < warp; ++w) wp += s_wsum[w];
        s_binstart[tid] = wp + s_binstart[tid] - c;
    }
    __syncthreads();

    // ---- keys (and values) to their tile-local sorted position
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const uint32_t d = (uint32_t)((key[i] >> a.shift) & 0xff);
        const uint32_t pos = s_binstart[d] + whist[warp * 256 + d] + rank[i];
        exch[pos] = key[i];
        if (PAIRS) vexch[pos] = val[i];
    }

    // ---- decoupled look-back: thread d sums digit d over all earlier tiles
    if (tid < 256) {
        uint32_t excl = 0;
        bool abort = false;
        if (tile > 0) {
            // kLook predecessors per round: the loads are independent, so one L2 round trip
            // resolves up to kLook tiles instead of one
            constexpr int kLook = 8;
            int64_t t = (int64_t)tile - 1;
            bool done = false;
            while (!done && !abort) {
                uint32_t w[kLook];
#pragma unroll
                for (int q = 0; q < kLook; ++q)
                    w[q] = (t - q >= 0) ? *reinterpret_cast<const volatile uint32_t*>(a.state + (size_t)(t - q) * 256 + tid) : kFlagPrefix;
#pragma unroll
                for (int q = 0; q < kLook; ++q) {
                    if (done || abort) break;
                    uint32_t v = w[q];
                    if ((v >> kFlagShift) == 0) {
                        const volatile uint32_t* wp = a.state + (size_t)(t - q) * 256 + tid;
                        uint32_t polls = 0;
                        v = *wp;
                        while ((v >> kFlagShift) == 0) {
                            ++polls;
                            if (polls > a.max_polls) { abort = true; break; }
                            if ((polls & 1023u) == 0 && error_latched(a.err_word)) { abort = true; break; }
                            if (polls > 32) __nanosleep(polls > 4096 ? 256 : 32);
                            v = *wp;
                        }
                        if (abort) break;
                    }
                    excl += v & kValueMask;
                    if ((v >> kFlagShift) == 2u) done = true;
                }
                t -= kLook;
            }
            if (!abort)
                *reinterpret_cast<volatile uint32_t*>(a.state + (size_t)tile * 256 + tid) = kFlagPrefix | (excl + c);
        }
        if (abort) {
            latch_error(a.err_word, B200_LOOKBACK_TIMEOUT);
            s_abort = 1;
        }
        s_goff[tid] = a.bin_base[tid] + excl - s_binstart[tid];
    }
    __syncthreads();
    if (s_abort) return;

    // ---- global scatter, in runs per digit
    UK* kout = reinterpret_cast<UK*>(a.keys_out);
#pragma unroll
    for (int j = 0; j < KPT; ++j) {
        const uint32_t pos = (uint32_t)j * kSortThreads + tid;
        if (pos < count) {
            const UK k = exch[pos];
            const uint32_t d = (uint32_t)((k >> a.shift) & 0xff);
            const uint32_t g = s_goff[d] + pos;
            if (a.perm_out == nullptr) kout[g] = a.last ? from_radix<UK>(k, a.kind, a.rev) : k;
            if (PAIRS) {
                if (a.perm_out) a.perm_out[g] = (int64_t)vexch[pos] + 1;
                else a.vals_out[g] = vexch[pos];
            }
        }
    }
}

template <typename UK> struct SortCfg { static constexpr int KPT = 16; };
template <> struct SortCfg<uint64_t> { static constexpr int KPT = 8; };

template <typename UK, bool PAIRS>
static size_t sweep_smem() {
    constexpr int TILE = kSortThreads * SortCfg<UK>::KPT;
    return (size_t)(kSortWarps * 256 + 512) * 4 + (size_t)TILE * sizeof(UK) + (PAIRS ? (size_t)TILE * 4 : 0);
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// x: raw keys (n).  perm == nullptr: sort x in place.  Otherwise x is left untouched and perm
// receives the stable 1-based permutation.
template <typename UK>
static int32_t radix_sort(b200_stream_t st, void* x, int64_t* perm, uint32_t n, int kind, int rev, uint64_t expmask) {
    constexpr int P = sizeof(UK);
    constexpr int KPT = SortCfg<UK>::KPT;
    constexpr int TILE = kSortThreads * KPT;
    const uint32_t ntiles = (n + TILE - 1) / TILE;
    const bool pairs = perm != nullptr;

    const size_t hist_bytes = (size_t)P * 256 * 4;
    const size_t state_bytes = (size_t)P * ntiles * 256 * 4;
    const size_t keys_bytes = align_up((size_t)n * sizeof(UK), 256);
    const size_t vals_bytes = align_up((size_t)n * 4, 256);
    size_t total = align_up(hist_bytes + state_bytes, 256) + hist_bytes + 256 + keys_bytes;
    if (pairs) total += keys_bytes + 2 * vals_bytes;
    void* scr = nullptr;
    unsigned int* counters = nullptr;
    B200_TRY(scratch(st, total, &scr, &counters));
    uint8_t* p = reinterpret_cast<uint8_t*>(scr);
    uint32_t* ghist = reinterpret_cast<uint32_t*>(p);
    uint32_t* state = ghist + P * 256;
    p += align_up(hist_bytes + state_bytes, 256);
    uint32_t* bin_base = reinterpret_cast<uint32_t*>(p);
    p += align_up(hist_bytes, 256);
    UK* tmp0 = reinterpret_cast<UK*>(p);
    p += keys_bytes;
    UK* tmp1 = nullptr;
    uint32_t *v0 = nullptr, *v1 = nullptr;
    if (pairs) {
        tmp1 = reinterpret_cast<UK*>(p); p += keys_bytes;
        v0 = reinterpret_cast<uint32_t*>(p); p += vals_bytes;
        v1 = reinterpret_cast<uint32_t*>(p); p += vals_bytes;
    }
    B200_CUDA(cudaMemsetAsync(ghist, 0, hist_bytes + state_bytes, st->s));

    const int sms = sm_count(st->dev);
    uint32_t hblocks = (n + kSortThreads * 16 - 1) / (kSortThreads * 16);
    if (hblocks > (uint32_t)sms * 4) hblocks = sms * 4;
    if (hblocks == 0) hblocks = 1;
    sort_histogram_kernel<UK><<<hblocks, kSortThreads, 0, st->s>>>((const UK*)x, n, kind, rev, (UK)expmask, ghist);
    sort_scan_histogram_kernel<<<P, 256, 0, st->s>>>(ghist, bin_base);

    uint32_t max_polls = 1u << 22;
    if (const char* e = getenv("B200_LOOKBACK_POLLS")) {
        long v = atol(e);
        if (v > 0) max_polls = (uint32_t)v;
    }
    unsigned int* ticket = counters + (kCounterBytes / sizeof(unsigned int) - 2);

    const size_t smem = pairs ? sweep_smem<UK, true>() : sweep_smem<UK, false>();
    if (pairs) B200_CUDA(cudaFuncSetAttribute(onesweep_kernel<UK, KPT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    else B200_CUDA(cudaFuncSetAttribute(onesweep_kernel<UK, KPT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));

    for (int pass = 0; pass < P; ++pass) {
        SweepArgs a{};
        a.n = n;
        a.ntiles = ntiles;
        a.shift = 8 * pass;
        a.first = pass == 0;
        a.last = pass == P - 1;
        a.kind = kind;
        a.rev = rev;
        a.expmask = expmask;
        a.bin_base = bin_base + pass * 256;
        a.state = state + (size_t)pass * ntiles * 256;
        a.ticket = ticket;
        a.err_word = device_error_word(st->dev);
        a.max_polls = max_polls;
        if (!pairs) {
            // x -> tmp0 -> x -> ... ; P is even, so the last pass lands in x
            a.keys_in = (pass % 2 == 0) ? x : (void*)tmp0;
            a.keys_out = (pass % 2 == 0) ? (void*)tmp0 : x;
            onesweep_kernel<UK, KPT, false><<<ntiles, kSortThreads, smem, st->s>>>(a);
        } else {
            // x -> (tmp0,v0) -> (tmp1,v1) -> (tmp0,v0) ... -> perm
            a.keys_in = pass == 0 ? x : (void*)((pass % 2 == 1) ? tmp0 : tmp1);
            a.keys_out = (pass % 2 == 0) ? tmp0 : tmp1;
            a.vals_in = (pass % 2 == 1) ? v0 : v1;
            a.vals_out = (pass % 2 == 0) ? v0 : v1;
            a.gen_index = pass == 0;
            a.last = 0;
            if (pass == P - 1) a.perm_out = perm;
            onesweep_kernel<UK, KPT, true><<<ntiles, kSortThreads, smem, st->s>>>(a);
        }
    }
    return B200_OK;
}

static int32_t key_info(int dtype, int* kind, uint64_t* expmask, int* width) {
    *expmask = 0;
    switch (dtype) {
        case B200_U16: *kind = KIND_UNSIGNED; *width = 2; return B200_OK;
        case B200_U32: *kind = KIND_UNSIGNED; *width = 4; return B200_OK;
        case B200_U64: *kind = KIND_UNSIGNED; *width = 8; return B200_OK;
        case B200_I16: *kind = KIND_SIGNED; *width = 2; return B200_OK;
        case B200_I32: *kind = KIND_SIGNED; *width = 4; return B200_OK;
        case B200_I64: *kind = KIND_SIGNED; *width = 8; return B200_OK;
        case B200_F16: *kind = KIND_FLOAT; *width = 2; *expmask = 0x7c00; return B200_OK;
        case B200_BF16: *kind = KIND_FLOAT; *width = 2; *expmask = 0x7f80; return B200_OK;
        case B200_F32: *kind = KIND_FLOAT; *width = 4; *expmask = 0x7f800000u; return B200_OK;
        case B200_F64: *kind = KIND_FLOAT; *width = 8; *expmask = 0x7ff0000000000000ull; return B200_OK;
        default: return fail(B200_UNSUPPORTED, "sort: element type %d is not supported", dtype);
    }
}

static int32_t sort_common(b200_stream_t st, const b200_tensor* x, const b200_tensor* ix, int32_t rev, const char* who) {
    B200_TRY(enter(st));
    StreamGuard guard(st);
    B200_TRY(check_tensor(x, who));
    int64_t n = tensor_numel(x);
    int nd = 0;
    for (int d = 0; d < x->ndim; ++d) if (x->shape[d] > 1) ++nd;
    if (nd > 1) return fail(B200_UNSUPPORTED, "%s: only vectors are supported", who);
    if (!tensor_is_contiguous(x)) return fail(B200_UNSUPPORTED, "%s: the vector must be dense", who);
    int64_t* perm = nullptr;
    if (ix) {
        B200_TRY(check_tensor(ix, who));
        if (ix->dtype != B200_I64) return fail(B200_UNSUPPORTED, "%s: the index vector must be Int64", who);
        if (tensor_numel(ix) != n || !tensor_is_contiguous(ix)) return fail(B200_INVALID_ARG, "%s: index vector must be dense with the length of the keys", who);
        perm = reinterpret_cast<int64_t*>(ix->ptr);
    }
    if (n == 0) return B200_OK;
    if (n >= ((int64_t)1 << 30)) return fail(B200_TOO_LARGE, "%s: at most 2^30-1 elements", who);
    int kind, width;
    uint64_t expmask;
    B200_TRY(key_info(x->dtype, &kind, &expmask, &width));
    int32_t s;
    switch (width) {
        case 2: s = radix_sort<uint16_t>(st, x->ptr, perm, (uint32_t)n, kind, rev ? 1 : 0, expmask); break;
        case 4: s = radix_sort<uint32_t>(st, x->ptr, perm, (uint32_t)n, kind, rev ? 1 : 0, expmask); break;
        default: s = radix_sort<uint64_t>(st, x->ptr, perm, (uint32_t)n, kind, rev ? 1 : 0, expmask); break;
    }
    B200_TRY(s);
    return finish(st, who);
}

}  // namespace b200

using namespace b200;

extern "C" int32_t b200_sort(b200_stream_t st, const b200_tensor* x, int32_t rev) {
    return sort_common(st, x, nullptr, rev, "sort!");
}

extern "C" int32_t b200_sortperm(b200_stream_t st, const b200_tensor* ix, const b200_tensor* x, int32_t rev) {
    if (!ix) return fail(B200_INVALID_ARG, "sortperm!: null index vector");
    return sort_common(st, x, ix, rev, "sortperm!");
}

