// accumulate! / cumsum / cumprod: B[i] = op(B[i-1], A[i]) along one dimension.
//
// Takes the place of AK.accumulate! as called from src/kernels/accumulate.jl:1-8 of the
// reference.  The main kernel is a single-pass chained scan with decoupled look-back: every
// tile of 1024 16-byte vectors is read once and written once (8 bytes per 4-byte element),
// publishes its aggregate, and resolves its exclusive prefix by inspecting 32 predecessor
// descriptors at a time.  Tiles take their index from an atomic ticket so that a tile's
// predecessors are always already running, and every wait is bounded: a tile that runs out of
// its poll budget latches B200_LOOKBACK_TIMEOUT in the device's error word and leaves; other
// waiters notice the latched word and leave too.
//
// The array is collapsed to (K, L, M) around the scanned dimension.  K*M independent columns
// of L elements (element stride K) run through the same kernel; very short columns and wide
// strided layouts use one thread per column, which is already coalesced for them.
#include "program.cuh"

#include <cstring>
#include <limits>
#include <mutex>
#include <type_traits>

namespace b200 {

constexpr int kScanThreads = 256;
constexpr int kScanVecs = 4;               // 16-byte vectors per thread
constexpr int kScanWarps = kScanThreads / 32;
static_assert(kScanVecs * kScanWarps == 32, "warp totals must fill exactly one warp");

enum : uint32_t { FLAG_EMPTY = 0, FLAG_AGGREGATE = 1, FLAG_PREFIX = 2 };

template <typename Acc, int OP>
__device__ __forceinline__ Acc scan_identity() {
    if constexpr (OP == B200_RED_ADD) return Acc(0);
    else if constexpr (OP == B200_RED_MUL) return Acc(1);
    else if constexpr (OP == B200_RED_MAX) {
        if constexpr (std::is_floating_point<Acc>::value) return -std::numeric_limits<Acc>::infinity();
        else return std::numeric_limits<Acc>::lowest();
    } else {
        if constexpr (std::is_floating_point<Acc>::value) return std::numeric_limits<Acc>::infinity();
        else return std::numeric_limits<Acc>::max();
    }
}
template <typename Acc, int OP>
__device__ __forceinline__ Acc scan_apply(Acc a, Acc b) {
    using A = Arith<Acc>;
    if constexpr (OP == B200_RED_ADD) return A::add(a, b);
    else if constexpr (OP == B200_RED_MUL) return A::mul(a, b);
    else if constexpr (OP == B200_RED_MAX) return A::max(a, b);
    else return A::min(a, b);
}

template <typename T> struct ScanAcc { using type = T; };
template <> struct ScanAcc<__half> { using type = float; };
template <> struct ScanAcc<__nv_bfloat16> { using type = float; };
template <typename T> __device__ __forceinline__ typename ScanAcc<T>::type scan_up(T v) { return v; }
template <> __device__ __forceinline__ float scan_up<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float scan_up<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T scan_down(typename ScanAcc<T>::type v) { return (T)v; }
template <> __device__ __forceinline__ __half scan_down<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 scan_down<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- tile descriptors ---------------------------------------------------------------------------------
// 4-byte accumulators: one 64-bit word {flag:32 | value:32}, written and read with single accesses.
// 8-byte accumulators: flag word plus two value slots, ordered by fences.
template <typename Acc, bool SMALL = (sizeof(Acc) == 4)>
struct TileState;

template <typename Acc>
struct TileState<Acc, true> {
    unsigned long long* words;
    static size_t bytes(int64_t ntiles) { return (size_t)ntiles * 8; }
    __host__ __device__ void bind(void* p, int64_t) { words = reinterpret_cast<unsigned long long*>(p); }
    __device__ __forceinline__ void publish(int64_t t, uint32_t flag, Acc v) {
        uint32_t bits;
        memcpy(&bits, &v, 4);
        *reinterpret_cast<volatile unsigned long long*>(words + t) = ((unsigned long long)flag << 32) | bits;
    }
    __device__ __forceinline__ uint32_t peek(int64_t t, Acc& v) {
        const unsigned long long w = *reinterpret_cast<volatile unsigned long long*>(words + t);
        const uint32_t bits = (uint32_t)w;
        memcpy(&v, &bits, 4);
        return (uint32_t)(w >> 32);
    }
};

template <typename Acc>
struct TileState<Acc, false> {
    uint32_t* flags;
    Acc* agg;
    Acc* pre;
    static size_t bytes(int64_t ntiles) { return (size_t)ntiles * (8 + 8 + 8); }
    __host__ __device__ void bind(void* p, int64_t ntiles) {
        agg = reinterpret_cast<Acc*>(p);
        pre = agg + ntiles;
        flags = reinterpret_cast<uint32_t*>(pre + ntiles);
    }
    __device__ __forceinline__ void publish(int64_t t, uint32_t flag, Acc v) {
        if (flag == FLAG_AGGREGATE) *reinterpret_cast<volatile Acc*>(agg + t) = v;
        else *reinterpret_cast<volatile Acc*>(pre + t) = v;
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(flags + t) = flag;
    }
    __device__ __forceinline__ uint32_t peek(int64_t t, Acc& v) {
        const uint32_t f = *reinterpret_cast<volatile uint32_t*>(flags + t);
        if (f == FLAG_EMPTY) return f;
        __threadfence();
        v = (f == FLAG_AGGREGATE) ? *reinterpret_cast<volatile Acc*>(agg + t) : *reinterpret_cast<volatile Acc*>(pre + t);
        return f;
    }
};

struct ScanPlan {
    int64_t K, L, M;         // columns c = (k, m): base k + K*L*m, element stride K
    int64_t tiles_per_col;
    int64_t ntiles;
    int32_t vec_ok;          // K == 1 and every column start is 16-byte aligned in A and B
    int32_t inclusive;
    int32_t has_init;
    uint32_t max_polls;
    uint64_t init;           // accumulator class bits (has_init == 1)
    const void* init_dev;    // one element of the array's type in device memory (has_init == 2)
};

template <typename T>
__device__ __forceinline__ typename ScanAcc<T>::type scan_seed(const ScanPlan& pl) {
    using Acc = typename ScanAcc<T>::type;
    if (pl.has_init == 2) return scan_up<T>(*reinterpret_cast<const T*>(pl.init_dev));
    return as_c<Acc, uint64_t>(pl.init);
}

// Inclusive warp scan over lanes; returns the inclusive value.
template <typename Acc, int OP>
__device__ __forceinline__ Acc warp_scan_inclusive(Acc v, int lane) {
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        Acc o = __shfl_up_sync(0xffffffffu, v, off);
        if (lane >= off) v = scan_apply<Acc, OP>(o, v);
    }
    return v;
}

template <typename T, int OP>
__global__ void __launch_bounds__(kScanThreads)
scan_lookback_kernel(const T* A, T* B, ScanPlan pl, void* state_mem, unsigned int* ticket, int32_t* err_word) {
    using Acc = typename ScanAcc<T>::type;
    constexpr int V = 16 / sizeof(T);
    constexpr int TILE = kScanThreads * kScanVecs * V;
    using VT = Vec<T, V>;

    __shared__ long long s_tile;
    __shared__ Acc s_warp[32];
    __shared__ Acc s_wex[32];
    __shared__ Acc s_prefix;
    __shared__ int s_abort;

    TileState<Acc> state;
    state.bind(state_mem, pl.ntiles);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        const unsigned int t = atomicAdd(ticket, 1u);
        if ((int64_t)t == pl.ntiles - 1) *ticket = 0;   // nobody takes a ticket after the last tile
        s_tile = t;
        s_abort = 0;
    }
    __syncthreads();
    const int64_t tile = s_tile;
    const int64_t col = tile / pl.tiles_per_col;
    const int64_t jt = tile - col * pl.tiles_per_col;   // tile index inside the column
    const int64_t m = col / pl.K, k = col - m * pl.K;
    const int64_t col_base = k + pl.K * pl.L * m;
    const int64_t e0 = jt * TILE;                        // first element of the tile in its column
    const int64_t left = pl.L - e0;
    const int count = left < TILE ? (int)left : TILE;

    // ---- load: vector j of thread tid covers elements (j*threads + tid)*V .. +V of the tile
    Acc x[kScanVecs][V];
    const bool full = (count == TILE);
    if (pl.vec_ok && full) {
        const uint4* src = reinterpret_cast<const uint4*>(A + col_base + e0);
#pragma unroll
        for (int j = 0; j < kScanVecs; ++j) {
            VT v = __builtin_bit_cast(VT, __ldcs(src + j * kScanThreads + tid));
#pragma unroll
            for (int q = 0; q < V; ++q) x[j][q] = scan_up<T>(v.v[q]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < kScanVecs; ++j)
#pragma unroll
            for (int q = 0; q < V; ++q) {
                const int e = (j * kScanThreads + tid) * V + q;
                x[j][q] = e < count ? scan_up<T>(A[col_base + (e0 + e) * pl.K]) : scan_identity<Acc, OP>();
            }
    }

    // ---- thread-local inclusive scans per vector, then warp scans of the vector totals
    Acc lane_ex[kScanVecs];
#pragma unroll
    for (int j = 0; j < kScanVecs; ++j) {
#pragma unroll
        for (int q = 1; q < V; ++q) x[j][q] = scan_apply<Acc, OP>(x[j][q - 1], x[j][q]);
        const Acc inc = warp_scan_inclusive<Acc, OP>(x[j][V - 1], lane);
        Acc ex = __shfl_up_sync(0xffffffffu, inc, 1);
        if (lane == 0) ex = scan_identity<Acc, OP>();
        lane_ex[j] = ex;
        if (lane == 31) s_warp[j * kScanWarps + warp] = inc;
    }
    __syncthreads();

    // ---- warp 0: scan the 32 warp totals, publish, look back
    if (warp == 0) {
        const Acc wt = s_warp[lane];
        const Acc winc = warp_scan_inclusive<Acc, OP>(wt, lane);
        Acc wex = __shfl_up_sync(0xffffffffu, winc, 1);
        if (lane == 0) wex = scan_identity<Acc, OP>();
        s_wex[lane] = wex;
        const Acc aggregate = __shfl_sync(0xffffffffu, winc, 31);

        Acc prefix = scan_identity<Acc, OP>();
        bool have_prefix = false;
        if (jt == 0) {
            if (pl.has_init) { prefix = scan_seed<T>(pl); have_prefix = true; }
            if (lane == 0) state.publish(tile, FLAG_PREFIX, have_prefix ? scan_apply<Acc, OP>(prefix, aggregate) : aggregate);
        } else {
            if (lane == 0) state.publish(tile, FLAG_AGGREGATE, aggregate);
            // window of 32 predecessors: lane i inspects tile - 1 - i (of the same column)
            int64_t look = jt - 1;        // column-local index of the nearest uninspected predecessor
            bool done = false, abort = false;
            Acc running = scan_identity<Acc, OP>();
            bool running_set = false;
            while (!done && !abort) {
                const int64_t mine = look - lane;
                Acc val = scan_identity<Acc, OP>();
                uint32_t flag = FLAG_PREFIX;     // positions before the column start terminate the walk
                bool real = mine >= 0;
                if (real) {
                    uint32_t polls = 0;
                    flag = state.peek(col * pl.tiles_per_col + mine, val);
                    while (flag == FLAG_EMPTY) {
                        ++polls;
                        if (polls > pl.max_polls) { abort = true; break; }
                        if ((polls & 1023u) == 0 && error_latched(err_word)) { abort = true; break; }
                        if (polls > 32) __nanosleep(polls > 4096 ? 256 : 32);
                        flag = state.peek(col * pl.tiles_per_col + mine, val);
                    }
                }
                abort = __any_sync(0xffffffffu, abort);
                if (abort) break;
                // nearest lane (smallest index) that holds a full prefix ends the walk
                const uint32_t pmask = __ballot_sync(0xffffffffu, flag == FLAG_PREFIX);
                const int stop = pmask ? (__ffs(pmask) - 1) : 32;
                // combine values of lanes 0..stop in tile order (farthest first)
                Acc contrib = (lane <= stop && (real || lane < stop)) ? val : scan_identity<Acc, OP>();
                if (!real) contrib = scan_identity<Acc, OP>();
                // reverse-order inclusive combine: result at lane 0 = v[stop] op ... op v[1] op v[0]
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    Acc o = __shfl_down_sync(0xffffffffu, contrib, off);
                    if (lane + off < 32) contrib = scan_apply<Acc, OP>(o, contrib);
                }
                const Acc window = __shfl_sync(0xffffffffu, contrib, 0);
                running = running_set ? scan_apply<Acc, OP>(window, running) : window;
                running_set = true;
                if (stop < 32) done = true;
                else look -= 32;
            }
            if (abort) {
                if (lane == 0) { latch_error(err_word, B200_LOOKBACK_TIMEOUT); s_abort = 1; }
            } else {
                prefix = running;
                have_prefix = true;
                if (lane == 0) state.publish(tile, FLAG_PREFIX, scan_apply<Acc, OP>(prefix, aggregate));
            }
        }
        if (lane == 0) s_prefix = prefix;
    }
    __syncthreads();
    if (s_abort) return;

    // ---- apply offsets and store
    const Acc tile_prefix = s_prefix;
    const bool seeded = (jt != 0) || pl.has_init;
#pragma unroll
    for (int j = 0; j < kScanVecs; ++j) {
        Acc off = scan_apply<Acc, OP>(s_wex[j * kScanWarps + warp], lane_ex[j]);
        if (seeded) off = scan_apply<Acc, OP>(tile_prefix, off);
        VT out;
        if (pl.inclusive) {
#pragma unroll
            for (int q = 0; q < V; ++q) out.v[q] = scan_down<T>(scan_apply<Acc, OP>(off, x[j][q]));
        } else {
            out.v[0] = scan_down<T>(off);
#pragma unroll
            for (int q = 1; q < V; ++q) out.v[q] = scan_down<T>(scan_apply<Acc, OP>(off, x[j][q - 1]));
        }
        if (pl.vec_ok && full) {
            __stcs(reinterpret_cast<uint4*>(B + col_base + e0) + j * kScanThreads + tid, __builtin_bit_cast(uint4, out));
        } else {
#pragma unroll
            for (int q = 0; q < V; ++q) {
                const int e = (j * kScanThreads + tid) * V + q;
                if (e < count) B[col_base + (e0 + e) * pl.K] = out.v[q];
            }
        }
    }
}

// One thread per column: sequential walk, coalesced across neighbouring columns when K > 1.
template <typename T, int OP>
__global__ void __launch_bounds__(256)
scan_column_thread_kernel(const T* A, T* B, ScanPlan pl) {
    using Acc = typename ScanAcc<T>::type;
    const int64_t ncols = pl.K * pl.M;
    const int64_t nthr = (int64_t)gridDim.x * blockDim.x;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < ncols; c += nthr) {
        const int64_t m = c / pl.K, k = c - m * pl.K;
        const int64_t base = k + pl.K * pl.L * m;
        Acc acc = pl.has_init ? scan_seed<T>(pl) : scan_identity<Acc, OP>();
        bool seeded = pl.has_init != 0;
        for (int64_t l = 0; l < pl.L; ++l) {
            const Acc v = scan_up<T>(A[base + l * pl.K]);
            const Acc next = seeded ? scan_apply<Acc, OP>(acc, v) : v;
            B[base + l * pl.K] = scan_down<T>(pl.inclusive ? next : acc);
            acc = next;
            seeded = true;
        }
    }
}

template <typename T, int OP>
static int32_t launch_scan(b200_stream_t st, const void* A, void* B, ScanPlan pl) {
    using Acc = typename ScanAcc<T>::type;
    constexpr int V = 16 / sizeof(T);
    constexpr int TILE = kScanThreads * kScanVecs * V;
    const int64_t ncols = pl.K * pl.M;
    const int64_t target = (int64_t)sm_count(st->dev) * 8;
    const bool thread_cols = (pl.L <= 32 && ncols >= 1024) || (pl.K > 1 && ncols >= 4096);
    if (thread_cols) {
        int64_t blocks = (ncols + 255) / 256;
        if (blocks > target) blocks = target;
        scan_column_thread_kernel<T, OP><<<(unsigned)blocks, 256, 0, st->s>>>((const T*)A, (T*)B, pl);
        return B200_OK;
    }
    pl.tiles_per_col = (pl.L + TILE - 1) / TILE;
    pl.ntiles = pl.tiles_per_col * ncols;
    if (pl.ntiles >= (int64_t)1 << 31) return fail(B200_TOO_LARGE, "accumulate: too many tiles");
    const bool aligned = reinterpret_cast<uintptr_t>(A) % 16 == 0 && reinterpret_cast<uintptr_t>(B) % 16 == 0;
    pl.vec_ok = (pl.K == 1 && aligned && (ncols == 1 || (pl.L * sizeof(T)) % 16 == 0)) ? 1 : 0;
    void* scr = nullptr;
    unsigned int* counters = nullptr;
    const size_t sbytes = TileState<Acc>::bytes(pl.ntiles);
    B200_TRY(scratch(st, sbytes, &scr, &counters));
    B200_CUDA(cudaMemsetAsync(scr, 0, sbytes, st->s));
    // the last counter slot serves as the tile ticket (it returns to zero by itself)
    unsigned int* ticket = counters + (kCounterBytes / sizeof(unsigned int) - 1);
    scan_lookback_kernel<T, OP><<<(unsigned)pl.ntiles, kScanThreads, 0, st->s>>>(
        (const T*)A, (T*)B, pl, scr, ticket, device_error_word(st->dev));
    return B200_OK;
}

template <typename T>
static int32_t launch_scan_op(b200_stream_t st, const void* A, void* B, const ScanPlan& pl, int op) {
    switch (op) {
        case B200_RED_ADD: return launch_scan<T, B200_RED_ADD>(st, A, B, pl);
        case B200_RED_MUL: return launch_scan<T, B200_RED_MUL>(st, A, B, pl);
        case B200_RED_MAX: return launch_scan<T, B200_RED_MAX>(st, A, B, pl);
        default: return launch_scan<T, B200_RED_MIN>(st, A, B, pl);
    }
}


// ---- scan without any allocation ---------------------------------------------------------------------
// Some callers may not allocate at all once they are running: a service that handed every byte
// of device memory to its own arena at start-up, a plug-in whose host forbids driver and pool
// allocations after initialisation, a control loop with a fixed latency budget that cannot absorb
// an allocator call.  For them the look-back descriptors and the tile ticket live in this
// file-scope device array instead of the stream's pool-backed scratch.  Every device that loads the
// library carries the array (1 MiB) until the process exits.
constexpr size_t kStaticScanBytes = size_t(1) << 20;
constexpr size_t kStaticScanHeader = 256;            // ticket word, then the descriptors
static __device__ __align__(256) unsigned char g_scan_static[kStaticScanBytes];

constexpr int kStaticMaxDevices = 64;
static std::mutex g_static_mu;
static void* g_static_addr[kStaticMaxDevices] = {nullptr};

// Device address of g_scan_static on the CURRENT device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel could use; the real address differs per device
// and is looked up once per device, with that device current.
static int32_t static_scan_scratch(int dev, void** out) {
    if (dev < 0 || dev >= kStaticMaxDevices) return fail(B200_INVALID_ARG, "device %d outside the static-scratch table", dev);
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_addr[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_scan_static);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_scan_static)");
        g_static_addr[dev] = p;
    }
    *out = g_static_addr[dev];
    return B200_OK;
}

template <typename T, int OP>
static int32_t launch_scan_static(b200_stream_t st, const void* A, void* B, ScanPlan pl) {
    using Acc = typename ScanAcc<T>::type;
    constexpr int V = 16 / sizeof(T);
    constexpr int TILE = kScanThreads * kScanVecs * V;
    const int64_t ncols = pl.K * pl.M;
    const int64_t target = (int64_t)sm_count(st->dev) * 8;
    const bool thread_cols = (pl.L <= 32 && ncols >= 1024) || (pl.K > 1 && ncols >= 4096);
    if (thread_cols) {   // this shape needs no scratch at all
        int64_t blocks = (ncols + 255) / 256;
        if (blocks > target) blocks = target;
        scan_column_thread_kernel<T, OP><<<(unsigned)blocks, 256, 0, st->s>>>((const T*)A, (T*)B, pl);
        return B200_OK;
    }
    pl.tiles_per_col = (pl.L + TILE - 1) / TILE;
    pl.ntiles = pl.tiles_per_col * ncols;
    const size_t state_bytes = TileState<Acc>::bytes(pl.ntiles);
    const int64_t max_tiles = (int64_t)((kStaticScanBytes - kStaticScanHeader) / TileState<Acc>::bytes(1));
    if (pl.ntiles > max_tiles)
        return fail(B200_TOO_LARGE, "accumulate (no-allocation variant): %lld tiles of %d elements needed, the built-in "
                    "scratch holds %lld for this element type; use b200_accumulate for larger inputs",
                    (long long)pl.ntiles, TILE, (long long)max_tiles);
    void* base = nullptr;
    B200_TRY(static_scan_scratch(st->dev, &base));
    const bool aligned = reinterpret_cast<uintptr_t>(A) % 16 == 0 && reinterpret_cast<uintptr_t>(B) % 16 == 0;
    pl.vec_ok = (pl.K == 1 && aligned && (ncols == 1 || (pl.L * sizeof(T)) % 16 == 0)) ? 1 : 0;
    // the array keeps whatever the previous call left: ticket and descriptors must start at zero
    B200_CUDA(cudaMemsetAsync(base, 0, kStaticScanHeader + state_bytes, st->s));
    scan_lookback_kernel<T, OP><<<(unsigned)pl.ntiles, kScanThreads, 0, st->s>>>(
        (const T*)A, (T*)B, pl, reinterpret_cast<unsigned char*>(base) + kStaticScanHeader,
        reinterpret_cast<unsigned int*>(base), device_error_word(st->dev));
    return B200_OK;
}

template <typename T>
static int32_t launch_scan_static_op(b200_stream_t st, const void* A, void* B, const ScanPlan& pl, int op) {
    switch (op) {
        case B200_RED_ADD: return launch_scan_static<T, B200_RED_ADD>(st, A, B, pl);
        case B200_RED_MUL: return launch_scan_static<T, B200_RED_MUL>(st, A, B, pl);
        case B200_RED_MAX: return launch_scan_static<T, B200_RED_MAX>(st, A, B, pl);
        default: return launch_scan_static<T, B200_RED_MIN>(st, A, B, pl);
    }
}

}  // namespace b200

using namespace b200;

static int32_t accumulate_common(b200_stream_t st, const b200_tensor* B, const b200_tensor* A, int32_t op,
                                 const void* init, const void* init_dev, int32_t dim, int32_t inclusive) {
    B200_TRY(enter(st));
    B200_TRY(check_tensor(B, "accumulate destination"));
    B200_TRY(check_tensor(A, "accumulate source"));
    if (op < 0 || op >= B200_RED_COUNT) return fail(B200_UNSUPPORTED, "accumulate: unknown operator %d", op);
    if (A->dtype != B->dtype) return fail(B200_UNSUPPORTED, "accumulate: source and destination element types differ");
    if (A->ndim != B->ndim) return fail(B200_INVALID_ARG, "accumulate: source and destination shapes differ");
    for (int d = 0; d < A->ndim; ++d)
        if (A->shape[d] != B->shape[d]) return fail(B200_INVALID_ARG, "accumulate: source and destination shapes differ");
    if (!tensor_is_contiguous(A) || !tensor_is_contiguous(B))
        return fail(B200_UNSUPPORTED, "accumulate: operands must be dense column-major arrays");
    const int64_t n = tensor_numel(A);
    if (n == 0) return B200_OK;
    if (dim < 0) return fail(B200_INVALID_ARG, "accumulate: negative dimension");

    ScanPlan pl{};
    pl.K = 1; pl.L = 1; pl.M = 1;
    for (int d = 0; d < A->ndim; ++d) {
        if (d < dim) pl.K *= A->shape[d];
        else if (d == dim) pl.L = A->shape[d];
        else pl.M *= A->shape[d];
    }
    pl.inclusive = inclusive ? 1 : 0;
    pl.has_init = init_dev ? 2 : (init ? 1 : 0);
    pl.init_dev = init_dev;
    if (init) {
        uint64_t bits = 0;
        memcpy(&bits, init, dtype_size(A->dtype));
        pl.init = scalar_to_class(A->dtype, bits);
    }
    pl.max_polls = 1u << 22;
    if (const char* e = getenv("B200_LOOKBACK_POLLS")) {
        long v = atol(e);
        if (v > 0) pl.max_polls = (uint32_t)v;
    }
    int32_t s;
    switch (A->dtype) {
        case B200_F32: s = launch_scan_op<float>(st, A->ptr, B->ptr, pl, op); break;
        case B200_F64: s = launch_scan_op<double>(st, A->ptr, B->ptr, pl, op); break;
        case B200_I32: s = launch_scan_op<int32_t>(st, A->ptr, B->ptr, pl, op); break;
        case B200_I64: s = launch_scan_op<int64_t>(st, A->ptr, B->ptr, pl, op); break;
        case B200_U32: s = launch_scan_op<uint32_t>(st, A->ptr, B->ptr, pl, op); break;
        case B200_U64: s = launch_scan_op<uint64_t>(st, A->ptr, B->ptr, pl, op); break;
        case B200_F16: s = launch_scan_op<__half>(st, A->ptr, B->ptr, pl, op); break;
        case B200_BF16: s = launch_scan_op<__nv_bfloat16>(st, A->ptr, B->ptr, pl, op); break;
        default: return fail(B200_UNSUPPORTED, "accumulate: element type %d is not supported", A->dtype);
    }
    B200_TRY(s);
    return finish(st, "b200_accumulate");
}

extern "C" int32_t b200_accumulate(b200_stream_t st, const b200_tensor* B, const b200_tensor* A, int32_t op,
                                   const void* init, int32_t dim, int32_t inclusive) {
    return accumulate_common(st, B, A, op, init, nullptr, dim, inclusive);
}

extern "C" int32_t b200_accumulate_carry(b200_stream_t st, const b200_tensor* B, const b200_tensor* A, int32_t op,
                                         const void* carry_dev, int32_t dim, int32_t inclusive) {
    if (!carry_dev) return fail(B200_INVALID_ARG, "accumulate: null carry pointer");
    return accumulate_common(st, B, A, op, nullptr, carry_dev, dim, inclusive);
}

// Allocation-free accumulate!: same arguments and results as b200_accumulate, but the scan's
// bookkeeping lives in a 1 MiB array built into the library, so the call never reaches an
// allocator (no cudaMalloc, no pool, no stream scratch).  Limits and rules:
//   * at most 131040 tiles for 4-byte (and 16-bit) element types, 43680 for 8-byte ones; a tile is
//     4096 four-byte, 2048 eight-byte or 8192 two-byte elements, and every scanned column takes
//     at least one tile - larger inputs are refused with B200_TOO_LARGE;
//   * the first call on each device looks up the array's device address; make that call during
//     start-up, before any stream capture begins;
//   * all calls on a device share the one array: two calls whose kernels could overlap on the GPU
//     (different streams without ordering between them) corrupt each other - keep them ordered.
extern "C" int32_t b200_accumulate_noalloc(b200_stream_t st, const b200_tensor* B, const b200_tensor* A, int32_t op,
                                           const void* init, int32_t dim, int32_t inclusive) {
    B200_TRY(enter(st));
    B200_TRY(check_tensor(B, "accumulate destination"));
    B200_TRY(check_tensor(A, "accumulate source"));
    if (op < 0 || op >= B200_RED_COUNT) return fail(B200_UNSUPPORTED, "accumulate: unknown operator %d", op);
    if (A->dtype != B->dtype) return fail(B200_UNSUPPORTED, "accumulate: source and destination element types differ");
    if (A->ndim != B->ndim) return fail(B200_INVALID_ARG, "accumulate: source and destination shapes differ");
    for (int d = 0; d < A->ndim; ++d)
        if (A->shape[d] != B->shape[d]) return fail(B200_INVALID_ARG, "accumulate: source and destination shapes differ");
    if (!tensor_is_contiguous(A) || !tensor_is_contiguous(B))
        return fail(B200_UNSUPPORTED, "accumulate: operands must be dense column-major arrays");
    if (tensor_numel(A) == 0) return B200_OK;
    if (dim < 0) return fail(B200_INVALID_ARG, "accumulate: negative dimension");
    ScanPlan pl{};
    pl.K = 1; pl.L = 1; pl.M = 1;
    for (int d = 0; d < A->ndim; ++d) {
        if (d < dim) pl.K *= A->shape[d];
        else if (d == dim) pl.L = A->shape[d];
        else pl.M *= A->shape[d];
    }
    pl.inclusive = inclusive ? 1 : 0;
    pl.has_init = init ? 1 : 0;
    if (init) {
        uint64_t bits = 0;
        memcpy(&bits, init, dtype_size(A->dtype));
        pl.init = scalar_to_class(A->dtype, bits);
    }
    pl.max_polls = 1u << 22;
    int32_t s;
    switch (A->dtype) {
        case B200_F32: s = launch_scan_static_op<float>(st, A->ptr, B->ptr, pl, op); break;
        case B200_F64: s = launch_scan_static_op<double>(st, A->ptr, B->ptr, pl, op); break;
        case B200_I32: s = launch_scan_static_op<int32_t>(st, A->ptr, B->ptr, pl, op); break;
        case B200_I64: s = launch_scan_static_op<int64_t>(st, A->ptr, B->ptr, pl, op); break;
        case B200_U32: s = launch_scan_static_op<uint32_t>(st, A->ptr, B->ptr, pl, op); break;
        case B200_U64: s = launch_scan_static_op<uint64_t>(st, A->ptr, B->ptr, pl, op); break;
        case B200_F16: s = launch_scan_static_op<__half>(st, A->ptr, B->ptr, pl, op); break;
        case B200_BF16: s = launch_scan_static_op<__nv_bfloat16>(st, A->ptr, B->ptr, pl, op); break;
        default: return fail(B200_UNSUPPORTED, "accumulate: element type %d is not supported", A->dtype);
    }
    B200_TRY(s);
    return finish(st, "b200_accumulate_noalloc");
}
