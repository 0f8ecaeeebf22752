// accumulate! / cumsum / cumprod: B[i] = op(B[i-1], A[i]) along one dimension.
//
// Takes the place of AK.accumulate! as called from src/kernels/accumulate.jl:1-8 of the
// reference.  Four kernels share one descriptor protocol (aggregate / inclusive-prefix words
// that successors poll):
//  * long dense vectors: persistent two-pass segment scan (scan_segment_kernel).  A block reduces
//    a 16-48 KiB segment from HBM, publishes its aggregate, resolves the prefix with one
//    block-wide look-back, then scans the segment out of L2; both passes are software-pipelined,
//    HBM sees one read and one write per element (8 bytes per 4-byte element);
//  * everything else with enough work per column: one tile of 1024 16-byte vectors per block,
//    chained scan with decoupled look-back, 256 predecessor descriptors per round; tiles take
//    their index from an atomic ticket so that a tile's predecessors are always running;
//  * long scans down a strided dimension (dims > 1 with at least a warp of columns): tiles of
//    32*VEC columns x 128 rows chained along the scanned dimension, vector-valued descriptors;
//  * very short columns and narrow strided layouts: one thread per column.
// Every wait is bounded: a block that runs out of its poll budget latches B200_LOOKBACK_TIMEOUT
// in the device's error word and leaves; other waiters notice the latched word and leave too.
//
// The array is collapsed to (K, L, M) around the scanned dimension: K*M independent columns of
// L elements with element stride K.
#include "scan_common.cuh"

#include <cstdlib>
#include <cstring>
#include <limits>
#include <mutex>
#include <type_traits>

namespace b200 {

constexpr int kScanThreads = 256;
constexpr int kScanVecs = 4;               // 16-byte vectors per thread
constexpr int kScanWarps = kScanThreads / 32;
static_assert(kScanVecs * kScanWarps == 32, "warp totals must fill exactly one warp");

// ---- tile descriptors ---------------------------------------------------------------------------------
// Every descriptor is a 64-bit word whose upper half is a tag, (launch number << 2) | state, so
// that words written by earlier launches read as EMPTY and the words never have to be cleared
// between launches (launch number 0: the caller cleared them).  The words of a stream live in a
// buffer that holds nothing but such words (b200::scan_state), whatever kernel wrote them.
// 4-byte accumulators: the lower half of the word is the value, one access publishes both.
// 8-byte accumulators: the values sit in two arrays beside the words, ordered by fences.
__device__ __forceinline__ uint32_t tag_state(unsigned long long w, uint32_t epoch) {
    const uint32_t tag = (uint32_t)(w >> 32);
    return (tag >> 2) == epoch ? (tag & 3u) : FLAG_EMPTY;
}
__device__ __forceinline__ unsigned long long tag_word(uint32_t epoch, uint32_t state, uint32_t low = 0) {
    return ((unsigned long long)((epoch << 2) | state) << 32) | low;
}

template <typename Acc, bool SMALL = (sizeof(Acc) == 4)>
struct TileState;

template <typename Acc>
struct TileState<Acc, true> {
    unsigned long long* words;
    uint32_t epoch;
    static size_t flag_bytes(int64_t ntiles) { return (size_t)ntiles * 8; }
    static size_t value_bytes(int64_t) { return 0; }
    __host__ __device__ void bind(void* flag_mem, void*, int64_t, uint32_t e) {
        words = reinterpret_cast<unsigned long long*>(flag_mem);
        epoch = e;
    }
    __device__ __forceinline__ void publish(int64_t t, uint32_t flag, Acc v) {
        uint32_t bits;
        memcpy(&bits, &v, 4);
        *reinterpret_cast<volatile unsigned long long*>(words + t) = tag_word(epoch, flag, bits);
    }
    __device__ __forceinline__ uint32_t peek(int64_t t, Acc& v) {
        const unsigned long long w = *reinterpret_cast<volatile unsigned long long*>(words + t);
        const uint32_t bits = (uint32_t)w;
        memcpy(&v, &bits, 4);
        return tag_state(w, epoch);
    }
};

template <typename Acc>
struct TileState<Acc, false> {
    unsigned long long* flags;
    Acc* agg;
    Acc* pre;
    uint32_t epoch;
    static size_t flag_bytes(int64_t ntiles) { return (size_t)ntiles * 8; }
    static size_t value_bytes(int64_t ntiles) { return (size_t)ntiles * 16; }
    __host__ __device__ void bind(void* flag_mem, void* value_mem, int64_t ntiles, uint32_t e) {
        flags = reinterpret_cast<unsigned long long*>(flag_mem);
        agg = reinterpret_cast<Acc*>(value_mem);
        pre = agg + ntiles;
        epoch = e;
    }
    __device__ __forceinline__ void publish(int64_t t, uint32_t flag, Acc v) {
        if (flag == FLAG_AGGREGATE) *reinterpret_cast<volatile Acc*>(agg + t) = v;
        else *reinterpret_cast<volatile Acc*>(pre + t) = v;
        __threadfence();
        *reinterpret_cast<volatile unsigned long long*>(flags + t) = tag_word(epoch, flag);
    }
    __device__ __forceinline__ uint32_t peek(int64_t t, Acc& v) {
        const uint32_t f = tag_state(*reinterpret_cast<volatile unsigned long long*>(flags + t), epoch);
        if (f == FLAG_EMPTY) return f;
        __threadfence();
        v = (f == FLAG_AGGREGATE) ? *reinterpret_cast<volatile Acc*>(agg + t) : *reinterpret_cast<volatile Acc*>(pre + t);
        return f;
    }
};

// Descriptor words (in the stream's tagged buffer) and value storage (stream scratch) of one launch.
template <typename Acc>
static int32_t descriptor_storage(b200_stream_t st, int64_t ntiles, void** flag_mem, void** value_mem, uint32_t* epoch) {
    void* state = nullptr;
    bool must_clear = false;
    const size_t fbytes = TileState<Acc>::flag_bytes(ntiles);
    B200_TRY(scan_state(st, fbytes, &state, epoch, &must_clear));
    *flag_mem = reinterpret_cast<unsigned char*>(state) + kScanStateHeader;
    // a replayed graph repeats its launch number: a captured launch clears its words itself
    if (must_clear) B200_CUDA(cudaMemsetAsync(*flag_mem, 0, fbytes, st->s));
    *value_mem = nullptr;
    if (TileState<Acc>::value_bytes(ntiles)) B200_TRY(scratch(st, TileState<Acc>::value_bytes(ntiles), value_mem));
    return B200_OK;
}

template <typename T, int OP>
__global__ void __launch_bounds__(kScanThreads)
scan_lookback_kernel(const T* A, T* B, ScanPlan pl, void* state_mem, unsigned int* ticket, int32_t* err_word) {
    grid_dependency_wait();
    using Acc = typename ScanAcc<T>::type;
    constexpr int V = 16 / sizeof(T);
    constexpr int TILE = kScanThreads * kScanVecs * V;
    using VT = Vec<T, V>;

    __shared__ long long s_tile;
    __shared__ Acc s_warp[32];
    __shared__ Acc s_wex[32];
    __shared__ Acc s_prefix;
    __shared__ Acc s_aggregate;
    __shared__ int s_wflag[kScanWarps];
    __shared__ int s_verdict;
    __shared__ int s_abort;

    TileState<Acc> state;
    state.bind(state_mem, pl.value_mem, pl.ntiles, pl.epoch);

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

    // ---- warp 0: scan the 32 warp totals; the tile aggregate goes to shared memory
    if (warp == 0) {
        const Acc wt = s_warp[lane];
        const Acc winc = warp_scan_inclusive<Acc, OP>(wt, lane);
        Acc wex = __shfl_up_sync(0xffffffffu, winc, 1);
        if (lane == 0) wex = scan_identity<Acc, OP>();
        s_wex[lane] = wex;
        if (lane == 31) s_aggregate = winc;
    }
    __syncthreads();
    const Acc aggregate = s_aggregate;

    // ---- publish, then look back with the WHOLE block: thread t inspects predecessor
    // look - t, so one round covers 256 tiles.  (A 32-wide window lets the resolved frontier
    // advance only 32 tiles per L2 round trip, which caps the kernel far below HBM speed once
    // the first wave of blocks has started in lock step.)
    if (jt == 0) {
        if (tid == 0) {
            Acc prefix = scan_identity<Acc, OP>();
            if (pl.has_init) prefix = scan_seed<T>(pl);
            state.publish(tile, FLAG_PREFIX, pl.has_init ? scan_apply<Acc, OP>(prefix, aggregate) : aggregate);
            s_prefix = prefix;
        }
    } else {
        if (tid == 0) state.publish(tile, FLAG_AGGREGATE, aggregate);
        int64_t look = jt - 1;            // column-local index of the nearest uninspected predecessor
        Acc running = scan_identity<Acc, OP>();   // maintained by thread 0
        bool running_set = false;
        while (true) {
            const int64_t mine = look - tid;
            Acc val = scan_identity<Acc, OP>();
            uint32_t flag = FLAG_PREFIX;  // positions before the column start terminate the walk
            const bool real = mine >= 0;
            bool abort = false;
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
            // inside the warp: the nearest lane holding a full prefix ends the walk; lanes up to it
            // are combined in tile order (farthest first)
            const uint32_t pmask = __ballot_sync(0xffffffffu, !abort && flag == FLAG_PREFIX);
            const int stop = pmask ? (__ffs(pmask) - 1) : 32;
            Acc contrib = (lane <= stop && real && !abort) ? val : scan_identity<Acc, OP>();
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                Acc o = __shfl_down_sync(0xffffffffu, contrib, off);
                if (lane + off < 32) contrib = scan_apply<Acc, OP>(o, contrib);
            }
            if (lane == 0) {
                s_warp[warp] = contrib;                       // s_warp is free again at this point
                s_wflag[warp] = abort ? 2 : (stop < 32 ? 1 : 0);
            }
            __syncthreads();
            if (tid == 0) {
                int verdict = 0;                              // 0: walk on, 1: resolved, 2: give up
                for (int w = 0; w < kScanWarps; ++w) {        // warp 0 holds the nearest predecessors
                    if (s_wflag[w] == 2) { verdict = 2; break; }
                    running = running_set ? scan_apply<Acc, OP>(s_warp[w], running) : s_warp[w];
                    running_set = true;
                    if (s_wflag[w] == 1) { verdict = 1; break; }
                }
                s_verdict = verdict;
            }
            __syncthreads();
            const int verdict = s_verdict;
            if (verdict != 0) {
                if (tid == 0) {
                    if (verdict == 2) { latch_error(err_word, B200_LOOKBACK_TIMEOUT); s_abort = 1; }
                    else {
                        state.publish(tile, FLAG_PREFIX, scan_apply<Acc, OP>(running, aggregate));
                        s_prefix = running;
                    }
                }
                break;
            }
            look -= kScanThreads;
        }
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

// ---- persistent two-pass scan over L2-sized segments ----------------------------------------------------
// Long dense vectors.  On this part a dependent descriptor read costs microseconds once the memory
// pipes are busy, so a look-back per 16 KiB tile cannot be hidden.  Here a block owns whole
// segments (dealt round-robin over a grid of one resident wave).  Pass 1 streams a segment from
// HBM and reduces it; the block publishes that aggregate and resolves the segment's prefix with
// ONE block-wide look-back; pass 2 reads the segment again - it is still in the 126 MB L2, the
// live segments of all blocks together stay well below that - scans it with the prefix and streams
// the result out.  The two passes are software-pipelined: while a block scans sub-tile s of its
// current segment it already reduces sub-tile s of its next one, so HBM reads never pause.  HBM
// sees one read and one write per element; descriptors and look-backs: one per segment.
constexpr int kSegThreads = 256;
constexpr int kSegWarps = kSegThreads / 32;
constexpr int kSubTileVecs = kSegThreads * kScanVecs;               // 1024 vectors = 16 KiB
static_assert(kScanVecs * kSegWarps == 32, "warp totals of a sub-tile must fill exactly one warp");

struct SegPlan {
    int64_t  nvec;           // 16-byte vectors in the whole array
    int64_t  seg_vecs;       // vectors per segment (a multiple of the sub-tile)
    int64_t  nsegs;
    int32_t  inclusive, has_init;
    uint32_t max_polls;
    uint64_t init;
    const void* init_dev;
    uint32_t epoch;
    void* value_mem;
};

template <typename T, int OP>
__global__ void __launch_bounds__(kSegThreads, 3)
scan_segment_kernel(const T* A, T* B, SegPlan pl, void* state_mem, int32_t* err_word) {
    using Acc = typename ScanAcc<T>::type;
    constexpr int V = 16 / sizeof(T);
    using VT = Vec<T, V>;
    // per-thread staging of the pass-2 sub-tile: thread t copies and later reads only its own
    // four vectors, so no barrier guards these buffers, only cp.async group waits
    __shared__ __align__(16) uint4 s_stage[2][kSubTileVecs];
    __shared__ Acc s_warp[32];
    __shared__ Acc s_wex[32];
    __shared__ Acc s_prefix, s_total;
    __shared__ int s_wflag[kSegWarps];
    __shared__ int s_verdict, s_abort;

    grid_dependency_wait();
    grid_dependency_release();
    TileState<Acc> state;
    state.bind(state_mem, pl.value_mem, pl.nsegs, pl.epoch);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint4* src = reinterpret_cast<const uint4*>(A);
    uint4* dst = reinterpret_cast<uint4*>(B);
    if (tid == 0) s_abort = 0;
    __syncthreads();
    const uint64_t keep = l2_policy_keep(), stream = l2_policy_stream();

    // Block-wide reduction of the per-thread pass-1 accumulators and publication of the segment's
    // aggregate (segment 0 publishes its inclusive prefix at once).  Returns the aggregate.
    auto publish_aggregate = [&](int64_t seg, Acc* acc) -> Acc {
        Acc r = acc[0];
#pragma unroll
        for (int q = 1; q < V; ++q) r = scan_apply<Acc, OP>(r, acc[q]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) r = scan_apply<Acc, OP>(r, __shfl_down_sync(0xffffffffu, r, o));
        if (lane == 0) s_warp[warp] = r;
        __syncthreads();
        if (warp == 0) {
            Acc t = lane < kSegWarps ? s_warp[lane] : scan_identity<Acc, OP>();
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t = scan_apply<Acc, OP>(t, __shfl_down_sync(0xffffffffu, t, o));
            if (lane == 0) {
                s_total = t;
                if (seg == 0) {
                    Acc prefix = scan_identity<Acc, OP>();
                    if (pl.has_init) prefix = (pl.has_init == 2) ? scan_up<T>(*reinterpret_cast<const T*>(pl.init_dev)) : as_c<Acc, uint64_t>(pl.init);
                    state.publish(0, FLAG_PREFIX, pl.has_init ? scan_apply<Acc, OP>(prefix, t) : t);
                } else {
                    state.publish(seg, FLAG_AGGREGATE, t);
                }
            }
        }
        __syncthreads();
        const Acc aggregate = s_total;
        __syncthreads();          // s_total / s_warp may be rewritten right after
        return aggregate;
    };

    // ONE block-wide look-back for segment `seg` (thread t inspects segment seg-1-t); leaves the
    // exclusive prefix in s_prefix and publishes the inclusive one.  False when a wait ran out.
    auto lookback = [&](int64_t seg, Acc aggregate) -> bool {
        if (seg == 0) {
            if (tid == 0) {
                Acc prefix = scan_identity<Acc, OP>();
                if (pl.has_init) prefix = (pl.has_init == 2) ? scan_up<T>(*reinterpret_cast<const T*>(pl.init_dev)) : as_c<Acc, uint64_t>(pl.init);
                s_prefix = prefix;
            }
            __syncthreads();
            return true;
        }
        int64_t look = seg - 1;
        Acc running = scan_identity<Acc, OP>();
        bool running_set = false;
        while (true) {
            const int64_t mine = look - tid;
            Acc val = scan_identity<Acc, OP>();
            uint32_t flag = FLAG_PREFIX;
            const bool real = mine >= 0;
            bool abort = false;
            if (real) {
                uint32_t polls = 0;
                flag = state.peek(mine, val);
                while (flag == FLAG_EMPTY) {
                    ++polls;
                    if (polls > pl.max_polls) { abort = true; break; }
                    if ((polls & 1023u) == 0 && error_latched(err_word)) { abort = true; break; }
                    __nanosleep(polls > 64 ? 512 : 128);
                    flag = state.peek(mine, val);
                }
            }
            abort = __any_sync(0xffffffffu, abort);
            const uint32_t pmask = __ballot_sync(0xffffffffu, !abort && flag == FLAG_PREFIX);
            const int stop = pmask ? (__ffs(pmask) - 1) : 32;
            Acc contrib = (lane <= stop && real && !abort) ? val : scan_identity<Acc, OP>();
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                Acc up = __shfl_down_sync(0xffffffffu, contrib, o);
                if (lane + o < 32) contrib = scan_apply<Acc, OP>(up, contrib);
            }
            if (lane == 0) {
                s_warp[warp] = contrib;
                s_wflag[warp] = abort ? 2 : (stop < 32 ? 1 : 0);
            }
            __syncthreads();
            if (tid == 0) {
                int verdict = 0;
                for (int w = 0; w < kSegWarps; ++w) {
                    if (s_wflag[w] == 2) { verdict = 2; break; }
                    running = running_set ? scan_apply<Acc, OP>(s_warp[w], running) : s_warp[w];
                    running_set = true;
                    if (s_wflag[w] == 1) { verdict = 1; break; }
                }
                s_verdict = verdict;
                if (verdict == 1) {
                    state.publish(seg, FLAG_PREFIX, scan_apply<Acc, OP>(running, aggregate));
                    s_prefix = running;
                } else if (verdict == 2) {
                    s_abort = 1;
                }
            }
            __syncthreads();
            if (s_verdict != 0) break;
            look -= kSegThreads;
        }
        return s_abort == 0;
    };

    // Pass 1 alone over one segment (prologue only).
    auto reduce_segment = [&](int64_t seg, Acc* acc) {
#pragma unroll
        for (int q = 0; q < V; ++q) acc[q] = scan_identity<Acc, OP>();
        const int64_t v0 = seg * pl.seg_vecs;
        const int64_t v1 = (v0 + pl.seg_vecs < pl.nvec) ? v0 + pl.seg_vecs : pl.nvec;
        // two sub-tiles per step: eight loads in flight per thread (nothing else keeps the memory
        // pipes busy during the prologue)
        constexpr int NL = 2 * kScanVecs;
        for (int64_t base = v0; base < v1; base += 2 * kSubTileVecs) {
            VT v[NL];
            bool on[NL];
#pragma unroll
            for (int j = 0; j < NL; ++j) {
                const int64_t vi = base + j * kSegThreads + tid;
                on[j] = vi < v1;
                if (on[j]) v[j] = __builtin_bit_cast(VT, ld_policy16(src + vi, keep));
            }
#pragma unroll
            for (int j = 0; j < NL; ++j)
                if (on[j]) {
#pragma unroll
                    for (int q = 0; q < V; ++q) acc[q] = scan_apply<Acc, OP>(acc[q], scan_up<T>(v[j].v[q]));
                }
        }
    };

    // ---- prologue: pass 1 of this block's first two segments.  Aggregates are always published
    // one whole segment before their prefix is needed, so look-backs find them waiting.
    const int64_t G = gridDim.x;
    int64_t seg = blockIdx.x;
    if (seg >= pl.nsegs) return;
    Acc acc[V];
    reduce_segment(seg, acc);
    Acc agg_cur = publish_aggregate(seg, acc);
    Acc agg_next = scan_identity<Acc, OP>();
    if (seg + G < pl.nsegs) {
        reduce_segment(seg + G, acc);
        agg_next = publish_aggregate(seg + G, acc);
    }

    while (true) {
        if (!lookback(seg, agg_cur)) break;
        const int64_t ahead = seg + 2 * G;                 // pass 1 runs two segments ahead
        const bool has_ahead = ahead < pl.nsegs;
        const int64_t v0 = seg * pl.seg_vecs;
        const int64_t v1 = (v0 + pl.seg_vecs < pl.nvec) ? v0 + pl.seg_vecs : pl.nvec;
        const int64_t n0 = ahead * pl.seg_vecs;
        const int64_t n1 = has_ahead ? ((n0 + pl.seg_vecs < pl.nvec) ? n0 + pl.seg_vecs : pl.nvec) : n0;
#pragma unroll
        for (int q = 0; q < V; ++q) acc[q] = scan_identity<Acc, OP>();
        Acc carry = s_prefix;
        bool seeded = (seg != 0) || pl.has_init;

        // stage the first pass-2 sub-tile
        auto stage = [&](int buf, int64_t sub) {
#pragma unroll
            for (int j = 0; j < kScanVecs; ++j) {
                const int64_t vi = v0 + sub + j * kSegThreads + tid;
                if (vi < v1) cp_async16_policy(&s_stage[buf][j * kSegThreads + tid], src + vi, stream);
            }
            cp_async_commit();
        };
        stage(0, 0);
        int buf = 0;
        for (int64_t sub = 0; sub < pl.seg_vecs; sub += kSubTileVecs, buf ^= 1) {
            if (v0 + sub >= v1 && n0 + sub >= n1) break;
            // start the copies of the NEXT pass-2 sub-tile (second read of those lines, they come
            // from L2) and the loads of pass 1 two segments ahead (from HBM, L2 is asked to keep them)
            stage(buf ^ 1, sub + kSubTileVecs);
            VT cur[kScanVecs], nxt[kScanVecs];
            bool non[kScanVecs];
#pragma unroll
            for (int j = 0; j < kScanVecs; ++j) {
                const int64_t ni = n0 + sub + j * kSegThreads + tid;
                non[j] = ni < n1;
                if (non[j]) nxt[j] = __builtin_bit_cast(VT, ld_policy16(src + ni, keep));
            }
            cp_async_wait<1>();          // this sub-tile's copies (one younger group may be in flight)
#pragma unroll
            for (int j = 0; j < kScanVecs; ++j) cur[j] = __builtin_bit_cast(VT, s_stage[buf][j * kSegThreads + tid]);
            // ---- pass 2 on the current sub-tile
            Acc x[kScanVecs][V];
            Acc lane_ex[kScanVecs];
#pragma unroll
            for (int j = 0; j < kScanVecs; ++j) {
                const int64_t vi = v0 + sub + j * kSegThreads + tid;
#pragma unroll
                for (int q = 0; q < V; ++q) x[j][q] = (vi < v1) ? scan_up<T>(cur[j].v[q]) : scan_identity<Acc, OP>();
#pragma unroll
                for (int q = 1; q < V; ++q) x[j][q] = scan_apply<Acc, OP>(x[j][q - 1], x[j][q]);
                const Acc inc = warp_scan_inclusive<Acc, OP>(x[j][V - 1], lane);
                Acc ex = __shfl_up_sync(0xffffffffu, inc, 1);
                if (lane == 0) ex = scan_identity<Acc, OP>();
                lane_ex[j] = ex;
                if (lane == 31) s_warp[j * kSegWarps + warp] = inc;
            }
            __syncthreads();
            if (warp == 0) {
                const Acc inc = warp_scan_inclusive<Acc, OP>(s_warp[lane], lane);
                Acc ex = __shfl_up_sync(0xffffffffu, inc, 1);
                if (lane == 0) ex = scan_identity<Acc, OP>();
                s_wex[lane] = ex;
                if (lane == 31) s_total = inc;
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < kScanVecs; ++j) {
                const int64_t vi = v0 + sub + j * kSegThreads + tid;
                Acc o = scan_apply<Acc, OP>(s_wex[j * kSegWarps + warp], lane_ex[j]);
                if (seeded) o = scan_apply<Acc, OP>(carry, o);
                VT out;
                if (pl.inclusive) {
#pragma unroll
                    for (int q = 0; q < V; ++q) out.v[q] = scan_down<T>(scan_apply<Acc, OP>(o, x[j][q]));
                } else {
                    out.v[0] = scan_down<T>(o);
#pragma unroll
                    for (int q = 1; q < V; ++q) out.v[q] = scan_down<T>(scan_apply<Acc, OP>(o, x[j][q - 1]));
                }
                if (vi < v1) st_policy16(dst + vi, __builtin_bit_cast(uint4, out), stream);
            }
            carry = seeded ? scan_apply<Acc, OP>(carry, s_total) : s_total;
            seeded = true;
            // ---- pass 1 on the sub-tile of the segment two ahead
#pragma unroll
            for (int j = 0; j < kScanVecs; ++j)
                if (non[j]) {
#pragma unroll
                    for (int q = 0; q < V; ++q) acc[q] = scan_apply<Acc, OP>(acc[q], scan_up<T>(nxt[j].v[q]));
                }
            __syncthreads();      // s_warp / s_wex / s_total are reused by the next sub-tile
        }
        cp_async_wait<0>();
        Acc agg_ahead = scan_identity<Acc, OP>();
        if (has_ahead) agg_ahead = publish_aggregate(ahead, acc);
        seg += G;
        if (seg >= pl.nsegs) break;
        agg_cur = agg_next;
        agg_next = agg_ahead;
    }
    if (s_abort && tid == 0) latch_error(err_word, B200_LOOKBACK_TIMEOUT);
}

// ---- scan along a strided dimension (K > 1) -----------------------------------------------------------
// cumsum(A; dims=2) and friends: neighbouring memory holds neighbouring COLUMNS, the scan runs
// down the rows with stride K.  A block takes a tile of 32*VEC columns x 128 (64) rows: a warp reads
// row segments of 512 bytes (coalesced), every thread scans its VEC columns down the 16 (8) rows of
// its warp with that many independent loads in flight, the 8 warps are stitched through shared memory, and
// tiles below each other are chained with the same aggregate / inclusive-prefix protocol as the
// 1-D scans - here the published value is a vector (one entry per column of the strip).  Tickets
// hand tiles out row-band by row-band, so the tile above a tile was handed out a whole band
// earlier and its prefix is normally waiting; HBM sees one read and one write per element.
constexpr int kSsWarps = 8;
// rows per warp: 64 values per thread whatever the vector width (16 rows of 4 floats, 8 rows of 8 halves)
__host__ __device__ constexpr int ss_rows(int vec) { return vec >= 8 ? 8 : 16; }

struct StridedScanPlan {
    int64_t K, L, M;
    int64_t S, NT;            // strips across K, tiles along L
    int64_t ntiles;           // M * S * NT
    int32_t inclusive, has_init;
    uint32_t max_polls;
    uint32_t epoch;
    uint64_t init;
    const void* init_dev;
};

template <typename T, int OP, int VEC>
__global__ void __launch_bounds__(256)
scan_strided_kernel(const T* A, T* B, StridedScanPlan pl, unsigned long long* flags, typename ScanAcc<T>::type* agg,
                    typename ScanAcc<T>::type* pre, unsigned int* ticket, int32_t* err_word) {
    grid_dependency_wait();
    using Acc = typename ScanAcc<T>::type;
    using VT = Vec<T, VEC>;
    constexpr int KX = 32 * VEC;                    // columns per strip
    constexpr int kSsRows = ss_rows(VEC), kSsLY = kSsWarps * kSsRows;
    __shared__ Acc s_tot[kSsWarps][KX];
    __shared__ Acc s_pref[KX];
    __shared__ long long s_tile;
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        const unsigned int t = atomicAdd(ticket, 1u);
        if ((int64_t)t == pl.ntiles - 1) *ticket = 0;   // nobody takes a ticket after the last tile
        s_tile = t;
        s_abort = 0;
    }
    __syncthreads();
    // tickets walk strips and slabs fastest, row bands slowest
    const int64_t id = s_tile;
    const int64_t per_band = pl.M * pl.S;
    const int64_t tt = id / per_band;
    const int64_t rem = id - tt * per_band;
    const int64_t m = rem / pl.S, s = rem - m * pl.S;
    const int64_t d = (m * pl.S + s) * pl.NT + tt;      // descriptor index; the tile above is d - 1
    const int64_t k0 = s * KX + lane * VEC;
    const int64_t slab = m * pl.K * pl.L;
    const int64_t l0 = tt * kSsLY + warp * kSsRows;

    // ---- load 8 rows, scan down them
    Acc x[kSsRows][VEC];
#pragma unroll
    for (int r = 0; r < kSsRows; ++r) {
        const int64_t l = l0 + r;
        const bool row_ok = l < pl.L;
        if (VEC > 1) {
            VT v;
            const bool ok = row_ok && k0 < pl.K;
            if (ok) v = *reinterpret_cast<const VT*>(A + slab + k0 + pl.K * l);
#pragma unroll
            for (int q = 0; q < VEC; ++q) x[r][q] = ok ? scan_up<T>(v.v[q]) : scan_identity<Acc, OP>();
        } else {
            x[r][0] = (row_ok && k0 < pl.K) ? scan_up<T>(A[slab + k0 + pl.K * l]) : scan_identity<Acc, OP>();
        }
    }
#pragma unroll
    for (int r = 1; r < kSsRows; ++r)
#pragma unroll
        for (int q = 0; q < VEC; ++q) x[r][q] = scan_apply<Acc, OP>(x[r - 1][q], x[r][q]);
#pragma unroll
    for (int q = 0; q < VEC; ++q) s_tot[warp][lane * VEC + q] = x[kSsRows - 1][q];
    __syncthreads();

    // ---- one thread per column of the strip: aggregate, look-back, prefix
    Acc column_total = scan_identity<Acc, OP>();
    if (tid < KX) {
        column_total = s_tot[0][tid];
#pragma unroll
        for (int w = 1; w < kSsWarps; ++w) column_total = scan_apply<Acc, OP>(column_total, s_tot[w][tid]);
        if (tt == 0) {
            Acc seed = scan_identity<Acc, OP>();
            if (pl.has_init) seed = (pl.has_init == 2) ? scan_up<T>(*reinterpret_cast<const T*>(pl.init_dev)) : as_c<Acc, uint64_t>(pl.init);
            s_pref[tid] = seed;
            *reinterpret_cast<volatile Acc*>(pre + d * KX + tid) = pl.has_init ? scan_apply<Acc, OP>(seed, column_total) : column_total;
        } else {
            *reinterpret_cast<volatile Acc*>(agg + d * KX + tid) = column_total;
        }
        __threadfence();
    }
    __syncthreads();
    if (tid == 0) *reinterpret_cast<volatile unsigned long long*>(flags + d) = tag_word(pl.epoch, (tt == 0) ? FLAG_PREFIX : FLAG_AGGREGATE);
    if (tid < KX && tt > 0) {
        Acc running = scan_identity<Acc, OP>();
        bool set = false, failed = false;
        for (int64_t p = d - 1;; --p) {                 // ends at the strip's first tile at the latest (always a full prefix)
            uint32_t f = tag_state(*reinterpret_cast<volatile unsigned long long*>(flags + p), pl.epoch);
            uint32_t polls = 0;
            while (f == FLAG_EMPTY) {
                ++polls;
                if (polls > pl.max_polls || ((polls & 1023u) == 0 && error_latched(err_word))) { failed = true; break; }
                if (polls > 32) __nanosleep(polls > 4096 ? 256 : 32);
                f = tag_state(*reinterpret_cast<volatile unsigned long long*>(flags + p), pl.epoch);
            }
            if (failed) break;
            __threadfence();
            const Acc v = *reinterpret_cast<volatile Acc*>((f == FLAG_PREFIX ? pre : agg) + p * KX + tid);
            running = set ? scan_apply<Acc, OP>(v, running) : v;
            set = true;
            if (f == FLAG_PREFIX) break;
        }
        if (failed) {
            s_abort = 1;
        } else {
            s_pref[tid] = running;
            *reinterpret_cast<volatile Acc*>(pre + d * KX + tid) = scan_apply<Acc, OP>(running, column_total);
            __threadfence();
        }
    }
    __syncthreads();
    if (s_abort) {
        if (tid == 0) latch_error(err_word, B200_LOOKBACK_TIMEOUT);
        return;
    }
    if (tid == 0 && tt > 0) *reinterpret_cast<volatile unsigned long long*>(flags + d) = tag_word(pl.epoch, FLAG_PREFIX);

    // ---- offsets and stores
    const bool seeded = tt > 0 || pl.has_init;
#pragma unroll
    for (int q = 0; q < VEC; ++q) {
        const int col = lane * VEC + q;
        Acc o = scan_identity<Acc, OP>();
        for (int w = 0; w < warp; ++w) o = scan_apply<Acc, OP>(o, s_tot[w][col]);
        if (seeded) o = scan_apply<Acc, OP>(s_pref[col], o);
        // x[r] becomes the output of row r (exclusive: the value of the row above)
        Acc above = o;
#pragma unroll
        for (int r = 0; r < kSsRows; ++r) {
            const Acc incl = scan_apply<Acc, OP>(o, x[r][q]);
            x[r][q] = pl.inclusive ? incl : above;
            above = incl;
        }
    }
#pragma unroll
    for (int r = 0; r < kSsRows; ++r) {
        const int64_t l = l0 + r;
        if (l >= pl.L || k0 >= pl.K) continue;
        if (VEC > 1) {
            VT v;
#pragma unroll
            for (int q = 0; q < VEC; ++q) v.v[q] = scan_down<T>(x[r][q]);
            *reinterpret_cast<VT*>(B + slab + k0 + pl.K * l) = v;
        } else {
            B[slab + k0 + pl.K * l] = scan_down<T>(x[r][0]);
        }
    }
}

template <typename T, int OP, int VEC>
static int32_t launch_scan_strided(b200_stream_t st, const void* A, void* B, const ScanPlan& pl) {
    using Acc = typename ScanAcc<T>::type;
    constexpr int KX = 32 * VEC;
    constexpr int kSsLY = kSsWarps * ss_rows(VEC);
    StridedScanPlan sp{};
    sp.K = pl.K; sp.L = pl.L; sp.M = pl.M;
    sp.S = (pl.K + KX - 1) / KX;
    sp.NT = (pl.L + kSsLY - 1) / kSsLY;
    sp.ntiles = sp.M * sp.S * sp.NT;
    if (sp.ntiles >= ((int64_t)1 << 31)) return fail(B200_TOO_LARGE, "accumulate: too many tiles");
    sp.inclusive = pl.inclusive;
    sp.has_init = pl.has_init;
    sp.max_polls = pl.max_polls;
    sp.init = pl.init;
    sp.init_dev = pl.init_dev;
    // flag words in the stream's tagged buffer (never cleared), the value vectors in scratch
    const size_t fbytes = (size_t)sp.ntiles * sizeof(unsigned long long);
    const size_t vbytes = (size_t)sp.ntiles * KX * sizeof(Acc);
    void* state = nullptr;
    bool must_clear = false;
    B200_TRY(scan_state(st, fbytes, &state, &sp.epoch, &must_clear));
    unsigned long long* flags = reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(state) + kScanStateHeader);
    if (must_clear) B200_CUDA(cudaMemsetAsync(flags, 0, fbytes, st->s));
    void* scr = nullptr;
    unsigned int* counters = nullptr;
    B200_TRY(scratch(st, 2 * vbytes, &scr, &counters));
    unsigned char* base = reinterpret_cast<unsigned char*>(scr);
    unsigned int* ticket = counters + (kCounterBytes / sizeof(unsigned int) - 1);
    launch_overlapped(scan_strided_kernel<T, OP, VEC>, (unsigned)sp.ntiles, 256, 0, st->s,
                      (const T*)A, (T*)B, sp, flags, reinterpret_cast<Acc*>(base),
                      reinterpret_cast<Acc*>(base + vbytes), ticket, device_error_word(st->dev));
    return B200_OK;
}

// ---- scan along a strided dimension with a few columns (2 <= K <= 4) -----------------------------------
// cumsum(A; dims=2) of a 3 x 1 000 000 matrix and the like: a handful of interleaved columns, each
// very long.  A tile is 256 * RPT consecutive ROWS, i.e. one contiguous piece of memory that holds
// all K columns of those rows; a thread takes RPT rows (whole 16-byte vectors), scans its K columns
// in registers, threads and warps are stitched with shuffles and shared memory, and tiles are
// chained per column with the aggregate / inclusive-prefix protocol of the 1-D scan - warp k
// looks back for column k over a 512-tile window.  Memory is read once and written once, in whole
// lines, where the per-column kernels read every line K times with stride-K accesses.
constexpr int kFcThreads = 256;
constexpr int kFcWarps = kFcThreads / 32;
constexpr int kFcWindow = 16;                        // descriptors per lane and look-back round: 512 tiles
// sixteen rows per thread (eight for 8-byte elements): a million rows are 245 (489) tiles, which one
// look-back round covers - under load every dependent descriptor read costs 2-3 us
__host__ __device__ constexpr int fc_rows_per_thread(size_t elem) { return elem >= 8 ? 8 : 16; }      // (2- and 4-byte elements are dispatched)

template <typename T, int OP, int KC>
__global__ void __launch_bounds__(kFcThreads)
scan_fewcols_kernel(const T* A, T* B, ScanPlan pl, void* flag_mem, unsigned int* ticket, int32_t* err_word) {
    grid_dependency_wait();
    using Acc = typename ScanAcc<T>::type;
    constexpr int RPT = fc_rows_per_thread(sizeof(T));   // rows per thread
    constexpr int E = RPT * KC;                      // elements per thread, element e = row e / KC, column e % KC
    constexpr int ROWS = kFcThreads * RPT;           // rows per tile
    constexpr int VE = 16 / sizeof(T);               // elements per 16-byte vector
    constexpr int NV = E / VE;                       // vectors per thread (RPT is a multiple of VE)
    using VT = Vec<T, VE>;
    static_assert(KC <= kFcWarps, "one warp per column does the look-back");
    __shared__ long long s_tile;
    __shared__ Acc s_wtot[kFcWarps][KC];
    __shared__ Acc s_coltot[KC];
    __shared__ Acc s_prefix[KC];
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        const unsigned int t = atomicAdd(ticket, 1u);
        if ((int64_t)t == pl.ntiles - 1) *ticket = 0;   // nobody takes a ticket after the last tile
        s_tile = t;
        s_abort = 0;
    }
    __syncthreads();
    const int64_t NT = pl.tiles_per_col;
    const int64_t id = s_tile;
    const int64_t tt = id / pl.M, m = id - tt * pl.M;     // all slabs' band tt before band tt + 1
    TileState<Acc> state;
    state.bind(flag_mem, pl.value_mem, pl.M * KC * NT, pl.epoch);
    const int64_t slab = m * pl.K * pl.L;
    const int64_t row0 = tt * ROWS + (int64_t)tid * RPT;
    const bool full = tt * ROWS + ROWS <= pl.L;
    const T* src = A + slab + row0 * KC;
    T* dst = B + slab + row0 * KC;

    Acc x[E];
    if (full && pl.vec_ok) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const VT v = __builtin_bit_cast(VT, __ldcs(reinterpret_cast<const uint4*>(src) + j));
#pragma unroll
            for (int q = 0; q < VE; ++q) x[j * VE + q] = scan_up<T>(v.v[q]);
        }
    } else {
#pragma unroll
        for (int e = 0; e < E; ++e) x[e] = (row0 + e / KC < pl.L) ? scan_up<T>(src[e]) : scan_identity<Acc, OP>();
    }
    // down the thread's rows, per column
#pragma unroll
    for (int e = KC; e < E; ++e) x[e] = scan_apply<Acc, OP>(x[e - KC], x[e]);
    // across the threads of the warp, then the warps
    Acc wex[KC];                                      // exclusive prefix of this thread inside its warp
#pragma unroll
    for (int k = 0; k < KC; ++k) {
        const Acc inc = warp_scan_inclusive<Acc, OP>(x[(RPT - 1) * KC + k], lane);
        Acc ex = __shfl_up_sync(0xffffffffu, inc, 1);
        if (lane == 0) ex = scan_identity<Acc, OP>();
        wex[k] = ex;
        if (lane == 31) s_wtot[warp][k] = inc;
    }
    __syncthreads();
    if (tid < KC) {
        Acc total = s_wtot[0][tid];
#pragma unroll
        for (int w = 1; w < kFcWarps; ++w) total = scan_apply<Acc, OP>(total, s_wtot[w][tid]);
        s_coltot[tid] = total;
        const int64_t d = (m * KC + tid) * NT + tt;
        if (tt == 0) {
            const Acc seed = pl.has_init ? scan_seed<T>(pl) : scan_identity<Acc, OP>();
            s_prefix[tid] = seed;
            state.publish(d, FLAG_PREFIX, pl.has_init ? scan_apply<Acc, OP>(seed, total) : total);
        } else {
            state.publish(d, FLAG_AGGREGATE, total);
        }
    }
    __syncthreads();
    // look-back: warp k resolves column k
    if (warp < KC && tt > 0) {
        const int64_t base = (m * KC + warp) * NT;
        int64_t look = tt - 1;
        Acc running = scan_identity<Acc, OP>();
        bool running_set = false, failed = false;
        bool done = false;
        while (!done && !failed) {
            // A round covers 32 * kFcWindow tiles: slab j holds the tiles look - 32 j - lane, so the
            // nearest 32 tiles - the ones most likely still EMPTY - sit in 32 different lanes and
            // are polled side by side.  All reads of the round go out together.
            uint32_t flag[kFcWindow];
            Acc val[kFcWindow];
#pragma unroll
            for (int j = 0; j < kFcWindow; ++j) {
                const int64_t mine = look - 32 * j - lane;
                val[j] = scan_identity<Acc, OP>();
                flag[j] = mine >= 0 ? state.peek(base + mine, val[j]) : (uint32_t)FLAG_PREFIX;
            }
#pragma unroll
            for (int j = 0; j < kFcWindow; ++j) {
                if (done || failed) continue;
                const int64_t mine = look - 32 * j - lane;
                bool abort = false;
                uint32_t polls = 0;
                while (flag[j] == FLAG_EMPTY) {
                    ++polls;
                    if (polls > pl.max_polls) { abort = true; break; }
                    if ((polls & 1023u) == 0 && error_latched(err_word)) { abort = true; break; }
                    if (polls > 32) __nanosleep(polls > 256 ? 256 : 32);      // the first reads just spin: neighbours publish within a microsecond
                    flag[j] = state.peek(base + mine, val[j]);
                }
                if (__any_sync(0xffffffffu, abort)) { failed = true; continue; }
                const uint32_t pmask = __ballot_sync(0xffffffffu, flag[j] == FLAG_PREFIX);
                const int stop = pmask ? (__ffs(pmask) - 1) : 32;
                Acc contrib = (lane <= stop && mine >= 0) ? val[j] : scan_identity<Acc, OP>();
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const Acc up = __shfl_down_sync(0xffffffffu, contrib, o);
                    if (lane + o < 32) contrib = scan_apply<Acc, OP>(up, contrib);
                }
                running = running_set ? scan_apply<Acc, OP>(contrib, running) : contrib;     // valid in lane 0
                running_set = true;
                if (stop < 32) done = true;
            }
            look -= 32 * kFcWindow;
        }
        if (lane == 0) {
            if (failed) {
                s_abort = 1;
            } else {
                s_prefix[warp] = running;
                state.publish(base + tt, FLAG_PREFIX, scan_apply<Acc, OP>(running, s_coltot[warp]));
            }
        }
    }
    __syncthreads();
    if (s_abort) {
        if (tid == 0) latch_error(err_word, B200_LOOKBACK_TIMEOUT);
        return;
    }
    // offsets, outputs, stores
    const bool seeded = tt > 0 || pl.has_init;
    Acc off[KC];
#pragma unroll
    for (int k = 0; k < KC; ++k) {
        Acc before = scan_identity<Acc, OP>();
        for (int w = 0; w < warp; ++w) before = scan_apply<Acc, OP>(before, s_wtot[w][k]);
        Acc o = scan_apply<Acc, OP>(before, wex[k]);
        if (seeded) o = scan_apply<Acc, OP>(s_prefix[k], o);
        off[k] = o;
    }
    T out[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
        if (pl.inclusive) out[e] = scan_down<T>(scan_apply<Acc, OP>(off[e % KC], x[e]));
        else out[e] = scan_down<T>(e < KC ? off[e % KC] : scan_apply<Acc, OP>(off[e % KC], x[e - KC]));
    }
    if (full && pl.vec_ok) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            VT v;
#pragma unroll
            for (int q = 0; q < VE; ++q) v.v[q] = out[j * VE + q];
            __stcs(reinterpret_cast<uint4*>(dst) + j, __builtin_bit_cast(uint4, v));
        }
    } else {
#pragma unroll
        for (int e = 0; e < E; ++e) if (row0 + e / KC < pl.L) dst[e] = out[e];
    }
}

template <typename T, int OP, int KC>
static int32_t launch_scan_fewcols(b200_stream_t st, const void* A, void* B, ScanPlan pl, bool aligned) {
    using Acc = typename ScanAcc<T>::type;
    constexpr int ROWS = kFcThreads * fc_rows_per_thread(sizeof(T));
    pl.tiles_per_col = (pl.L + ROWS - 1) / ROWS;
    pl.ntiles = pl.tiles_per_col * pl.M;
    if (pl.ntiles * KC >= (int64_t)1 << 31) return fail(B200_TOO_LARGE, "accumulate: too many tiles");
    // every tile start is 16-byte aligned when the slabs are
    pl.vec_ok = (aligned && (pl.M == 1 || (pl.K * pl.L * (int64_t)sizeof(T)) % 16 == 0)) ? 1 : 0;
    void* flags = nullptr;
    B200_TRY(descriptor_storage<Acc>(st, pl.ntiles * KC, &flags, &pl.value_mem, &pl.epoch));
    void* unused = nullptr;
    unsigned int* counters = nullptr;
    B200_TRY(scratch(st, 0, &unused, &counters));
    unsigned int* ticket = counters + (kCounterBytes / sizeof(unsigned int) - 1);
    launch_overlapped(scan_fewcols_kernel<T, OP, KC>, (unsigned)pl.ntiles, kFcThreads, 0, st->s, (const T*)A, (T*)B, pl, flags, ticket,
                      device_error_word(st->dev));
    return B200_OK;
}

// One thread per column: sequential walk, coalesced across neighbouring columns when K > 1.
template <typename T, int OP>
__global__ void __launch_bounds__(256)
scan_column_thread_kernel(const T* A, T* B, ScanPlan pl) {
    grid_dependency_wait();
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

// One warp per contiguous column (K == 1): cumsum(A; dims=1) of a 512 x 1000 matrix and the like -
// many columns, each a few dozen to two thousand elements.  A lane takes a 16-byte vector per
// step (scalar elements when the columns are not 16-byte aligned), the warp scans the vector totals
// with shuffles and carries the running value down the column; the loads of four steps are in
// flight together.  No descriptors, no tickets, no waiting on other blocks: the tiled kernels
// spend a whole 256-thread tile and a look-back on such a column.
template <typename T, int OP, bool VEC>
__global__ void __launch_bounds__(256)
scan_column_warp_kernel(const T* A, T* B, ScanPlan pl) {
    grid_dependency_wait();
    using Acc = typename ScanAcc<T>::type;
    constexpr int V = VEC ? 16 / (int)sizeof(T) : 1;
    constexpr int U = 4;
    using VT = Vec<T, V>;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const int64_t steps = (pl.L + 32 * V - 1) / (32 * V);
    for (int64_t col = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); col < pl.M; col += nwarps) {
        const T* src = A + col * pl.L;
        T* dst = B + col * pl.L;
        Acc carry = pl.has_init ? scan_seed<T>(pl) : scan_identity<Acc, OP>();
        bool seeded = pl.has_init != 0;
        for (int64_t s0 = 0; s0 < steps; s0 += U) {
            Acc x[U][V];
            bool on[U][V];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t e0 = ((s0 + u) * 32 + lane) * V;
                bool whole = false;
                if constexpr (VEC) {
                    whole = e0 + V <= pl.L;
                    if (whole) {
                        const VT v = __builtin_bit_cast(VT, __ldcs(reinterpret_cast<const uint4*>(src + e0)));
#pragma unroll
                        for (int q = 0; q < V; ++q) { x[u][q] = scan_up<T>(v.v[q]); on[u][q] = true; }
                    }
                }
                if (!whole) {
#pragma unroll
                    for (int q = 0; q < V; ++q) {
                        on[u][q] = e0 + q < pl.L;
                        x[u][q] = on[u][q] ? scan_up<T>(src[e0 + q]) : scan_identity<Acc, OP>();
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (s0 + u >= steps) continue;                   // uniform over the warp
#pragma unroll
                for (int q = 1; q < V; ++q) x[u][q] = scan_apply<Acc, OP>(x[u][q - 1], x[u][q]);
                const Acc inc = warp_scan_inclusive<Acc, OP>(x[u][V - 1], lane);
                Acc before = __shfl_up_sync(0xffffffffu, inc, 1);           // total of the lanes in front
                const Acc total = __shfl_sync(0xffffffffu, inc, 31);
                Acc off = carry;
                bool off_set = seeded;
                if (lane > 0) { off = off_set ? scan_apply<Acc, OP>(carry, before) : before; off_set = true; }
                const int64_t e0 = ((s0 + u) * 32 + lane) * V;
                T outv[V];
#pragma unroll
                for (int q = 0; q < V; ++q) {
                    const Acc incl = off_set ? scan_apply<Acc, OP>(off, x[u][q]) : x[u][q];
                    const Acc excl = q == 0 ? (off_set ? off : scan_identity<Acc, OP>())
                                            : (off_set ? scan_apply<Acc, OP>(off, x[u][q - 1]) : x[u][q - 1]);
                    outv[q] = scan_down<T>(pl.inclusive ? incl : excl);
                }
                bool whole = false;
                if constexpr (VEC) {
                    whole = e0 + V <= pl.L;
                    if (whole) {
                        VT v;
#pragma unroll
                        for (int q = 0; q < V; ++q) v.v[q] = outv[q];
                        __stcs(reinterpret_cast<uint4*>(dst + e0), __builtin_bit_cast(uint4, v));
                    }
                }
                if (!whole) {
#pragma unroll
                    for (int q = 0; q < V; ++q) if (on[u][q]) dst[e0 + q] = outv[q];
                }
                carry = seeded ? scan_apply<Acc, OP>(carry, total) : total;
                seeded = true;
            }
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
    const bool aligned = reinterpret_cast<uintptr_t>(A) % 16 == 0 && reinterpret_cast<uintptr_t>(B) % 16 == 0;
    if (pl.K >= 32 && pl.L > 32) {      // long scans down a strided dimension: tiled, chained along L
        constexpr int V = 16 / sizeof(T);
        if (aligned && (pl.K * sizeof(T)) % 16 == 0) return launch_scan_strided<T, OP, V>(st, A, B, pl);
        return launch_scan_strided<T, OP, 1>(st, A, B, pl);
    }
    // a few long interleaved columns: one tile holds all of them (8-byte elements measured no
    // faster than the per-column tiles: their tiles are half as long, the chain twice as long)
    if constexpr (sizeof(T) <= 4) if (pl.K >= 2 && pl.K <= 4 && pl.L >= 4096) {
        switch (pl.K) {
            case 2: return launch_scan_fewcols<T, OP, 2>(st, A, B, pl, aligned);
            case 3: return launch_scan_fewcols<T, OP, 3>(st, A, B, pl, aligned);
            default: return launch_scan_fewcols<T, OP, 4>(st, A, B, pl, aligned);
        }
    }
    const bool thread_cols = (pl.L <= 32 && ncols >= 1024) || (pl.K > 1 && ncols >= 4096);
    if (thread_cols) {
        int64_t blocks = (ncols + 255) / 256;
        if (blocks > target) blocks = target;
        scan_column_thread_kernel<T, OP><<<(unsigned)blocks, 256, 0, st->s>>>((const T*)A, (T*)B, pl);
        return B200_OK;
    }
    // many contiguous columns of up to half a tile (8 KiB): a warp per column.  Longer columns fill
    // the tiles of the look-back kernel well enough (8192 x 8192 Float32: 0.103 ms there, 0.121 ms here)
    if (pl.K == 1 && pl.M >= 64 && pl.L > 32 && pl.L * (int64_t)sizeof(T) <= 8192) {
        int64_t blocks = (pl.M + 7) / 8;
        if (blocks > target) blocks = target;
        if (aligned && (pl.L * sizeof(T)) % 16 == 0)
            launch_overlapped(scan_column_warp_kernel<T, OP, true>, (unsigned)blocks, 256, 0, st->s, (const T*)A, (T*)B, pl);
        else
            launch_overlapped(scan_column_warp_kernel<T, OP, false>, (unsigned)blocks, 256, 0, st->s, (const T*)A, (T*)B, pl);
        return B200_OK;
    }
    if (ncols == 1 && aligned && (pl.L * sizeof(T)) % 16 == 0 && pl.L * (int64_t)sizeof(T) >= (int64_t)(1 << 20)) {
        SegPlan sp{};
        sp.nvec = pl.L * (int64_t)sizeof(T) / 16;
        int64_t grid = resident_blocks(scan_segment_kernel<T, OP>, kSegThreads, 0, st->dev);
        // segments are whole sub-tiles of 16 KiB: 48 KiB measured best for long vectors (look-backs
        // are rare enough and the live segments of all blocks stay far below the L2 capacity)
        const int64_t subv = kSubTileVecs;
        const int64_t nsub = (sp.nvec + subv - 1) / subv;
        int64_t per = nsub / (grid * 3);     // short vectors: smaller segments, so that every block has work
        if (per < 1) per = 1;
        if (per > 3) per = 3;     // two segments per block are live in L2: 2 x 48 KiB x 444 blocks = 43 MB
        sp.seg_vecs = per * subv;
        sp.nsegs = (sp.nvec + sp.seg_vecs - 1) / sp.seg_vecs;
        sp.inclusive = pl.inclusive;
        sp.has_init = pl.has_init;
        sp.max_polls = pl.max_polls;
        sp.init = pl.init;
        sp.init_dev = pl.init_dev;
        void* scr = nullptr;
        B200_TRY(descriptor_storage<Acc>(st, sp.nsegs, &scr, &sp.value_mem, &sp.epoch));
        if (grid > sp.nsegs) grid = sp.nsegs;
        launch_overlapped(scan_segment_kernel<T, OP>, (unsigned)grid, kSegThreads, 0, st->s,
                          (const T*)A, (T*)B, sp, scr, device_error_word(st->dev));
        return B200_OK;
    }
    pl.tiles_per_col = (pl.L + TILE - 1) / TILE;
    pl.ntiles = pl.tiles_per_col * ncols;
    if (pl.ntiles >= (int64_t)1 << 31) return fail(B200_TOO_LARGE, "accumulate: too many tiles");
    pl.vec_ok = (pl.K == 1 && aligned && (ncols == 1 || (pl.L * sizeof(T)) % 16 == 0)) ? 1 : 0;
    void* scr = nullptr;
    unsigned int* counters = nullptr;
    B200_TRY(descriptor_storage<Acc>(st, pl.ntiles, &scr, &pl.value_mem, &pl.epoch));
    void* unused = nullptr;
    B200_TRY(scratch(st, 0, &unused, &counters));
    // the last counter slot serves as the tile ticket (it returns to zero by itself)
    unsigned int* ticket = counters + (kCounterBytes / sizeof(unsigned int) - 1);
    launch_overlapped(scan_lookback_kernel<T, OP>, (unsigned)pl.ntiles, kScanThreads, 0, st->s,
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
    const size_t flag_bytes = TileState<Acc>::flag_bytes(pl.ntiles);
    const int64_t max_tiles = (int64_t)((kStaticScanBytes - kStaticScanHeader) / (TileState<Acc>::flag_bytes(1) + TileState<Acc>::value_bytes(1)));
    if (pl.ntiles > max_tiles)
        return fail(B200_TOO_LARGE, "accumulate (no-allocation variant): %lld tiles of %d elements needed, the built-in "
                    "scratch holds %lld for this element type; use b200_accumulate for larger inputs",
                    (long long)pl.ntiles, TILE, (long long)max_tiles);
    void* base = nullptr;
    B200_TRY(static_scan_scratch(st->dev, &base));
    const bool aligned = reinterpret_cast<uintptr_t>(A) % 16 == 0 && reinterpret_cast<uintptr_t>(B) % 16 == 0;
    pl.vec_ok = (pl.K == 1 && aligned && (ncols == 1 || (pl.L * sizeof(T)) % 16 == 0)) ? 1 : 0;
    // the array keeps whatever the previous call left: ticket and descriptor words must start at
    // zero (launch number 0 = "the words were cleared"); the values behind them need no clearing
    B200_CUDA(cudaMemsetAsync(base, 0, kStaticScanHeader + flag_bytes, st->s));
    pl.epoch = 0;
    pl.value_mem = reinterpret_cast<unsigned char*>(base) + kStaticScanHeader + flag_bytes;
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

// Validation and plan shared by every accumulate entry point: checks the descriptors, collapses
// the shape to (K, L, M) around the scanned dimension and folds the seed into the plan.  `*empty`
// is set for arrays without elements (nothing to launch).
static int32_t scan_plan(const b200_tensor* B, const b200_tensor* A, int32_t op, const void* init, const void* init_dev,
                         int32_t dim, int32_t inclusive, ScanPlan* out, bool* empty) {
    B200_TRY(check_tensor(B, "accumulate destination"));
    B200_TRY(check_tensor(A, "accumulate source"));
    if (op < 0 || op >= B200_RED_COUNT) return fail(B200_UNSUPPORTED, "accumulate: unknown operator %d", op);
    if (A->dtype != B->dtype) return fail(B200_UNSUPPORTED, "accumulate: source and destination element types differ");
    if (A->ndim != B->ndim) return fail(B200_INVALID_ARG, "accumulate: source and destination shapes differ");
    for (int d = 0; d < A->ndim; ++d)
        if (A->shape[d] != B->shape[d]) return fail(B200_INVALID_ARG, "accumulate: source and destination shapes differ");
    if (!tensor_is_contiguous(A) || !tensor_is_contiguous(B))
        return fail(B200_UNSUPPORTED, "accumulate: operands must be dense column-major arrays");
    *empty = tensor_numel(A) == 0;
    if (*empty) return B200_OK;
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
    *out = pl;
    return B200_OK;
}

#define B200_SCAN_DTYPE_SWITCH(LAUNCH)                                                                  \
    switch (A->dtype) {                                                                                 \
        case B200_F32: s = LAUNCH<float>(st, A->ptr, B->ptr, pl, op); break;                            \
        case B200_F64: s = LAUNCH<double>(st, A->ptr, B->ptr, pl, op); break;                           \
        case B200_I32: s = LAUNCH<int32_t>(st, A->ptr, B->ptr, pl, op); break;                          \
        case B200_I64: s = LAUNCH<int64_t>(st, A->ptr, B->ptr, pl, op); break;                          \
        case B200_U32: s = LAUNCH<uint32_t>(st, A->ptr, B->ptr, pl, op); break;                         \
        case B200_U64: s = LAUNCH<uint64_t>(st, A->ptr, B->ptr, pl, op); break;                         \
        case B200_F16: s = LAUNCH<__half>(st, A->ptr, B->ptr, pl, op); break;                           \
        case B200_BF16: s = LAUNCH<__nv_bfloat16>(st, A->ptr, B->ptr, pl, op); break;                   \
        default: return fail(B200_UNSUPPORTED, "accumulate: element type %d is not supported", A->dtype); \
    }

static int32_t accumulate_common(b200_stream_t st, const b200_tensor* B, const b200_tensor* A, int32_t op,
                                 const void* init, const void* init_dev, int32_t dim, int32_t inclusive) {
    B200_TRY(enter(st));
    StreamGuard guard(st);
    ScanPlan pl{};
    bool empty = false;
    B200_TRY(scan_plan(B, A, op, init, init_dev, dim, inclusive, &pl, &empty));
    if (empty) return B200_OK;
    int32_t s;
    B200_SCAN_DTYPE_SWITCH(launch_scan_op)
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
    StreamGuard guard(st);
    ScanPlan pl{};
    bool empty = false;
    B200_TRY(scan_plan(B, A, op, init, nullptr, dim, inclusive, &pl, &empty));
    if (empty) return B200_OK;
    int32_t s;
    B200_SCAN_DTYPE_SWITCH(launch_scan_static_op)
    B200_TRY(s);
    return finish(st, "b200_accumulate_noalloc");
}

// Self-test of the bounded wait: runs ONE tile of the chained scan whose ticket says it is tile 1
// while tile 0 never exists, with a poll budget of `polls`.  The block gives up after that many
// polls, latches B200_LOOKBACK_TIMEOUT and returns; the next b200_stream_sync reports it and the
// context stays usable.  Nothing faults and nothing spins without a limit.
extern "C" int32_t b200_selftest_wait_timeout(b200_stream_t st, uint32_t polls) {
    B200_TRY(enter(st));
    StreamGuard guard(st);
    if (polls == 0 || polls > (1u << 20)) return fail(B200_INVALID_ARG, "poll budget must be in 1..2^20");
    constexpr int TILE = kScanThreads * kScanVecs * 4;
    void* scr = nullptr;
    unsigned int* counters = nullptr;
    const size_t data_bytes = 2 * (size_t)TILE * sizeof(int32_t);
    const size_t sbytes = 256 + TileState<int32_t>::flag_bytes(2) + 2 * data_bytes;   // cleared below: launch number 0
    B200_TRY(scratch(st, sbytes, &scr, &counters));
    B200_CUDA(cudaMemsetAsync(scr, 0, sbytes, st->s));
    unsigned char* base = reinterpret_cast<unsigned char*>(scr);
    unsigned int* ticket = reinterpret_cast<unsigned int*>(base);
    const unsigned int one = 1;
    B200_CUDA(cudaMemcpyAsync(ticket, &one, sizeof one, cudaMemcpyHostToDevice, st->s));   // first ticket handed out is 1
    int32_t* in = reinterpret_cast<int32_t*>(base + 256 + 256);
    int32_t* out = in + 2 * TILE;
    ScanPlan pl{};
    pl.K = 1; pl.L = 2 * TILE; pl.M = 1;
    pl.tiles_per_col = 2; pl.ntiles = 2;
    pl.vec_ok = 1; pl.inclusive = 1; pl.has_init = 0;
    pl.max_polls = polls;
    scan_lookback_kernel<int32_t, B200_RED_ADD><<<1, kScanThreads, 0, st->s>>>(in, out, pl, base + 256, ticket, device_error_word(st->dev));
    B200_CUDA(cudaMemsetAsync(ticket, 0, sizeof(unsigned int), st->s));
    return finish(st, "b200_selftest_wait_timeout");
}
