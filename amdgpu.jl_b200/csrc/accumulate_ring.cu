// One-pass scan of a long dense vector: every element crosses HBM once in and once out.
//
// Takes the place of AK.accumulate! as called from src/kernels/accumulate.jl:1-8 of the reference
// for the long 1-D case.  One block per SM, specialised warps around a ring of shared-memory
// stages:
//   * the producer (one thread) takes tile numbers from an atomic ticket and fills free stages
//     with bulk asynchronous copies (cp.async.bulk + mbarrier transaction counts), a bounded
//     number of tiles in flight;
//   * 16 consumer warps run two phases per tile, `lead` tiles apart: phase A reduces a tile that
//     has just landed (per-warp totals stay in shared memory) and publishes the tile's aggregate;
//     phase C scans the tile out of shared memory with its prefix and streams the result to HBM;
//   * four prefix warps, one tile each in rotation, compute the prefixes.  A block knows the
//     inclusive prefix of its own previous tile, so the prefix of its next tile only needs the
//     AGGREGATES of the tiles in between (about one per other block), never another block's
//     resolved prefix: there is no chain of dependent waits across blocks.  A prefix warp starts
//     reading those aggregates as soon as the producer holds the ticket, while the tile's own
//     data is still on its way.
// Descriptors are 64-bit words {launch number:32 | aggregate:32}; words of earlier launches read
// as empty, nothing is cleared between launches.  Every wait (mbarrier or descriptor) is bounded;
// a wait that runs out latches B200_LOOKBACK_TIMEOUT, all roles leave, and the block drains its
// copies before it returns.
#include "scan_common.cuh"

#include <cstdlib>

namespace b200 {

constexpr int kRingConsumerWarps = 16;
constexpr int kRingConsumers = kRingConsumerWarps * 32;
constexpr int kRingPrefixWarps = 4;
constexpr int kRingThreads = kRingConsumers + 32 + 32 * kRingPrefixWarps;   // + producer warp + prefix warps
constexpr int kRingBytes = 192 * 1024;                   // shared memory given to the stages
constexpr int kRingWindows = 8;                          // aggregates are gathered 8 x 32 at a time

struct RingPlan {
    int64_t  nvec;            // 16-byte vectors in the array
    int64_t  ntiles;
    int32_t  inclusive, has_init;
    uint32_t max_polls;
    uint32_t epoch;
    int32_t  lead;            // tiles between phase A and phase C
    int32_t  inflight;        // tiles the producer keeps in flight
    uint64_t init;
    const void* init_dev;
};

// ---- PTX helpers ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the budget ran out or another role has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile int* abort_flag, uint32_t budget) {
    uint32_t tries = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (++tries > budget || *abort_flag) return false;
    }
    return true;
}
// Bulk copy global -> this block's shared memory, completion counted on `bar` (no multicast).
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}
__device__ __forceinline__ unsigned long long desc_load(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void desc_store(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Barrier over the consumer threads only, OR-reducing a flag (named barrier 1).
__device__ __forceinline__ bool consumers_any(bool flag) {
    uint32_t out;
    asm volatile("{\n .reg .pred p, q;\n setp.ne.u32 p, %1, 0;\n barrier.cta.red.or.pred q, 1, %2, p;\n selp.u32 %0, 1, 0, q;\n}"
                 : "=r"(out) : "r"((uint32_t)flag), "n"(kRingConsumers) : "memory");
    return out != 0;
}

template <typename Acc>
__device__ __forceinline__ uint32_t acc_bits(Acc v) {
    static_assert(sizeof(Acc) == 4, "the ring scan carries 4-byte accumulators");
    return __builtin_bit_cast(uint32_t, v);
}
template <typename Acc>
__device__ __forceinline__ Acc acc_from(uint32_t b) { return __builtin_bit_cast(Acc, b); }

template <typename Acc, int NV>
struct RingShared {
    static constexpr int kTileBytes = kRingConsumers * NV * 16;
    static constexpr int kStages = kRingBytes / kTileBytes;
    static constexpr int kTotals = NV * kRingConsumerWarps;
    alignas(128) unsigned char stage[kStages][kTileBytes];
    uint64_t  full[kStages], empty[kStages], aggready[kStages], resolved[kStages], ticketed[kStages];
    long long tile_of[kStages];
    long long tiles[2 * kStages];          // tile numbers of the last 2 x stages local tiles (prefix warps)
    long long last_local;                  // local index at which the producer ran out of tiles (-1: not yet)
    Acc       agg[kStages], prefix[kStages];
    Acc       wtot[kStages][kTotals];      // inclusive totals of (vector row j, warp w), phase A
    Acc       wex[kStages][kTotals];       // their exclusive scan in element order
    int       abort;
};

// Fold of the aggregates of tiles lo .. hi-1 in tile order (identity for an empty range).  Whole
// warp; the result is valid in every lane.  Waits (bounded) for aggregates that are not out yet.
template <typename Acc, int OP>
__device__ __forceinline__ bool ring_gather(const unsigned long long* desc, int64_t lo, int64_t hi, uint32_t epoch,
                                            uint32_t max_polls, const int32_t* err_word, const volatile int* abort_flag,
                                            int lane, Acc* out) {
    Acc running = scan_identity<Acc, OP>();
    uint32_t polls = 0;
    for (int64_t base = hi - 1; base >= lo; base -= 32 * kRingWindows) {
        unsigned long long w[kRingWindows];
#pragma unroll
        for (int k = 0; k < kRingWindows; ++k) {
            const int64_t idx = base - 32 * k - lane;
            w[k] = idx >= lo ? desc_load(desc + idx) : 0ull;
        }
#pragma unroll
        for (int k = 0; k < kRingWindows; ++k) {
            if (base - 32 * k < lo) break;               // uniform: this window lies before the range
            const int64_t idx = base - 32 * k - lane;
            unsigned long long cur = w[k];
            while (true) {
                const bool missing = idx >= lo && (uint32_t)(cur >> 32) != epoch;
                if (!__any_sync(0xffffffffu, missing)) break;
                if (++polls > max_polls) return false;
                if ((polls & 255u) == 0 && (error_latched(err_word) || *abort_flag)) return false;
                __nanosleep(40);
                if (missing) cur = desc_load(desc + idx);
            }
            Acc contrib = idx >= lo ? acc_from<Acc>((uint32_t)cur) : scan_identity<Acc, OP>();
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {             // lane 0 ends with farthest (+) ... (+) nearest
                const Acc far = __shfl_down_sync(0xffffffffu, contrib, o);
                if (lane + o < 32) contrib = scan_apply<Acc, OP>(far, contrib);
            }
            running = scan_apply<Acc, OP>(__shfl_sync(0xffffffffu, contrib, 0), running);
        }
    }
    *out = running;
    return true;
}

template <typename T, int OP, int NV>
__global__ void __launch_bounds__(kRingThreads, 1)
scan_ring_kernel(const T* A, T* B, RingPlan pl, unsigned long long* desc, unsigned int* tickets, int32_t* err_word) {
    using Acc = typename ScanAcc<T>::type;
    using SM = RingShared<Acc, NV>;
    constexpr int V = 16 / sizeof(T);
    constexpr int S = SM::kStages;
    constexpr int TILE_VECS = kRingConsumers * NV;
    constexpr int PER = SM::kTotals / 32;        // warp totals per lane in the scan of the totals
    static_assert(SM::kTotals % 32 == 0, "totals must fill whole warps");
    using VT = Vec<T, V>;
    extern __shared__ __align__(128) unsigned char ring_smem[];
    SM& sm = *reinterpret_cast<SM*>(ring_smem);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // two ticket words take turns: a launch counts on the word of its parity and clears the other
    // one for the launch that follows, so a launch that was cut short leaves no stale count behind
    unsigned int* ticket = tickets + (pl.epoch & 1u);
    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], kRingConsumerWarps);
            mbar_init(&sm.aggready[s], 1);
            mbar_init(&sm.resolved[s], 1);
            mbar_init(&sm.ticketed[s], 1);
        }
        sm.abort = 0;
        sm.last_local = -1;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (blockIdx.x == 0) tickets[(pl.epoch + 1u) & 1u] = 0;
    }
    __syncthreads();
    volatile int* abort_flag = &sm.abort;
    const uint32_t budget = pl.max_polls;
    auto give_up = [&]() {
        *abort_flag = 1;
        latch_error(err_word, B200_LOOKBACK_TIMEOUT);
    };
    auto tile_vecs = [&](int64_t t) -> int {
        const int64_t left = pl.nvec - t * TILE_VECS;
        return left < TILE_VECS ? (int)left : TILE_VECS;
    };

    int64_t issued = 0;                          // producer: tiles whose copy was started
    if (warp == kRingConsumerWarps) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            const uint64_t stream = l2_policy_stream();
            const int inflight = pl.inflight < 1 ? 1 : (pl.inflight > S ? S : pl.inflight);
            unsigned int t = atomicAdd(ticket, 1u);
            for (int64_t i = 0;; ++i) {
                const int s = (int)(i % S);
                if (i >= S && !mbar_wait(&sm.empty[s], (uint32_t)((i / S) - 1) & 1u, abort_flag, budget)) { give_up(); break; }
                if (i >= inflight) {             // bound the copies in flight
                    const int64_t j = i - inflight;
                    if (!mbar_wait(&sm.full[j % S], (uint32_t)(j / S) & 1u, abort_flag, budget)) { give_up(); break; }
                }
                if ((int64_t)t >= pl.ntiles) {   // no tile left: tell the other roles
                    sm.tile_of[s] = -1;
                    sm.tiles[i % (2 * S)] = -1;
                    *(volatile long long*)&sm.last_local = i;
                    mbar_arrive(&sm.ticketed[s]);
                    mbar_arrive(&sm.full[s]);
                    break;
                }
                sm.tile_of[s] = (long long)t;
                sm.tiles[i % (2 * S)] = (long long)t;
                mbar_arrive(&sm.ticketed[s]);    // the prefix warp of this tile may start gathering
                const uint32_t bytes = (uint32_t)tile_vecs(t) * 16u;
                mbar_arrive_expect_tx(&sm.full[s], bytes);
                bulk_load(sm.stage[s], reinterpret_cast<const unsigned char*>(A) + (int64_t)t * TILE_VECS * 16, bytes, &sm.full[s], stream);
                issued = i + 1;
                t = atomicAdd(ticket, 1u);       // the next ticket travels while this thread waits for a stage
            }
        }
    } else if (warp > kRingConsumerWarps) {
        // ---------------------------------------------------------------- prefix warps
        // local tile i belongs to prefix warp i mod 4; its exclusive prefix is
        //   (inclusive prefix of local tile i-1)  (+)  aggregates of the tiles between the two
        for (int64_t i = warp - kRingConsumerWarps - 1;; i += kRingPrefixWarps) {
            const int s = (int)(i % S);
            const uint32_t par = (uint32_t)(i / S) & 1u;
            // the producer stops at some local index; prefix warps whose next tile lies beyond it leave
            bool ticket = false, over = false;
            for (uint32_t tries = 0; !(ticket = mbar_try_wait(&sm.ticketed[s], par)); ++tries) {
                const long long last = *(volatile long long*)&sm.last_local;
                if (last >= 0 && i > last) { over = true; break; }
                if (tries > budget || *abort_flag) break;
            }
            if (over) break;
            if (!ticket) { if (lane == 0) give_up(); break; }
            const int64_t t = sm.tiles[i % (2 * S)];
            if (t < 0) break;
            const int64_t t_prev = i > 0 ? sm.tiles[(i - 1) % (2 * S)] : -1;
            Acc between;
            if (!ring_gather<Acc, OP>(desc, t_prev + 1, t, pl.epoch, pl.max_polls, err_word, abort_flag, lane, &between)) {
                if (lane == 0) give_up();
                break;
            }
            Acc base = scan_identity<Acc, OP>();
            if (i == 0) {
                if (pl.has_init) base = (pl.has_init == 2) ? scan_up<T>(*reinterpret_cast<const T*>(pl.init_dev)) : as_c<Acc, uint64_t>(pl.init);
            } else {
                const int sp = (int)((i - 1) % S);
                const uint32_t pp = (uint32_t)((i - 1) / S) & 1u;
                if (!mbar_wait(&sm.resolved[sp], pp, abort_flag, budget) || !mbar_wait(&sm.aggready[sp], pp, abort_flag, budget)) {
                    if (lane == 0) give_up();
                    break;
                }
                base = scan_apply<Acc, OP>(sm.prefix[sp], sm.agg[sp]);
            }
            if (lane == 0) {
                sm.prefix[s] = scan_apply<Acc, OP>(base, between);
                mbar_arrive(&sm.resolved[s]);
            }
            __syncwarp();
        }
    } else {
        // ---------------------------------------------------------------- consumers
        const uint64_t stream = l2_policy_stream();
        // phase A of local tile i: 1 = a tile was reduced, 0 = no tile left, -1 = give up
        auto phase_a = [&](int64_t i) -> int {
            const int s = (int)(i % S);
            const uint32_t par = (uint32_t)(i / S) & 1u;
            const bool ok = mbar_wait(&sm.full[s], par, abort_flag, budget);
            int64_t t = -1;
            if (ok) {
                t = sm.tile_of[s];
                if (t >= 0) {
                    const int nv = tile_vecs(t);
#pragma unroll
                    for (int j = 0; j < NV; ++j) {
                        const int v = j * kRingConsumers + tid;
                        Acc tot = scan_identity<Acc, OP>();
                        if (v < nv) {
                            const VT x = __builtin_bit_cast(VT, *reinterpret_cast<const uint4*>(sm.stage[s] + (size_t)v * 16));
                            tot = scan_up<T>(x.v[0]);
#pragma unroll
                            for (int q = 1; q < V; ++q) tot = scan_apply<Acc, OP>(tot, scan_up<T>(x.v[q]));
                        }
                        const Acc inc = warp_scan_inclusive<Acc, OP>(tot, lane);
                        if (lane == 31) sm.wtot[s][j * kRingConsumerWarps + warp] = inc;
                    }
                }
            }
            if (consumers_any(!ok)) {
                if (!ok && lane == 0) give_up();
                return -1;
            }
            if (t < 0) return 0;
            if (warp == 0) {
                // exclusive scan of the warp totals in element order (row j, then warp w)
                Acc a[PER];
                Acc pair = scan_identity<Acc, OP>();
#pragma unroll
                for (int p = 0; p < PER; ++p) {
                    a[p] = sm.wtot[s][lane * PER + p];
                    pair = p == 0 ? a[0] : scan_apply<Acc, OP>(pair, a[p]);
                }
                const Acc inc = warp_scan_inclusive<Acc, OP>(pair, lane);
                Acc ex = __shfl_up_sync(0xffffffffu, inc, 1);
                if (lane == 0) ex = scan_identity<Acc, OP>();
#pragma unroll
                for (int p = 0; p < PER; ++p) {
                    sm.wex[s][lane * PER + p] = ex;
                    ex = scan_apply<Acc, OP>(ex, a[p]);
                }
                if (lane == 31) {
                    sm.agg[s] = inc;
                    desc_store(desc + t, ((unsigned long long)pl.epoch << 32) | acc_bits(inc));   // at once: other blocks wait for it
                }
                __syncwarp();
                if (lane == 31) mbar_arrive(&sm.aggready[s]);
            }
            return 1;
        };
        // phase C of local tile i: scan out of shared memory, stream to HBM
        auto phase_c = [&](int64_t i) -> bool {
            const int s = (int)(i % S);
            const uint32_t par = (uint32_t)(i / S) & 1u;
            if (!mbar_wait(&sm.resolved[s], par, abort_flag, budget)) {
                if (lane == 0) give_up();
                return false;
            }
            const int64_t t = sm.tile_of[s];
            const int nv = tile_vecs(t);
            const Acc prefix = sm.prefix[s];
            const bool seeded = t != 0 || pl.has_init;
            VT x[NV];
            Acc wex[NV];
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int v = j * kRingConsumers + tid;
                wex[j] = sm.wex[s][j * kRingConsumerWarps + warp];
                if (v < nv) x[j] = __builtin_bit_cast(VT, *reinterpret_cast<const uint4*>(sm.stage[s] + (size_t)v * 16));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.empty[s]);      // the stage is in registers now
            uint4* dst = reinterpret_cast<uint4*>(B) + t * (int64_t)TILE_VECS;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int v = j * kRingConsumers + tid;
                const bool on = v < nv;
                Acc y[V];
#pragma unroll
                for (int q = 0; q < V; ++q) y[q] = on ? scan_up<T>(x[j].v[q]) : scan_identity<Acc, OP>();
#pragma unroll
                for (int q = 1; q < V; ++q) y[q] = scan_apply<Acc, OP>(y[q - 1], y[q]);
                const Acc inc = warp_scan_inclusive<Acc, OP>(y[V - 1], lane);
                Acc ex = __shfl_up_sync(0xffffffffu, inc, 1);
                if (lane == 0) ex = scan_identity<Acc, OP>();
                Acc off = scan_apply<Acc, OP>(wex[j], ex);
                if (seeded) off = scan_apply<Acc, OP>(prefix, off);
                VT out;
                if (pl.inclusive) {
#pragma unroll
                    for (int q = 0; q < V; ++q) out.v[q] = scan_down<T>(scan_apply<Acc, OP>(off, y[q]));
                } else {
                    out.v[0] = scan_down<T>(off);
#pragma unroll
                    for (int q = 1; q < V; ++q) out.v[q] = scan_down<T>(scan_apply<Acc, OP>(off, y[q - 1]));
                }
                if (on) st_policy16(dst + v, __builtin_bit_cast(uint4, out), stream);
            }
            return true;
        };

        const int lead = pl.lead < 1 ? 1 : (pl.lead > S - 2 ? S - 2 : pl.lead);
        int64_t reduced = 0;                     // tiles that went through phase A
        int more = 1;
        for (int k = 0; k < lead && more == 1; ++k) {
            more = phase_a(reduced);
            if (more == 1) ++reduced;
        }
        bool failed = false;
        for (int64_t c = 0; more >= 0; ++c) {
            if (more == 1) {
                more = phase_a(reduced);         // every consumer reaches this barrier, also after a failed phase C
                if (more == 1) ++reduced;
                if (more < 0) break;
            }
            if (failed || c >= reduced) break;
            if (!phase_c(c)) {
                failed = true;
                if (more != 1) break;            // no barrier ahead: leave at once
            }
        }
    }
    __syncthreads();
    // a block that gave up may still have copies in flight: they must land before it returns
    if (sm.abort && warp == kRingConsumerWarps && lane == 0) {
        const int64_t first = issued > S ? issued - S : 0;
        for (int64_t j = first; j < issued; ++j) {
            uint32_t tries = 0;
            while (!mbar_try_wait(&sm.full[j % S], (uint32_t)(j / S) & 1u) && ++tries < (1u << 20)) { }
        }
    }
}

// ---- host ------------------------------------------------------------------------------------------------
static int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    if (!e || !e[0]) return dflt;
    return atoi(e);
}

template <typename T, int OP, int NV>
static int32_t launch_ring(b200_stream_t st, const void* A, void* B, const ScanPlan& pl) {
    using Acc = typename ScanAcc<T>::type;
    using SM = RingShared<Acc, NV>;
    constexpr int TILE_VECS = kRingConsumers * NV;
    RingPlan rp{};
    rp.nvec = pl.L * (int64_t)sizeof(T) / 16;
    rp.ntiles = (rp.nvec + TILE_VECS - 1) / TILE_VECS;
    if (rp.ntiles >= ((int64_t)1 << 31) - 1024) return fail(B200_TOO_LARGE, "accumulate: too many tiles");
    rp.inclusive = pl.inclusive;
    rp.has_init = pl.has_init;
    rp.max_polls = pl.max_polls;
    rp.init = pl.init;
    rp.init_dev = pl.init_dev;
    static const int lead = env_int("B200_SCAN_RING_LEAD", 4);
    static const int inflight = env_int("B200_SCAN_RING_INFLIGHT", 2);
    rp.lead = lead;
    rp.inflight = inflight;
    void* state = nullptr;
    bool must_clear = false;
    const size_t dbytes = (size_t)rp.ntiles * sizeof(unsigned long long);
    B200_TRY(scan_state(st, dbytes, &state, &rp.epoch, &must_clear));
    if (must_clear) B200_CUDA(cudaMemsetAsync(state, 0, kScanStateHeader + dbytes, st->s));
    auto kernel = scan_ring_kernel<T, OP, NV>;
    static bool configured[64] = {false};
    if (st->dev < 64 && !configured[st->dev]) {
        B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SM)));
        configured[st->dev] = true;
    }
    int64_t grid = sm_count(st->dev);
    if (grid > rp.ntiles) grid = rp.ntiles;
    kernel<<<(unsigned)grid, kRingThreads, sizeof(SM), st->s>>>(
        (const T*)A, (T*)B, rp, reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(state) + kScanStateHeader),
        reinterpret_cast<unsigned int*>(state), device_error_word(st->dev));
    // a replayed graph repeats its tag and its ticket word: leave both ticket words at zero behind it
    if (must_clear) B200_CUDA(cudaMemsetAsync(state, 0, kScanStateHeader, st->s));
    return B200_OK;
}

template <typename T, int NV>
static int32_t launch_ring_op(b200_stream_t st, int op, const void* A, void* B, const ScanPlan& pl) {
    switch (op) {
        case B200_RED_ADD: return launch_ring<T, B200_RED_ADD, NV>(st, A, B, pl);
        case B200_RED_MUL: return launch_ring<T, B200_RED_MUL, NV>(st, A, B, pl);
        case B200_RED_MAX: return launch_ring<T, B200_RED_MAX, NV>(st, A, B, pl);
        default: return launch_ring<T, B200_RED_MIN, NV>(st, A, B, pl);
    }
}

int32_t launch_scan_ring(b200_stream_t st, int32_t dtype, int32_t op, const void* A, void* B, const ScanPlan& pl) {
    static const int enabled = env_int("B200_SCAN_RING", 0);
    static const int nv = env_int("B200_SCAN_RING_VECS", 4);
    if (!enabled) return B200_UNSUPPORTED;
    if (pl.K != 1 || pl.M != 1) return B200_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(A) % 16 || reinterpret_cast<uintptr_t>(B) % 16 || (pl.L * dtype_size(dtype)) % 16) return B200_UNSUPPORTED;
#define B200_RING_DISPATCH(T)                                                        \
    return nv == 2 ? launch_ring_op<T, 2>(st, op, A, B, pl) : launch_ring_op<T, 4>(st, op, A, B, pl)
    switch (dtype) {
        case B200_F32: B200_RING_DISPATCH(float);
        case B200_I32: B200_RING_DISPATCH(int32_t);
        case B200_U32: B200_RING_DISPATCH(uint32_t);
        case B200_F16: B200_RING_DISPATCH(__half);
        case B200_BF16: B200_RING_DISPATCH(__nv_bfloat16);
        default: return B200_UNSUPPORTED;      // 8-byte accumulators keep the two-pass kernel
    }
#undef B200_RING_DISPATCH
}

}  // namespace b200
