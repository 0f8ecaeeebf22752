// mapreduce with dims: R[Iother] = op over Ireduce of f(A[I]).
//
// Takes the place of GPUArrays.mapreducedim! as implemented in src/kernels/mapreduce.jl:86-173
// of the reference (partial_mapreduce_device :43-82, reduce_group :8-34).  Where the reference
// needs up to three launches and two pool temporaries for one scalar (a 256-wide LDS tree per
// group, recursion over the partials), every path here is ONE launch: threads fold 128-bit
// vectors into registers, warps combine by shuffle, blocks through one shared-memory hop, and
// when several blocks share an output the last one to take a ticket folds their partials in a
// fixed order - results are reproducible run to run.
//
// Index spaces are collapsed to (K, L, M): K kept elements that are contiguous in memory, L
// reduced, M kept outer.  K == 1 streams contiguous runs (dims = leading dimensions, or all);
// K > 1 maps threads along K so that loads stay coalesced while each thread walks the strided
// reduced dimension (dims = 2 of a column-major matrix).  Anything else - a whole broadcast
// tree as the mapped function, several operands, gaps in the reduced dimensions, strided
// views - goes through the program evaluator.  Algorithmic traffic: sizeof(T) per input
// element plus the outputs.
#include "reduce_program.cuh"

#include <cstdlib>
#include <cstring>
#include <limits>
#include <type_traits>

namespace b200 {

enum { MAP_ID = 0, MAP_ABS = 1, MAP_ABS2 = 2 };

// ---- operator algebra ---------------------------------------------------------------------------------
template <typename Acc, int OP>
__device__ __forceinline__ Acc red_identity() {
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
__device__ __forceinline__ Acc red_apply(Acc a, Acc b) {
    using A = Arith<Acc>;
    if constexpr (OP == B200_RED_ADD) return A::add(a, b);
    else if constexpr (OP == B200_RED_MUL) return A::mul(a, b);
    else if constexpr (OP == B200_RED_MAX) return A::max(a, b);
    else return A::min(a, b);
}

template <typename T> struct InClass { using type = T; };
template <> struct InClass<__half> { using type = float; };
template <> struct InClass<__nv_bfloat16> { using type = float; };
template <typename T> __device__ __forceinline__ typename InClass<T>::type widen(T v) { return v; }
template <> __device__ __forceinline__ float widen<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// f is applied in the element's own arithmetic class, then the value widens to the accumulator.
template <typename Tin, typename Acc, int MAP>
__device__ __forceinline__ Acc map_elem(Tin x) {
    using C = typename InClass<Tin>::type;
    C v = widen(x);
    if constexpr (MAP == MAP_ABS) v = Arith<C>::abs(v);
    else if constexpr (MAP == MAP_ABS2) v = Arith<C>::mul(v, v);
    return (Acc)v;
}

// Extrema of 16-bit floats are exact in the element type: pairs are folded with ONE packed
// instruction per 32-bit word and widened once after the loop, instead of a conversion and a
// binary32 max per element.  Same semantics as the binary32 forms (NaN-propagating, -0.0 below
// +0.0).  Used for f = identity or abs.
template <typename Tin, int MAP, int OP>
constexpr bool kPackedExtremum = (std::is_same<Tin, __half>::value || std::is_same<Tin, __nv_bfloat16>::value) &&
                                 (OP == B200_RED_MAX || OP == B200_RED_MIN) && (MAP == MAP_ID || MAP == MAP_ABS);
template <typename Tin, int OP>
__device__ __forceinline__ uint32_t packed_extremum(uint32_t a, uint32_t b) {
    uint32_t r;
    if constexpr (std::is_same<Tin, __half>::value) {
        if constexpr (OP == B200_RED_MAX) asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        else asm("min.NaN.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    } else {
        if constexpr (OP == B200_RED_MAX) asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        else asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    }
    return r;
}
// -Inf (max) or +Inf (min) in both halves.
template <typename Tin, int OP>
__device__ __forceinline__ uint32_t packed_identity() {
    const uint32_t inf = std::is_same<Tin, __half>::value ? 0x7c00u : 0x7f80u;
    const uint32_t one = OP == B200_RED_MAX ? (inf | 0x8000u) : inf;
    return one | (one << 16);
}
template <typename Tin, int MAP, int OP>
__device__ __forceinline__ void packed_fold(uint32_t pacc[4], uint4 w) {
    if constexpr (MAP == MAP_ABS) { w.x &= 0x7fff7fffu; w.y &= 0x7fff7fffu; w.z &= 0x7fff7fffu; w.w &= 0x7fff7fffu; }
    pacc[0] = packed_extremum<Tin, OP>(pacc[0], w.x);
    pacc[1] = packed_extremum<Tin, OP>(pacc[1], w.y);
    pacc[2] = packed_extremum<Tin, OP>(pacc[2], w.z);
    pacc[3] = packed_extremum<Tin, OP>(pacc[3], w.w);
}
template <typename Tin>
__device__ __forceinline__ float unpack16(uint32_t w, int hi) {
    const unsigned short bits = (unsigned short)(hi ? (w >> 16) : (w & 0xffffu));
    if constexpr (std::is_same<Tin, __half>::value) return __half2float(__ushort_as_half(bits));
    else return __bfloat162float(__ushort_as_bfloat16(bits));
}

template <typename Acc>
__device__ __forceinline__ void store_result(void* R, int dt, int64_t idx, Acc v) {
    store_bits(R, dtype_bytes(dt), idx, encode<uint64_t>(dt, raw_of<uint64_t>(v)));
}
template <typename Acc>
__device__ __forceinline__ Acc load_result(const void* R, int dt, int64_t idx) {
    return as_c<Acc, uint64_t>(decode<uint64_t>(dt, load_bits(R, dtype_bytes(dt), idx)));
}

template <typename Acc, int OP>
__device__ __forceinline__ Acc warp_reduce(Acc v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = red_apply<Acc, OP>(v, __shfl_down_sync(0xffffffffu, v, off));
    return v;
}
// Result valid in thread 0.  `smem` holds 32 values.
template <typename Acc, int OP>
__device__ __forceinline__ Acc block_reduce(Acc v, Acc* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_reduce<Acc, OP>(v);
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < nwarps ? smem[lane] : red_identity<Acc, OP>();
        v = warp_reduce<Acc, OP>(v);
    }
    __syncthreads();
    return v;
}

// Folds n contiguous elements starting at p into acc[0..V), cooperatively over `nthr` threads.
template <typename Tin, typename Acc, int MAP, int OP, int V>
__device__ __forceinline__ void segment_accumulate(const Tin* p, int64_t n, int tid, int nthr, Acc acc[V]) {
    using VT = Vec<Tin, V>;
    int64_t head = (int64_t)(((16 - (reinterpret_cast<uintptr_t>(p) & 15)) & 15) / sizeof(Tin));
    if (head > n) head = n;
    if (tid < head) acc[0] = red_apply<Acc, OP>(acc[0], map_elem<Tin, Acc, MAP>(p[tid]));
    const uint4* vp = reinterpret_cast<const uint4*>(p + head);
    const int64_t nv = (n - head) / V;
    constexpr int U = 4;
    int64_t i = tid;
    if constexpr (kPackedExtremum<Tin, MAP, OP> && V == 8) {
        uint32_t pacc[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) pacc[q] = packed_identity<Tin, OP>();
        for (; i + (int64_t)(U - 1) * nthr < nv; i += (int64_t)U * nthr) {
            uint4 w[U];
#pragma unroll
            for (int u = 0; u < U; ++u) w[u] = __ldcs(vp + i + (int64_t)u * nthr);
#pragma unroll
            for (int u = 0; u < U; ++u) packed_fold<Tin, MAP, OP>(pacc, w[u]);
        }
        for (; i < nv; i += nthr) packed_fold<Tin, MAP, OP>(pacc, __ldcs(vp + i));
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] = red_apply<Acc, OP>(acc[k], (Acc)unpack16<Tin>(pacc[k / 2], k & 1));
    } else {
        for (; i + (int64_t)(U - 1) * nthr < nv; i += (int64_t)U * nthr) {
            VT v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = __builtin_bit_cast(VT, __ldcs(vp + i + (int64_t)u * nthr));
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] = red_apply<Acc, OP>(acc[k], map_elem<Tin, Acc, MAP>(v[u].v[k]));
        }
        for (; i < nv; i += nthr) {
            VT v = __builtin_bit_cast(VT, __ldcs(vp + i));
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] = red_apply<Acc, OP>(acc[k], map_elem<Tin, Acc, MAP>(v.v[k]));
        }
    }
    const int64_t done = head + nv * V;
    if (tid < n - done) acc[0] = red_apply<Acc, OP>(acc[0], map_elem<Tin, Acc, MAP>(p[done + tid]));
}

template <typename Acc, int OP, int V>
__device__ __forceinline__ Acc fold_lanes(const Acc acc[V]) {
    Acc r = acc[0];
#pragma unroll
    for (int k = 1; k < V; ++k) r = red_apply<Acc, OP>(r, acc[k]);
    return r;
}


template <typename Acc, int OP>
__device__ __forceinline__ void finalize(const RedOut& o, int64_t idx, Acc v) {
    Acc seed = o.use_init ? as_c<Acc, uint64_t>(o.init) : load_result<Acc>(o.R, o.rdtype, idx);
    store_result<Acc>(o.R, o.rdtype, idx, red_apply<Acc, OP>(seed, v));
}

// Final step of a full reduction.  Without peers: thread 0 stores op(seed, v).  With peers (the
// fused reduce + all-reduce): the block stores this rank's partial into every rank's exchange
// slot over NVLink, waits (bounded) until the partials of all ranks have arrived in its own
// buffer and folds them in rank order, so every rank obtains the same bits.  `v` is valid in
// thread 0; all threads of the block must call.
template <typename Acc, int OP>
__device__ __forceinline__ void block_finalize(const RedOut& o, const PeerCtx& peer, int64_t idx, Acc v) {
    if (peer.nranks == 0) {
        if (threadIdx.x == 0) finalize<Acc, OP>(o, idx, v);
        return;
    }
    __shared__ unsigned long long s_bits[kMaxPeers];
    __shared__ int s_peer_abort;
    const int tid = threadIdx.x;
    const int bank = (int)(peer.seq & 1ull) * kMaxPeers;
    if (tid == 0) { s_bits[0] = raw_of<uint64_t>(v); s_peer_abort = 0; }
    __syncthreads();
    const unsigned long long mine = s_bits[0];
    __syncthreads();
    if (tid < peer.nranks) {
        // my partial -> slot [bank][rank] of rank `tid` (a peer store unless tid == rank)
        volatile PeerSlot* dst = peer.bufs[tid] + bank + peer.rank;
        dst->value = mine;
        __threadfence_system();
        dst->seq = peer.seq;
        // rank tid's partial <- my own buffer
        volatile PeerSlot* src = peer.bufs[peer.rank] + bank + tid;
        uint32_t polls = 0;
        bool ok = true;
        while (src->seq != peer.seq) {
            if (++polls > peer.max_polls) { ok = false; break; }
            if ((polls & 1023u) == 0 && error_latched(peer.err_word)) { ok = false; break; }
            __nanosleep(polls > 256 ? 256 : 32);
        }
        if (ok) {
            __threadfence_system();
            s_bits[tid] = src->value;
        } else {
            s_peer_abort = 1;
        }
    }
    __syncthreads();
    if (tid == 0) {
        if (s_peer_abort) {
            latch_error(peer.err_word, B200_LOOKBACK_TIMEOUT);
        } else {
            Acc total = as_c<Acc, uint64_t>(s_bits[0]);
            for (int r = 1; r < peer.nranks; ++r) total = red_apply<Acc, OP>(total, as_c<Acc, uint64_t>(s_bits[r]));
            finalize<Acc, OP>(o, idx, total);
        }
    }
    __syncthreads();
}

// (map, op) pairs with a statically specialised inner loop; everything else uses the evaluator.
#define B200_MAPOP(MAPV, OPV) ((MAPV) * 4 + (OPV))
#define B200_MAPOP_SWITCH(mapop, CALL)                                                             \
    switch (mapop) {                                                                               \
        case B200_MAPOP(MAP_ID, B200_RED_ADD): CALL(MAP_ID, B200_RED_ADD); break;                  \
        case B200_MAPOP(MAP_ID, B200_RED_MUL): CALL(MAP_ID, B200_RED_MUL); break;                  \
        case B200_MAPOP(MAP_ID, B200_RED_MAX): CALL(MAP_ID, B200_RED_MAX); break;                  \
        case B200_MAPOP(MAP_ID, B200_RED_MIN): CALL(MAP_ID, B200_RED_MIN); break;                  \
        case B200_MAPOP(MAP_ABS, B200_RED_ADD): CALL(MAP_ABS, B200_RED_ADD); break;                \
        case B200_MAPOP(MAP_ABS, B200_RED_MAX): CALL(MAP_ABS, B200_RED_MAX); break;                \
        case B200_MAPOP(MAP_ABS, B200_RED_MIN): CALL(MAP_ABS, B200_RED_MIN); break;                \
        case B200_MAPOP(MAP_ABS2, B200_RED_ADD): CALL(MAP_ABS2, B200_RED_ADD); break;              \
        default: break;                                                                            \
    }
static bool mapop_supported(int map, int op) {
    if (map == MAP_ID) return true;
    if (map == MAP_ABS) return op != B200_RED_MUL;
    return op == B200_RED_ADD;
}

// ---- K == 1: contiguous runs --------------------------------------------------------------------------
// One block per (column, chunk).  With B > 1 chunks per column the last block to finish a column
// folds the B partials.
template <typename Tin, typename Acc, int MAP, int OP>
__device__ __forceinline__ void contig_block_body(const Tin* A, int64_t L, int64_t M, int B, int64_t chunk,
                                                  Acc* partials, unsigned int* counters, const RedOut& out,
                                                  const PeerCtx& peer) {
    constexpr int V = 16 / sizeof(Tin);
    __shared__ Acc smem[32];
    __shared__ int s_last;
    const int64_t items = M * B;
    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const int64_t m = item / B;
        const int b = (int)(item - m * B);
        const int64_t beg = (int64_t)b * chunk;
        int64_t end = beg + chunk;
        if (end > L) end = L;
        Acc acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] = red_identity<Acc, OP>();
        if (end > beg) segment_accumulate<Tin, Acc, MAP, OP, V>(A + m * L + beg, end - beg, threadIdx.x, blockDim.x, acc);
        Acc v = block_reduce<Acc, OP>(fold_lanes<Acc, OP, V>(acc), smem);
        if (B == 1) {
            block_finalize<Acc, OP>(out, peer, m, v);
            continue;
        }
        if (threadIdx.x == 0) {
            partials[m * B + b] = v;
            __threadfence();
            const unsigned int t = atomicAdd(&counters[m], 1u);
            s_last = (t == (unsigned int)(B - 1));
            if (s_last) counters[m] = 0;
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            Acc p = red_identity<Acc, OP>();
            for (int j = threadIdx.x; j < B; j += blockDim.x) p = red_apply<Acc, OP>(p, __ldcg(&partials[m * B + j]));
            p = block_reduce<Acc, OP>(p, smem);
            block_finalize<Acc, OP>(out, peer, m, p);
        }
        __syncthreads();
    }
}

template <typename Tin, typename Acc>
__global__ void __launch_bounds__(kRedThreads)
reduce_contig_block_kernel(const Tin* A, int64_t L, int64_t M, int B, int64_t chunk, int mapop,
                           Acc* partials, unsigned int* counters, RedOut out, const __grid_constant__ PeerCtx peer) {
    grid_dependency_wait();
    grid_dependency_release();
#define CALL(MAPV, OPV) contig_block_body<Tin, Acc, MAPV, OPV>(A, L, M, B, chunk, partials, counters, out, peer)
    B200_MAPOP_SWITCH(mapop, CALL)
#undef CALL
}

// One warp per column.
template <typename Tin, typename Acc, int MAP, int OP>
__device__ __forceinline__ void contig_warp_body(const Tin* A, int64_t L, int64_t M, const RedOut& out) {
    constexpr int V = 16 / sizeof(Tin);
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t m = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); m < M; m += nwarps) {
        Acc acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] = red_identity<Acc, OP>();
        segment_accumulate<Tin, Acc, MAP, OP, V>(A + m * L, L, lane, 32, acc);
        Acc v = warp_reduce<Acc, OP>(fold_lanes<Acc, OP, V>(acc));
        if (lane == 0) finalize<Acc, OP>(out, m, v);
    }
}
template <typename Tin, typename Acc>
__global__ void __launch_bounds__(kRedThreads)
reduce_contig_warp_kernel(const Tin* A, int64_t L, int64_t M, int mapop, RedOut out) {
    grid_dependency_wait();
    grid_dependency_release();
#define CALL(MAPV, OPV) contig_warp_body<Tin, Acc, MAPV, OPV>(A, L, M, out)
    B200_MAPOP_SWITCH(mapop, CALL)
#undef CALL
}

// One thread per column (very short columns; neighbouring threads read neighbouring columns).
template <typename Tin, typename Acc, int MAP, int OP>
__device__ __forceinline__ void contig_thread_body(const Tin* A, int64_t L, int64_t M, const RedOut& out) {
    const int64_t nthr = (int64_t)gridDim.x * blockDim.x;
    for (int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; m < M; m += nthr) {
        Acc v = red_identity<Acc, OP>();
        const Tin* p = A + m * L;
        for (int64_t l = 0; l < L; ++l) v = red_apply<Acc, OP>(v, map_elem<Tin, Acc, MAP>(p[l]));
        finalize<Acc, OP>(out, m, v);
    }
}
template <typename Tin, typename Acc>
__global__ void __launch_bounds__(kRedThreads)
reduce_contig_thread_kernel(const Tin* A, int64_t L, int64_t M, int mapop, RedOut out) {
    grid_dependency_wait();
    grid_dependency_release();
#define CALL(MAPV, OPV) contig_thread_body<Tin, Acc, MAPV, OPV>(A, L, M, out)
    B200_MAPOP_SWITCH(mapop, CALL)
#undef CALL
}

// ---- K > 1: strided reduced dimension ---------------------------------------------------------------
struct StridedPlan {
    int64_t K, L, M;
    int     kx, ly;        // threads along K (each owning V consecutive k) and along L
    int64_t LS;            // rows per strip
    int     nstrips;
    int64_t kblocks;
};

template <typename Tin, typename Acc, int MAP, int OP, int V>
__device__ __forceinline__ void strided_body(const Tin* A, const StridedPlan& pl, Acc* partials,
                                             unsigned int* counters, const RedOut& out, Acc* smem) {
    using VT = Vec<Tin, V>;
    __shared__ int s_last;
    const int tx = threadIdx.x % pl.kx, ty = threadIdx.x / pl.kx;
    const bool lane_on = ty < pl.ly;
    const int64_t items = pl.kblocks * pl.nstrips * pl.M;
    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const int64_t kb = item % pl.kblocks;
        const int64_t rest = item / pl.kblocks;
        const int strip = (int)(rest % pl.nstrips);
        const int64_t m = rest / pl.nstrips;
        const int64_t k0 = (kb * pl.kx + tx) * V;
        const bool on = lane_on && k0 < pl.K;
        const int64_t lbeg = (int64_t)strip * pl.LS;
        int64_t lend = lbeg + pl.LS;
        if (lend > pl.L) lend = pl.L;
        Acc acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] = red_identity<Acc, OP>();
        if (on) {
            const Tin* base = A + k0 + pl.K * (pl.L * m);
            constexpr int U = 8;
            int64_t l = lbeg + ty;
            if constexpr (kPackedExtremum<Tin, MAP, OP> && V == 8) {
                uint32_t pacc[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) pacc[q] = packed_identity<Tin, OP>();
                for (; l + (int64_t)(U - 1) * pl.ly < lend; l += (int64_t)U * pl.ly) {
                    uint4 w[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) w[u] = __ldcs(reinterpret_cast<const uint4*>(base + pl.K * (l + (int64_t)u * pl.ly)));
#pragma unroll
                    for (int u = 0; u < U; ++u) packed_fold<Tin, MAP, OP>(pacc, w[u]);
                }
                for (; l < lend; l += pl.ly) packed_fold<Tin, MAP, OP>(pacc, __ldcs(reinterpret_cast<const uint4*>(base + pl.K * l)));
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] = red_apply<Acc, OP>(acc[k], (Acc)unpack16<Tin>(pacc[k / 2], k & 1));
            }
            for (; l + (int64_t)(U - 1) * pl.ly < lend; l += (int64_t)U * pl.ly) {
                VT v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const Tin* p = base + pl.K * (l + (int64_t)u * pl.ly);
                    if constexpr (V * sizeof(Tin) == 16) v[u] = __builtin_bit_cast(VT, __ldcs(reinterpret_cast<const uint4*>(p)));
                    else v[u].v[0] = *p;
                }
#pragma unroll
                for (int u = 0; u < U; ++u)
#pragma unroll
                    for (int k = 0; k < V; ++k) acc[k] = red_apply<Acc, OP>(acc[k], map_elem<Tin, Acc, MAP>(v[u].v[k]));
            }
            for (; l < lend; l += pl.ly) {
                const Tin* p = base + pl.K * l;
                VT v;
                if constexpr (V * sizeof(Tin) == 16) v = __builtin_bit_cast(VT, __ldcs(reinterpret_cast<const uint4*>(p)));
                else v.v[0] = *p;
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] = red_apply<Acc, OP>(acc[k], map_elem<Tin, Acc, MAP>(v.v[k]));
            }
        }
        // Two forms of the tail.  Eight-lane tiles (16-bit elements): one thread per output column
        // from here on - their row-group layout would be read with 8-way bank conflicts by a single
        // warp, and 23 strips would be folded by eight-deep dependent loops (measured 28.9 -> 27.3 us
        // on 8192 x 8192).  Narrower tiles keep the row-group form, which measured about 1 us faster
        // for them (Float32 matrix 43.8 against 44.5 us, 3 x 1 000 000 8.2 against 8.9 us).
        if constexpr (V == 8) {
            // Combine the ly row groups through shared memory, in row-group order.  The values are laid
            // out [row group][lane k][column tx], so that neighbouring threads touch neighbouring words,
            // and from here on thread c < kx * V owns ONE output column: lane kc = c / kx of the
            // vector of thread-column tc = c % kx.
            if (lane_on) {
    #pragma unroll
                for (int k = 0; k < V; ++k) smem[(ty * V + k) * pl.kx + tx] = acc[k];
            }
            __syncthreads();
            const int width = pl.kx * V;
            const int c = threadIdx.x;
            const int kc = c / pl.kx, tc = c - kc * pl.kx;
            const int64_t col = (kb * pl.kx + tc) * V + kc;                 // column of the matrix
            const bool col_on = c < width && col < pl.K;
            Acc val = red_identity<Acc, OP>();
            if (c < width) {
                val = smem[c];
                for (int y = 1; y < pl.ly; ++y) val = red_apply<Acc, OP>(val, smem[y * width + c]);
            }
            const int64_t tile = m * pl.kblocks + kb;
            if (pl.nstrips == 1) {
                if (col_on) finalize<Acc, OP>(out, col + pl.K * m, val);
                __syncthreads();
                continue;
            }
            if (c < width) partials[(tile * pl.nstrips + strip) * width + c] = val;
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                const unsigned int t = atomicAdd(&counters[tile], 1u);
                s_last = (t == (unsigned int)(pl.nstrips - 1));
                if (s_last) counters[tile] = 0;
            }
            __syncthreads();
            if (s_last) {
                __threadfence();
                // The last block of a tile folds the strips.  With a full-width tile every thread owns
                // one column and walks the strips in order, four reads in flight; a narrow tile (few
                // columns, many strips) splits the strips over kRedThreads / width thread groups, whose
                // results are combined through shared memory in group order.  Fixed orders both.
                const int groups = kRedThreads / width;
                const int g = c / width, cc = c - g * width;
                const int64_t gcol = (kb * pl.kx + (cc % pl.kx)) * V + cc / pl.kx;
                const bool g_on = g < groups && gcol < pl.K;
                Acc part = red_identity<Acc, OP>();
                if (g_on) {
                    const Acc* src = partials + tile * pl.nstrips * width + cc;
                    int s = g;
                    for (; s + 3 * groups < pl.nstrips; s += 4 * groups) {
                        const Acc p0 = __ldcg(src + (int64_t)s * width), p1 = __ldcg(src + (int64_t)(s + groups) * width);
                        const Acc p2 = __ldcg(src + (int64_t)(s + 2 * groups) * width), p3 = __ldcg(src + (int64_t)(s + 3 * groups) * width);
                        part = red_apply<Acc, OP>(red_apply<Acc, OP>(red_apply<Acc, OP>(red_apply<Acc, OP>(part, p0), p1), p2), p3);
                    }
                    for (; s < pl.nstrips; s += groups) part = red_apply<Acc, OP>(part, __ldcg(src + (int64_t)s * width));
                }
                if (groups > 1) {
                    if (g < groups) smem[g * width + cc] = part;
                    __syncthreads();
                    if (g == 0 && g_on)
                        for (int y = 1; y < groups; ++y) part = red_apply<Acc, OP>(part, smem[y * width + cc]);
                }
                if (g == 0 && g_on) finalize<Acc, OP>(out, gcol + pl.K * m, part);
            }
        } else {
            // combine the ly row groups through shared memory, in row-group order
            if (lane_on) {
    #pragma unroll
                for (int k = 0; k < V; ++k) smem[(ty * pl.kx + tx) * V + k] = acc[k];
            }
            __syncthreads();
            if (ty == 0) {
                for (int y = 1; y < pl.ly; ++y)
    #pragma unroll
                    for (int k = 0; k < V; ++k) acc[k] = red_apply<Acc, OP>(acc[k], smem[(y * pl.kx + tx) * V + k]);
            }
            const int64_t tile = m * pl.kblocks + kb;
            if (pl.nstrips == 1) {
                if (ty == 0 && k0 < pl.K) {
    #pragma unroll
                    for (int k = 0; k < V; ++k) finalize<Acc, OP>(out, k0 + k + pl.K * m, acc[k]);
                }
                __syncthreads();
                continue;
            }
            const int64_t width = (int64_t)pl.kx * V;
            if (ty == 0) {
    #pragma unroll
                for (int k = 0; k < V; ++k) partials[(tile * pl.nstrips + strip) * width + tx * V + k] = acc[k];
            }
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                const unsigned int t = atomicAdd(&counters[tile], 1u);
                s_last = (t == (unsigned int)(pl.nstrips - 1));
                if (s_last) counters[tile] = 0;
            }
            __syncthreads();
            if (s_last) {
                __threadfence();
                // every row group folds its share of the strips (strip s goes to group s % ly), then
                // the groups are combined through shared memory in group order: a fixed order, and
                // the whole block takes part instead of one warp
                Acc part[V];
    #pragma unroll
                for (int k = 0; k < V; ++k) part[k] = red_identity<Acc, OP>();
                if (lane_on && k0 < pl.K) {
                    const Acc* src = partials + tile * pl.nstrips * width + tx * V;
                    for (int s = ty; s < pl.nstrips; s += pl.ly) {
    #pragma unroll
                        for (int k = 0; k < V; ++k) part[k] = red_apply<Acc, OP>(part[k], __ldcg(src + (int64_t)s * width + k));
                    }
                }
                if (lane_on) {
    #pragma unroll
                    for (int k = 0; k < V; ++k) smem[(ty * pl.kx + tx) * V + k] = part[k];
                }
                __syncthreads();
                if (ty == 0 && k0 < pl.K) {
                    for (int y = 1; y < pl.ly; ++y)
    #pragma unroll
                        for (int k = 0; k < V; ++k) part[k] = red_apply<Acc, OP>(part[k], smem[(y * pl.kx + tx) * V + k]);
    #pragma unroll
                    for (int k = 0; k < V; ++k) finalize<Acc, OP>(out, k0 + k + pl.K * m, part[k]);
                }
            }
        }
        __syncthreads();
    }
}

template <typename Tin, typename Acc, int V>
__global__ void __launch_bounds__(kRedThreads, V >= 8 ? 5 : 1)
reduce_strided_kernel(const Tin* A, StridedPlan pl, int mapop, Acc* partials, unsigned int* counters, RedOut out) {
    __shared__ Acc smem[kRedThreads * V];
    grid_dependency_wait();
    grid_dependency_release();
#define CALL(MAPV, OPV) strided_body<Tin, Acc, MAPV, OPV, V>(A, pl, partials, counters, out, smem)
    B200_MAPOP_SWITCH(mapop, CALL)
#undef CALL
}

// ---- host ------------------------------------------------------------------------------------------------
static int acc_dtype_of(int rdtype) {
    switch (dtype_class(rdtype)) {
        case CF32: return B200_F32;
        case CF64: return B200_F64;
        case CI32: return B200_I32;
        case CI64: return B200_I64;
        case CU32: return B200_U32;
        default: return B200_U64;
    }
}

static uint64_t identity_bits(int redop, int acc_dtype) {
    auto f32 = [](float f) { uint32_t u; memcpy(&u, &f, 4); return (uint64_t)u; };
    auto f64 = [](double d) { uint64_t u; memcpy(&u, &d, 8); return u; };
    switch (acc_dtype) {
        case B200_F32:
            return redop == B200_RED_ADD ? f32(0.f) : redop == B200_RED_MUL ? f32(1.f)
                 : redop == B200_RED_MAX ? f32(-std::numeric_limits<float>::infinity()) : f32(std::numeric_limits<float>::infinity());
        case B200_F64:
            return redop == B200_RED_ADD ? f64(0.) : redop == B200_RED_MUL ? f64(1.)
                 : redop == B200_RED_MAX ? f64(-std::numeric_limits<double>::infinity()) : f64(std::numeric_limits<double>::infinity());
        case B200_I32:
            return redop == B200_RED_ADD ? 0u : redop == B200_RED_MUL ? 1u
                 : redop == B200_RED_MAX ? (uint64_t)(uint32_t)INT32_MIN : (uint64_t)(uint32_t)INT32_MAX;
        case B200_I64:
            return redop == B200_RED_ADD ? 0u : redop == B200_RED_MUL ? 1u
                 : redop == B200_RED_MAX ? (uint64_t)INT64_MIN : (uint64_t)INT64_MAX;
        case B200_U32:
            return redop == B200_RED_ADD ? 0u : redop == B200_RED_MUL ? 1u
                 : redop == B200_RED_MAX ? 0u : (uint64_t)UINT32_MAX;
        default:
            return redop == B200_RED_ADD ? 0u : redop == B200_RED_MUL ? 1u
                 : redop == B200_RED_MAX ? 0u : UINT64_MAX;
    }
}

template <typename Tin, typename Acc>
static int32_t launch_fast(b200_stream_t st, const void* A, int64_t K, int64_t L, int64_t M, int mapop, const RedOut& out,
                           b200_peer_t peer = nullptr) {
    void* scr = nullptr;
    unsigned int* counters = nullptr;
    PeerCtx pc{};
    if (peer && (K != 1 || M != 1)) return fail(B200_UNSUPPORTED, "the fused reduce + all-reduce handles full reductions only");
    if (K == 1) {
        if (!peer && M > 1 && L <= 16) {
            const int64_t res = resident_blocks(reduce_contig_thread_kernel<Tin, Acc>, kRedThreads, 0, st->dev);
            launch_overlapped(reduce_contig_thread_kernel<Tin, Acc>, balanced_grid((M + kRedThreads - 1) / kRedThreads, res), kRedThreads, 0, st->s,
                              (const Tin*)A, L, M, mapop, out);
            return B200_OK;
        }
        const int64_t wres = resident_blocks(reduce_contig_warp_kernel<Tin, Acc>, kRedThreads, 0, st->dev);
        if (!peer && M >= wres * 8 && (size_t)L * sizeof(Tin) <= 65536) {
            launch_overlapped(reduce_contig_warp_kernel<Tin, Acc>, balanced_grid((M + 7) / 8, wres), kRedThreads, 0, st->s,
                              (const Tin*)A, L, M, mapop, out);
            return B200_OK;
        }
        // the grid is exactly one resident wave: blocks per column fill it, each block with at
        // least 16 KiB of input
        const int64_t target = resident_blocks(reduce_contig_block_kernel<Tin, Acc>, kRedThreads, 0, st->dev);
        const int64_t min_chunk = (int64_t)(16384 / sizeof(Tin));
        int64_t B = target / M;
        const int64_t maxB = (L + min_chunk - 1) / min_chunk;
        if (B > maxB) B = maxB;
        if (B < 1) B = 1;
        if (B > 1 && (size_t)M * sizeof(unsigned int) > kCounterBytes) B = 1;
        int64_t chunk = (L + B - 1) / B;
        const int64_t grain = (int64_t)kRedThreads * (16 / sizeof(Tin));
        chunk = (chunk + grain - 1) / grain * grain;
        B = (L + chunk - 1) / chunk;
        B200_TRY(scratch(st, (size_t)(M * B) * sizeof(Acc), &scr, &counters));
        // the collective's sequence number is taken last: a call that fails above must not count
        if (peer) B200_TRY(peer_next_context(peer, st, &pc));
        launch_overlapped(reduce_contig_block_kernel<Tin, Acc>, balanced_grid(M * B, target), kRedThreads, 0, st->s,
                          (const Tin*)A, L, M, (int)B, chunk, mapop, (Acc*)scr, counters, out, pc);
        return B200_OK;
    }
    // strided
    constexpr int VMAX = 16 / sizeof(Tin);
    const bool vec = (K % VMAX == 0) && (reinterpret_cast<uintptr_t>(A) % 16 == 0) && K / VMAX >= 8;
    StridedPlan pl{};
    pl.K = K; pl.L = L; pl.M = M;
    const int V = vec ? VMAX : 1;
    const int64_t kv = (K + V - 1) / V;
    // a warp covers 32 vectors (512 B) of a row, the block's other warps take other rows; wider
    // row chunks measured slower on B200 (fewer column blocks leave more strips to combine)
    pl.kx = (int)(kv < 32 ? kv : 32);
    pl.ly = kRedThreads / pl.kx;
    if ((int64_t)pl.ly > L) pl.ly = (int)L;
    pl.kblocks = (kv + pl.kx - 1) / pl.kx;
    const int64_t target = vec ? resident_blocks(reduce_strided_kernel<Tin, Acc, VMAX>, kRedThreads, 0, st->dev)
                               : resident_blocks(reduce_strided_kernel<Tin, Acc, 1>, kRedThreads, 0, st->dev);
    const int64_t base_blocks = pl.kblocks * M;
    int64_t ns = target / base_blocks;        // strips fill one resident wave
    const int64_t max_ns = (L + (int64_t)pl.ly * 4 - 1) / ((int64_t)pl.ly * 4);
    if (ns > max_ns) ns = max_ns;
    if (ns < 1) ns = 1;
    if (ns > 1 && (size_t)base_blocks * sizeof(unsigned int) > kCounterBytes) ns = 1;
    pl.LS = (L + ns - 1) / ns;
    pl.LS = (pl.LS + pl.ly - 1) / pl.ly * pl.ly;
    pl.nstrips = (int)((L + pl.LS - 1) / pl.LS);
    B200_TRY(scratch(st, (size_t)(base_blocks * pl.nstrips * pl.kx * V) * sizeof(Acc), &scr, &counters));
    const unsigned blocks = balanced_grid(base_blocks * pl.nstrips, target);
    if (vec) launch_overlapped(reduce_strided_kernel<Tin, Acc, VMAX>, (unsigned)blocks, kRedThreads, 0, st->s, (const Tin*)A, pl, mapop, (Acc*)scr, counters, out);
    else launch_overlapped(reduce_strided_kernel<Tin, Acc, 1>, (unsigned)blocks, kRedThreads, 0, st->s, (const Tin*)A, pl, mapop, (Acc*)scr, counters, out);
    return B200_OK;
}

}  // namespace b200

using namespace b200;

// A rank with an empty shard still takes part in the fused all-reduce: one warp publishes the
// operator's neutral element as this rank's partial and folds the partials of all ranks.
template <typename Acc>
__global__ void __launch_bounds__(32) peer_neutral_kernel(int op, RedOut out, const __grid_constant__ PeerCtx peer) {
    switch (op) {
        case B200_RED_ADD: block_finalize<Acc, B200_RED_ADD>(out, peer, 0, red_identity<Acc, B200_RED_ADD>()); break;
        case B200_RED_MUL: block_finalize<Acc, B200_RED_MUL>(out, peer, 0, red_identity<Acc, B200_RED_MUL>()); break;
        case B200_RED_MAX: block_finalize<Acc, B200_RED_MAX>(out, peer, 0, red_identity<Acc, B200_RED_MAX>()); break;
        default: block_finalize<Acc, B200_RED_MIN>(out, peer, 0, red_identity<Acc, B200_RED_MIN>()); break;
    }
}

static int32_t launch_peer_neutral(b200_stream_t st, b200_peer_t peer, int acc_dt, int op, const RedOut& out) {
    PeerCtx pc{};
    B200_TRY(peer_next_context(peer, st, &pc));
    switch (acc_dt) {
        case B200_F32: peer_neutral_kernel<float><<<1, 32, 0, st->s>>>(op, out, pc); break;
        case B200_F64: peer_neutral_kernel<double><<<1, 32, 0, st->s>>>(op, out, pc); break;
        case B200_I32: peer_neutral_kernel<int32_t><<<1, 32, 0, st->s>>>(op, out, pc); break;
        case B200_I64: peer_neutral_kernel<int64_t><<<1, 32, 0, st->s>>>(op, out, pc); break;
        case B200_U32: peer_neutral_kernel<uint32_t><<<1, 32, 0, st->s>>>(op, out, pc); break;
        default: peer_neutral_kernel<uint64_t><<<1, 32, 0, st->s>>>(op, out, pc); break;
    }
    return B200_OK;
}

static int32_t mapreduce_impl(b200_stream_t st, const b200_tensor* R, const int64_t* shape, int32_t ndim,
                              const b200_leaf* leaves, int32_t nleaves, const uint8_t* program,
                              int32_t ninstr, int32_t op, const void* init, b200_peer_t peer, bool prepare_only = false) {
    // prepare_only: validate, and compile the kernel this call would need; no stream, no device
    if (!prepare_only) B200_TRY(enter(st));
    std::unique_lock<std::recursive_mutex> guard;
    if (!prepare_only) guard = std::unique_lock<std::recursive_mutex>(st->mu);
    B200_TRY(check_tensor(R, "mapreduce destination"));
    if (!shape && ndim > 0) return fail(B200_INVALID_ARG, "mapreduce: null shape");
    if (ndim < 0 || ndim > B200_MAX_DIMS) return fail(B200_INVALID_ARG, "mapreduce: ndim %d outside [0,%d]", ndim, B200_MAX_DIMS);
    if (op < 0 || op >= B200_RED_COUNT) return fail(B200_UNSUPPORTED, "mapreduce: unknown operator %d", op);
    if (R->dtype == B200_BOOL) return fail(B200_UNSUPPORTED, "mapreduce: Bool destinations are not supported");
    if (R->ndim > ndim) {
        for (int d = ndim; d < R->ndim; ++d)
            if (R->shape[d] != 1) return fail(B200_INVALID_ARG, "mapreduce: destination has more dimensions than the input");
    }
    uint32_t mask = 0;
    int64_t n = 1, n_out = 1, n_red = 1;
    for (int d = 0; d < ndim; ++d) {
        if (shape[d] < 0) return fail(B200_INVALID_ARG, "mapreduce: negative extent");
        const int64_t re = d < R->ndim ? R->shape[d] : 1;
        n *= shape[d];
        if (re == shape[d]) n_out *= shape[d];
        else if (re == 1) { mask |= 1u << d; n_red *= shape[d]; }
        else return fail(B200_INVALID_ARG, "mapreduce: destination extent %lld in dim %d matches neither %lld nor 1 (check_reducedims)", (long long)re, d, (long long)shape[d]);
    }
    if (n == 0 && !peer) return B200_OK;   // empty input: R is returned untouched

    const int acc_dt = acc_dtype_of(R->dtype);
    RedOut out{};
    out.R = R->ptr;
    out.rdtype = R->dtype;
    out.use_init = init ? 1 : 0;
    if (init) {
        uint64_t bits = 0;
        memcpy(&bits, init, dtype_size(R->dtype));
        out.init = scalar_to_class(R->dtype, bits);
    }
    Compiled C;
    B200_TRY(compile_program(shape, ndim, leaves, nleaves, program, ninstr, acc_dt, &C));
    // operands that are transposed / permuted views: dense copies first (one pool allocation, freed
    // on the stream when this call has enqueued its kernels)
    struct PoolTemp {
        b200_stream_t st;
        void* ptr = nullptr;
        ~PoolTemp() { if (ptr) b200_free_async(ptr, st); }
    } temp{st};
    b200_leaf fixed[B200_MAX_LEAVES];
    if (!prepare_only && !C.P.linear && n > 0 && leaves && nleaves > 0 && nleaves <= B200_MAX_LEAVES) {
        B200_TRY(densify_permuted_leaves(st, shape, ndim, leaves, nleaves, fixed, &temp.ptr));
        if (temp.ptr) B200_TRY(compile_program(shape, ndim, fixed, nleaves, program, ninstr, acc_dt, &C));
    }

    // ---- fast paths: one dense array, f in {identity, abs, abs2}
    const ProgramDesc& P = C.P;
    // (a one-element "reduction" is a plain map and goes to the evaluator, except in the fused
    // all-reduce, where the shard of a rank may well hold a single element)
    bool fast = C.n_array_leaves == 1 && P.linear && tensor_is_contiguous(R) && (n_red > 1 || peer);
    int map = MAP_ID, leaf = -1, in_dt = -1;
    if (fast) {
        int pc = 0;
        if (P.code[0] != B200_OP_LEAF || P.leaves[P.code[1]].is_scalar) fast = false;
        else { leaf = P.code[1]; in_dt = P.leaves[leaf].dtype; pc = 1; }
        if (fast && pc < P.ninstr && (P.code[2 * pc] == B200_OP_ABS || P.code[2 * pc] == B200_OP_ABS2)) {
            map = P.code[2 * pc] == B200_OP_ABS ? MAP_ABS : MAP_ABS2;
            ++pc;
        }
        if (fast && pc < P.ninstr && P.code[2 * pc] == B200_OP_CONVERT && (P.code[2 * pc + 1] >> 4) == in_dt) ++pc;
        if (pc != P.ninstr) fast = false;
        if (fast && !mapop_supported(map, op)) fast = false;
    }
    int64_t K = 1, L = 1, M = 1;
    if (fast) {
        int i0 = -1, i1 = -1;
        for (int d = 0; d < ndim; ++d) if (((mask >> d) & 1u) && shape[d] > 1) { if (i0 < 0) i0 = d; i1 = d; }
        if (i0 < 0) {
            // no reduced dimension longer than one element (a one-element shard of a sharded
            // reduction): every element is its own run
            M = n;
        } else {
            for (int d = i0; d <= i1 && fast; ++d) if (shape[d] > 1 && !((mask >> d) & 1u)) fast = false;
            if (fast) {
                for (int d = 0; d < i0; ++d) K *= shape[d];
                for (int d = i0; d <= i1; ++d) L *= shape[d];
                for (int d = i1 + 1; d < ndim; ++d) M *= shape[d];
            }
        }
    }
    if (prepare_only && fast) return B200_OK;     // served by a kernel that is part of the library
    if (fast && n == 0) {
        // empty shard of a sharded reduction; whether the expression is one the fused kernel
        // handles was decided above exactly as on the ranks that hold data
        const bool typed = (acc_dt == B200_F32 && (in_dt == B200_F32 || in_dt == B200_F16 || in_dt == B200_BF16)) ||
                           (acc_dt == B200_F64 && in_dt == B200_F64) || (acc_dt == B200_I32 && in_dt == B200_I32) ||
                           (acc_dt == B200_I64 && (in_dt == B200_I32 || in_dt == B200_I64));
        if (typed) {
            B200_TRY(launch_peer_neutral(st, peer, acc_dt, op, out));
            return finish(st, "b200_mapreduce_allreduce");
        }
        fast = false;
    }
    if (fast) {
        const void* A = P.leaves[leaf].ptr;
        const int mapop = B200_MAPOP(map, op);
        int32_t s = -1;
        if (in_dt == B200_F32 && acc_dt == B200_F32) s = launch_fast<float, float>(st, A, K, L, M, mapop, out, peer);
        else if (in_dt == B200_F16 && acc_dt == B200_F32) s = launch_fast<__half, float>(st, A, K, L, M, mapop, out, peer);
        else if (in_dt == B200_BF16 && acc_dt == B200_F32) s = launch_fast<__nv_bfloat16, float>(st, A, K, L, M, mapop, out, peer);
        else if (in_dt == B200_F64 && acc_dt == B200_F64) s = launch_fast<double, double>(st, A, K, L, M, mapop, out, peer);
        else if (in_dt == B200_I32 && acc_dt == B200_I32) s = launch_fast<int32_t, int32_t>(st, A, K, L, M, mapop, out, peer);
        else if (in_dt == B200_I32 && acc_dt == B200_I64) s = launch_fast<int32_t, int64_t>(st, A, K, L, M, mapop, out, peer);
        else if (in_dt == B200_I64 && acc_dt == B200_I64) s = launch_fast<int64_t, int64_t>(st, A, K, L, M, mapop, out, peer);
        if (s >= 0) {
            B200_TRY(s);
            return finish(st, "b200_mapreduce");
        }
    }

    if (peer) return fail(B200_UNSUPPORTED, "the fused reduce + all-reduce needs a full reduction of one dense array with "
                          "f in {identity, abs, abs2}; use b200_mapreduce followed by b200_allreduce for anything else");

    // ---- evaluator path
    GenericPlan G{};
    G.n_out = n_out;
    G.n_red = n_red;
    G.reduced_mask = mask;
    G.full = (n_out == 1) ? 1 : 0;
    G.redop = op;
    G.acc_dtype = acc_dt;
    G.identity = identity_bits(op, acc_dt);
    if (!G.full) { C.P.linear = 0; C.P.vec_ok = 0; }
    if (prepare_only) return jit_prepare_reduce(C, R->dtype, op, acc_dt, G.full);
    // the kernel specialised for this expression at run time if there is one, else the interpreter
    LeafDesc O{};
    O.ptr = R->ptr;
    O.dtype = R->dtype;
    for (int d = 0; d < ndim; ++d) O.stride[d] = (d < R->ndim && R->shape[d] != 1) ? R->stride[d] : 0;
    const void* special = nullptr;
    int64_t special_resident = 0;
    const int got = jit_reduce_kernel(st, C, O.dtype, op, acc_dt, G.full, &special, &special_resident);
    if (got < 0)
        return fail(B200_UNSUPPORTED, "first use of this mapreduce expression inside a stream capture: its kernel has to "
                    "be compiled and loaded, run the expression once before capturing");
    const int64_t target = special ? special_resident
                         : C.wide ? resident_blocks(reduce_program_kernel<true>, kRedThreads, 0, st->dev)
                                  : resident_blocks(reduce_program_kernel<false>, kRedThreads, 0, st->dev);
    int64_t B = target / n_out;
    const int64_t min_chunk = 16384;
    const int64_t maxB = (n_red + min_chunk - 1) / min_chunk;
    if (B > maxB) B = maxB;
    if (B < 1) B = 1;
    if (B > 1 && (size_t)n_out * sizeof(unsigned int) > kCounterBytes) B = 1;
    int64_t chunk = (n_red + B - 1) / B;
    chunk = (chunk + kVec * kRedThreads - 1) / (kVec * kRedThreads) * (kVec * kRedThreads);
    B = (n_red + chunk - 1) / chunk;
    G.B = (int)B;
    G.chunk = chunk;
    void* scr = nullptr;
    unsigned int* counters = nullptr;
    B200_TRY(scratch(st, (size_t)(n_out * B) * 8, &scr, &counters));
    const unsigned blocks = balanced_grid(n_out * B, target);
    if (special) {
        void* args[] = {(void*)&C.P, (void*)&O, (void*)&G, (void*)&scr, (void*)&counters, (void*)&out};
        if (launch_overlapped_handle(special, blocks, kRedThreads, args, st->s) == cudaSuccess)
            return finish(st, "b200_mapreduce");
        cudaGetLastError();      // fall through to the interpreter
    }
    if (C.wide) reduce_program_kernel<true><<<blocks, kRedThreads, 0, st->s>>>(C.P, O, G, (uint64_t*)scr, counters, out);
    else reduce_program_kernel<false><<<blocks, kRedThreads, 0, st->s>>>(C.P, O, G, (uint32_t*)scr, counters, out);
    return finish(st, "b200_mapreduce");
}

extern "C" int32_t b200_mapreduce(b200_stream_t st, const b200_tensor* R, const int64_t* shape, int32_t ndim,
                                  const b200_leaf* leaves, int32_t nleaves, const uint8_t* program,
                                  int32_t ninstr, int32_t op, const void* init) {
    return mapreduce_impl(st, R, shape, ndim, leaves, nleaves, program, ninstr, op, init, nullptr);
}

extern "C" int32_t b200_mapreduce_prepare(const b200_tensor* R, const int64_t* shape, int32_t ndim, const b200_leaf* leaves,
                                          int32_t nleaves, const uint8_t* program, int32_t ninstr, int32_t op) {
    return mapreduce_impl(nullptr, R, shape, ndim, leaves, nleaves, program, ninstr, op, nullptr, nullptr, true);
}

extern "C" int32_t b200_mapreduce_allreduce(b200_peer_t peer, b200_stream_t st, const b200_tensor* R, const int64_t* shape,
                                            int32_t ndim, const b200_leaf* leaves, int32_t nleaves,
                                            const uint8_t* program, int32_t ninstr, int32_t op, const void* init) {
    if (!peer) return fail(B200_INVALID_ARG, "null peer group");
    if (R && tensor_numel(R) != 1) return fail(B200_UNSUPPORTED, "the fused reduce + all-reduce produces one element");
    // the group's sequence number advances only when a kernel that exchanges is really launched
    return mapreduce_impl(st, R, shape, ndim, leaves, nleaves, program, ninstr, op, init, peer);
}
