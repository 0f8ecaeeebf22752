// Definitions the scan kernels (accumulate.cu) share: operator algebra, accumulator types, the
// plan a launch is described by, and the warp scan.
#pragma once
#include "program.cuh"

#include <limits>
#include <type_traits>

namespace b200 {

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
    uint32_t epoch;          // tag of this launch in the descriptor words (0: the words were cleared)
    void* value_mem;         // 8-byte accumulators: aggregate / prefix values beside the flag words
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


}  // namespace b200
