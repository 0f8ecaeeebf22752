// mapreducedim! over an arbitrary map expression: the evaluator of program.cuh as the loader of a
// block reduction.  In a header of its own because the run-time compiler (jit.cu) builds this
// kernel, too, from the library's sources.
#pragma once
#include "program.cuh"

namespace b200 {

constexpr int kRedThreads = 256;

struct RedOut {
    void*    R;
    int32_t  rdtype;
    int32_t  use_init;
    uint64_t init;      // class bits of the accumulator type
};

struct GenericPlan {
    int64_t n_out, n_red;
    int     B;             // blocks per output
    int64_t chunk;         // reduced elements per block
    uint32_t reduced_mask; // bit d set: dimension d is reduced
    int32_t full;          // every dimension reduced: index = r, linear access allowed
    int32_t redop, acc_dtype;
    uint64_t identity;     // class bits
};

#ifdef __CUDACC__
template <typename C, typename R>
__device__ __forceinline__ R red_raw_c(int redop, R a, R b) {
    using A = Arith<C>;
    const C x = as_c<C>(a), y = as_c<C>(b);
    switch (redop) {
        case B200_RED_ADD: return raw_of<R>(A::add(x, y));
        case B200_RED_MUL: return raw_of<R>(A::mul(x, y));
        case B200_RED_MAX: return raw_of<R>(A::max(x, y));
        default: return raw_of<R>(A::min(x, y));
    }
}
template <bool WIDE, typename R>
__device__ __forceinline__ R red_raw(int redop, int cls, R a, R b) {
    switch (cls) {
        case CF32: return red_raw_c<float>(redop, a, b);
        case CI32: return red_raw_c<int32_t>(redop, a, b);
        case CU32: return red_raw_c<uint32_t>(redop, a, b);
        default:
            if constexpr (WIDE) {
                if (cls == CF64) return red_raw_c<double>(redop, a, b);
                if (cls == CI64) return red_raw_c<int64_t>(redop, a, b);
                return red_raw_c<uint64_t>(redop, a, b);
            }
            return a;
    }
}

// The reduction over an arbitrary map expression.  Like the broadcast loop it exists twice: with
// DynamicCode inside the library (reduce_program_kernel) and with the program, the reduction
// operator and the accumulator class as constants when compiled at run time.
template <bool WIDE, typename S>
__device__ __forceinline__ void reduce_program_body(const ProgramDesc& P, const LeafDesc& O, const GenericPlan& G,
                                                    typename RawOf<WIDE>::type* partials, unsigned int* counters,
                                                    const RedOut& out) {
    using R = typename RawOf<WIDE>::type;
    __shared__ R smem[kRedThreads];
    __shared__ int s_last;
    const int cls = dtype_class(S::is_static ? (int)S::acc_dtype : G.acc_dtype);
    const int redop = S::is_static ? (int)S::redop : G.redop;
    const bool full = S::is_static ? S::full != 0 : G.full != 0;
    const int out_dtype = S::is_static ? (int)S::out_dtype : O.dtype;
    const int64_t items = G.n_out * G.B;
    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const int64_t o = item / G.B;
        const int b = (int)(item - o * G.B);
        const int64_t rbeg = (int64_t)b * G.chunk;
        int64_t rend = rbeg + G.chunk;
        if (rend > G.n_red) rend = G.n_red;
        // one accumulator per vector lane: four short dependency chains instead of one long one
        R accv[kVec];
#pragma unroll
        for (int j = 0; j < kVec; ++j) accv[j] = (R)G.identity;
        for (int64_t r = rbeg + (int64_t)threadIdx.x * kVec; r < rend; r += (int64_t)blockDim.x * kVec) {
            const int64_t left = rend - r;
            const int nvalid = left < kVec ? (int)left : kVec;
            int64_t lin[kVec];
            if (full) {
#pragma unroll
                for (int j = 0; j < kVec; ++j) lin[j] = r + j;
            } else {
#pragma unroll
                for (int j = 0; j < kVec; ++j) {
                    int64_t rr = r + j, oo = o, mult = 1, li = 0;
                    for (int d = 0; d < P.ndim; ++d) {
                        const int64_t e = P.shape[d];
                        int64_t idx;
                        if ((G.reduced_mask >> d) & 1u) { idx = rr % e; rr /= e; }
                        else { idx = oo % e; oo /= e; }
                        li += idx * mult;
                        mult *= e;
                    }
                    lin[j] = li;
                }
            }
            R res[kVec];
            eval_program<WIDE, S>(P, lin, nvalid, res);
#pragma unroll
            for (int j = 0; j < kVec; ++j) if (j < nvalid) accv[j] = red_raw<WIDE, R>(redop, cls, accv[j], res[j]);
        }
        R acc = red_raw<WIDE, R>(redop, cls, red_raw<WIDE, R>(redop, cls, accv[0], accv[1]),
                                 red_raw<WIDE, R>(redop, cls, accv[2], accv[3]));
        smem[threadIdx.x] = acc;
        __syncthreads();
        for (int s = kRedThreads / 2; s > 0; s >>= 1) {
            if ((int)threadIdx.x < s) smem[threadIdx.x] = red_raw<WIDE, R>(redop, cls, smem[threadIdx.x], smem[threadIdx.x + s]);
            __syncthreads();
        }
        R v = smem[0];
        __syncthreads();
        bool write = (G.B == 1);
        if (G.B > 1) {
            if (threadIdx.x == 0) {
                partials[o * G.B + b] = v;
                __threadfence();
                const unsigned int t = atomicAdd(&counters[o], 1u);
                s_last = (t == (unsigned int)(G.B - 1));
                if (s_last) counters[o] = 0;
            }
            __syncthreads();
            if (s_last && threadIdx.x == 0) {
                __threadfence();
                v = (R)G.identity;
                for (int j = 0; j < G.B; ++j) v = red_raw<WIDE, R>(redop, cls, v, __ldcg(&partials[o * G.B + j]));
                write = true;
            }
            __syncthreads();
        }
        if (write && threadIdx.x == 0) {
            // offset of output o inside R (reduced dimensions have extent 1 there)
            int64_t oo = o, off = 0;
            for (int d = 0; d < P.ndim; ++d) {
                if ((G.reduced_mask >> d) & 1u) continue;
                const int64_t e = P.shape[d];
                off += (oo % e) * O.stride[d];
                oo /= e;
            }
            const int bytes = dtype_bytes(out_dtype);
            R seed = out.use_init ? (R)out.init : decode<R>(out_dtype, load_bits(O.ptr, bytes, off));
            v = red_raw<WIDE, R>(redop, cls, seed, v);
            store_bits(const_cast<void*>(O.ptr), bytes, off, encode<R>(out_dtype, v));
        }
    }
}

template <bool WIDE>
__global__ void __launch_bounds__(kRedThreads)
reduce_program_kernel(const __grid_constant__ ProgramDesc P, const __grid_constant__ LeafDesc O,
                      const __grid_constant__ GenericPlan G, typename RawOf<WIDE>::type* partials,
                      unsigned int* counters, RedOut out) {
    reduce_program_body<WIDE, DynamicCode>(P, O, G, partials, counters, out);
}
#endif  // __CUDACC__

}  // namespace b200
