// Elementwise programs: host-side validation ("compile") of the postfix byte code that the
// C ABI accepts, and the device-side evaluator shared by the broadcast and mapreduce kernels.
//
// The evaluator is a stack machine whose stack lives in REGISTERS: the top of the stack is
// always the same named register vector, pushes and pops shift the (at most five) live slots
// with plain moves, so no slot is ever addressed dynamically, nothing goes to local memory and
// every instruction is ONE indirect branch on a handler number that the host computed.  Each
// instruction is decoded once per thread for a vector of kVec consecutive elements.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int kVec = 4;        // elements evaluated per thread per decode
constexpr int kMaxStack = 5;   // deepest value stack a program may need
constexpr int kPrefetch = 4;   // array leaves whose loads are issued before decoding starts

// Value classes: the arithmetic type an element type computes in.
enum { CF32 = 0, CF64 = 1, CI32 = 2, CI64 = 3, CU32 = 4, CU64 = 5 };

__host__ __device__ inline int dtype_class(int dt) {
    switch (dt) {
        case B200_F16: case B200_BF16: case B200_F32: return CF32;
        case B200_F64: return CF64;
        case B200_I8: case B200_I16: case B200_I32: return CI32;
        case B200_I64: return CI64;
        case B200_U64: return CU64;
        default: return CU32;
    }
}
__host__ __device__ inline bool dtype_is_narrow(int dt) {
    return dt == B200_F16 || dt == B200_BF16 || dt == B200_I8 || dt == B200_I16 ||
           dt == B200_U8 || dt == B200_U16 || dt == B200_BOOL;
}
__host__ __device__ inline int dtype_bytes(int dt) {
    switch (dt) {
        case B200_F16: case B200_BF16: case B200_I16: case B200_U16: return 2;
        case B200_F32: case B200_I32: case B200_U32: return 4;
        case B200_F64: case B200_I64: case B200_U64: return 8;
        default: return 1;
    }
}

struct LeafDesc {
    const void* ptr;
    uint64_t    scalar;                  // class representation (f16 scalar already widened)
    int64_t     stride[B200_MAX_DIMS];   // elements; 0 in broadcast dims
    int32_t     dtype;
    int32_t     is_scalar;
};

struct ProgramDesc {
    int32_t  ninstr, nleaves, ndim;
    int32_t  linear;      // every array leaf is dense with the shape of the index space
    int32_t  vec_ok;      // ... and 4-element accesses are aligned for every array leaf
    int32_t  _pad;
    int64_t  shape[B200_MAX_DIMS];
    uint8_t  code[2 * (B200_MAX_PROGRAM + 2)];    // validated (opcode, dtype) pairs, for the host
    uint8_t  hcode[2 * (B200_MAX_PROGRAM + 2)];   // (handler, operand) pairs, what the device runs
    LeafDesc leaves[B200_MAX_LEAVES];
};

// Handler numbers of the device evaluator.  Operators: kHOps + class * kNumOps + (opcode - ADD).
enum { kHPre0 = 0, kHPre1 = 1, kHPre2 = 2, kHPre3 = 3, kHLeafMem = 4, kHConvert = 5, kHOps = 6, kNumOps = 11 };

struct Compiled {
    ProgramDesc P;
    int32_t result_dtype;   // dtype left on the stack by the last instruction
    bool    wide;           // some value needs a 64-bit class
    // Expression tree in postfix order for pattern matching by the operators.
    int32_t n_array_leaves;
};

#ifndef __CUDACC_RTC__
// Validates `program` against `leaves` and the index space `shape`; appends a conversion to
// `final_dtype` when that is >= 0 and differs from the program's result type.
int32_t compile_program(const int64_t* shape, int32_t ndim, const b200_leaf* leaves,
                        int32_t nleaves, const uint8_t* program, int32_t ninstr,
                        int32_t final_dtype, Compiled* out);

// Run-time specialisation (jit.cu): launch the kernel compiled for exactly this expression
// (1), report that there is none so that the caller interprets (0), or that it cannot be built
// inside a stream capture (-1); compile it without launching.
int jit_broadcast(b200_stream_t st, const Compiled& C, const LeafDesc& O, int64_t n);
int32_t jit_prepare_reduce(const Compiled& C, int out_dtype, int redop, int acc_dtype, int full);
// Replaces operands that are transposed / permuted views by dense copies (broadcast.cu).
int32_t densify_permuted_leaves(b200_stream_t st, const int64_t* shape, int32_t ndim, const b200_leaf* leaves,
                                int32_t nleaves, b200_leaf* fixed, void** pool_temp);
int32_t jit_prepare(const Compiled& C, int out_dtype);
int jit_reduce_kernel(b200_stream_t st, const Compiled& C, int out_dtype, int redop, int acc_dtype, int full,
                      const void** kernel, int64_t* resident);

// Converts one scalar between its storage bits and the class representation (host side).
uint64_t scalar_to_class(int32_t dtype, uint64_t bits);
uint64_t class_to_storage(int32_t dtype, uint64_t cls);
#endif  // !__CUDACC_RTC__

#ifdef __CUDACC__

template <bool WIDE> struct RawOf { using type = uint32_t; };
template <> struct RawOf<true> { using type = uint64_t; };

// ---- raw <-> class value ------------------------------------------------------------------------
template <typename C, typename R> __device__ __forceinline__ C as_c(R r);
template <> __device__ __forceinline__ float as_c<float, uint32_t>(uint32_t r) { return __uint_as_float(r); }
template <> __device__ __forceinline__ float as_c<float, uint64_t>(uint64_t r) { return __uint_as_float((uint32_t)r); }
template <> __device__ __forceinline__ double as_c<double, uint64_t>(uint64_t r) { return __longlong_as_double((long long)r); }
template <> __device__ __forceinline__ double as_c<double, uint32_t>(uint32_t r) { return (double)__uint_as_float(r); }
template <> __device__ __forceinline__ int32_t as_c<int32_t, uint32_t>(uint32_t r) { return (int32_t)r; }
template <> __device__ __forceinline__ int32_t as_c<int32_t, uint64_t>(uint64_t r) { return (int32_t)(uint32_t)r; }
template <> __device__ __forceinline__ uint32_t as_c<uint32_t, uint32_t>(uint32_t r) { return r; }
template <> __device__ __forceinline__ uint32_t as_c<uint32_t, uint64_t>(uint64_t r) { return (uint32_t)r; }
template <> __device__ __forceinline__ int64_t as_c<int64_t, uint64_t>(uint64_t r) { return (int64_t)r; }
template <> __device__ __forceinline__ int64_t as_c<int64_t, uint32_t>(uint32_t r) { return (int64_t)(int32_t)r; }
template <> __device__ __forceinline__ uint64_t as_c<uint64_t, uint64_t>(uint64_t r) { return r; }
template <> __device__ __forceinline__ uint64_t as_c<uint64_t, uint32_t>(uint32_t r) { return r; }

template <typename R> __device__ __forceinline__ R raw_of(float v) { return (R)__float_as_uint(v); }
template <typename R> __device__ __forceinline__ R raw_of(double v) { return (R)(uint64_t)__double_as_longlong(v); }
template <typename R> __device__ __forceinline__ R raw_of(int32_t v) { return (R)(uint32_t)v; }
template <typename R> __device__ __forceinline__ R raw_of(uint32_t v) { return (R)v; }
template <typename R> __device__ __forceinline__ R raw_of(int64_t v) { return (R)(uint64_t)v; }
template <typename R> __device__ __forceinline__ R raw_of(uint64_t v) { return (R)v; }

// ---- arithmetic per class (no contraction of separate multiply and add) --------------------------
template <typename C> struct Arith;
template <> struct Arith<float> {
    static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
    static __device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
    static __device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
    static __device__ __forceinline__ float div(float a, float b) { return __fdiv_rn(a, b); }
    static __device__ __forceinline__ float muladd(float a, float b, float c) { return fmaf(a, b, c); }
    static __device__ __forceinline__ float abs(float a) { return fabsf(a); }
    static __device__ __forceinline__ float exp(float a) { return expf(a); }
    static __device__ __forceinline__ float neg(float a) { return -a; }
    static __device__ __forceinline__ float max(float a, float b) { return jl_max(a, b); }
    static __device__ __forceinline__ float min(float a, float b) { return jl_min(a, b); }
};
template <> struct Arith<double> {
    static __device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }
    static __device__ __forceinline__ double sub(double a, double b) { return __dsub_rn(a, b); }
    static __device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
    static __device__ __forceinline__ double div(double a, double b) { return __ddiv_rn(a, b); }
    static __device__ __forceinline__ double muladd(double a, double b, double c) { return fma(a, b, c); }
    static __device__ __forceinline__ double abs(double a) { return fabs(a); }
    static __device__ __forceinline__ double exp(double a) { return ::exp(a); }
    static __device__ __forceinline__ double neg(double a) { return -a; }
    static __device__ __forceinline__ double max(double a, double b) { return jl_max(a, b); }
    static __device__ __forceinline__ double min(double a, double b) { return jl_min(a, b); }
};
template <typename I, typename U, bool SIGNED> struct IntArith {
    static __device__ __forceinline__ I add(I a, I b) { return (I)((U)a + (U)b); }
    static __device__ __forceinline__ I sub(I a, I b) { return (I)((U)a - (U)b); }
    static __device__ __forceinline__ I mul(I a, I b) { return (I)((U)a * (U)b); }
    static __device__ __forceinline__ I div(I a, I) { return a; }   // rejected by the validator
    static __device__ __forceinline__ I muladd(I a, I b, I c) { return (I)((U)a * (U)b + (U)c); }
    static __device__ __forceinline__ I abs(I a) { return (SIGNED && a < 0) ? (I)((U)0 - (U)a) : a; }
    static __device__ __forceinline__ I exp(I a) { return a; }      // rejected by the validator
    static __device__ __forceinline__ I neg(I a) { return (I)((U)0 - (U)a); }
    static __device__ __forceinline__ I max(I a, I b) { return a > b ? a : b; }
    static __device__ __forceinline__ I min(I a, I b) { return a < b ? a : b; }
};
template <> struct Arith<int32_t> : IntArith<int32_t, uint32_t, true> {};
template <> struct Arith<uint32_t> : IntArith<uint32_t, uint32_t, false> {};
template <> struct Arith<int64_t> : IntArith<int64_t, uint64_t, true> {};
template <> struct Arith<uint64_t> : IntArith<uint64_t, uint64_t, false> {};

// Rounds / wraps a class value to a narrow element type (Base computes Float16 in Float32 and
// rounds after every operation; Int8/Int16 arithmetic wraps).
template <typename R>
__device__ __forceinline__ R narrow(int dt, R r) {
    switch (dt) {
        case B200_F16: return raw_of<R>(__half2float(__float2half_rn(as_c<float>(r))));
        case B200_BF16: return raw_of<R>(__bfloat162float(__float2bfloat16_rn(as_c<float>(r))));
        case B200_I8: return raw_of<R>((int32_t)(int8_t)as_c<int32_t>(r));
        case B200_I16: return raw_of<R>((int32_t)(int16_t)as_c<int32_t>(r));
        case B200_U8: return raw_of<R>(as_c<uint32_t>(r) & 0xffu);
        case B200_U16: return raw_of<R>(as_c<uint32_t>(r) & 0xffffu);
        case B200_BOOL: return raw_of<R>(as_c<uint32_t>(r) & 1u);
        default: return r;
    }
}

// ---- element <-> class value -----------------------------------------------------------------------
template <typename R>
__device__ __forceinline__ R decode(int dt, uint64_t bits) {
    switch (dt) {
        case B200_F16: return raw_of<R>(__half2float(__ushort_as_half((unsigned short)bits)));
        case B200_BF16: return (R)((uint32_t)bits << 16);
        case B200_I8: return raw_of<R>((int32_t)(int8_t)bits);
        case B200_I16: return raw_of<R>((int32_t)(int16_t)bits);
        case B200_U8: case B200_BOOL: return (R)(bits & 0xffu);
        case B200_U16: return (R)(bits & 0xffffu);
        case B200_F32: case B200_I32: case B200_U32: return (R)(uint32_t)bits;
        default: return (R)bits;
    }
}
template <typename R>
__device__ __forceinline__ uint64_t encode(int dt, R r) {
    switch (dt) {
        case B200_F16: return __half_as_ushort(__float2half_rn(as_c<float>(r)));
        case B200_BF16: return __bfloat16_as_ushort(__float2bfloat16_rn(as_c<float>(r)));
        default: return (uint64_t)r;   // integer storage keeps the low bytes
    }
}

__device__ __forceinline__ uint64_t load_bits(const void* p, int bytes, int64_t off) {
    switch (bytes) {
        case 1: return __ldcs(reinterpret_cast<const uint8_t*>(p) + off);
        case 2: return __ldcs(reinterpret_cast<const uint16_t*>(p) + off);
        case 4: return __ldcs(reinterpret_cast<const uint32_t*>(p) + off);
        default: return __ldcs(reinterpret_cast<const unsigned long long*>(p) + off);
    }
}
__device__ __forceinline__ void store_bits(void* p, int bytes, int64_t off, uint64_t v) {
    switch (bytes) {
        case 1: reinterpret_cast<uint8_t*>(p)[off] = (uint8_t)v; break;
        case 2: reinterpret_cast<uint16_t*>(p)[off] = (uint16_t)v; break;
        case 4: __stcs(reinterpret_cast<uint32_t*>(p) + off, (uint32_t)v); break;
        default: __stcs(reinterpret_cast<unsigned long long*>(p) + off, (unsigned long long)v); break;
    }
}

// Four consecutive elements starting at element `off` (aligned access when `vec`).  The element
// type is switched on ONCE per vector, not per element: the evaluator's code size (and with it
// its instruction-cache behaviour) depends on it.
template <typename R>
__device__ __forceinline__ void load_vec4(const void* p, int dt, int64_t off, bool vec, int nvalid, R out[kVec]) {
    const bool fast = vec && nvalid == kVec;
    switch (dt) {
        case B200_F32: case B200_I32: case B200_U32: {
            const uint32_t* q = reinterpret_cast<const uint32_t*>(p) + off;
            uint4 w = make_uint4(0, 0, 0, 0);
            if (fast) w = __ldcs(reinterpret_cast<const uint4*>(q));
            else {
                if (0 < nvalid) w.x = __ldcs(q);
                if (1 < nvalid) w.y = __ldcs(q + 1);
                if (2 < nvalid) w.z = __ldcs(q + 2);
                if (3 < nvalid) w.w = __ldcs(q + 3);
            }
            out[0] = (R)w.x; out[1] = (R)w.y; out[2] = (R)w.z; out[3] = (R)w.w;
            break;
        }
        case B200_F64: case B200_I64: case B200_U64: {
            const unsigned long long* q = reinterpret_cast<const unsigned long long*>(p) + off;
            unsigned long long w[kVec] = {0, 0, 0, 0};
            if (fast) {
                const ulonglong2 a = __ldcs(reinterpret_cast<const ulonglong2*>(q)), c = __ldcs(reinterpret_cast<const ulonglong2*>(q) + 1);
                w[0] = a.x; w[1] = a.y; w[2] = c.x; w[3] = c.y;
            } else {
#pragma unroll
                for (int k = 0; k < kVec; ++k) if (k < nvalid) w[k] = __ldcs(q + k);
            }
#pragma unroll
            for (int k = 0; k < kVec; ++k) out[k] = (R)w[k];
            break;
        }
        case B200_F16: case B200_BF16: case B200_I16: case B200_U16: {
            const uint16_t* q = reinterpret_cast<const uint16_t*>(p) + off;
            uint32_t h[kVec] = {0, 0, 0, 0};
            if (fast) {
                const uint2 w = __ldcs(reinterpret_cast<const uint2*>(q));
                h[0] = w.x & 0xffff; h[1] = w.x >> 16; h[2] = w.y & 0xffff; h[3] = w.y >> 16;
            } else {
#pragma unroll
                for (int k = 0; k < kVec; ++k) if (k < nvalid) h[k] = __ldcs(q + k);
            }
            if (dt == B200_F16) {
#pragma unroll
                for (int k = 0; k < kVec; ++k) out[k] = raw_of<R>(__half2float(__ushort_as_half((unsigned short)h[k])));
            } else if (dt == B200_BF16) {
#pragma unroll
                for (int k = 0; k < kVec; ++k) out[k] = (R)(h[k] << 16);
            } else if (dt == B200_I16) {
#pragma unroll
                for (int k = 0; k < kVec; ++k) out[k] = raw_of<R>((int32_t)(int16_t)h[k]);
            } else {
#pragma unroll
                for (int k = 0; k < kVec; ++k) out[k] = (R)h[k];
            }
            break;
        }
        default: {
            const uint8_t* q = reinterpret_cast<const uint8_t*>(p) + off;
            uint32_t h[kVec] = {0, 0, 0, 0};
            if (fast) {
                const uint32_t w = __ldcs(reinterpret_cast<const uint32_t*>(q));
                h[0] = w & 0xff; h[1] = (w >> 8) & 0xff; h[2] = (w >> 16) & 0xff; h[3] = w >> 24;
            } else {
#pragma unroll
                for (int k = 0; k < kVec; ++k) if (k < nvalid) h[k] = __ldcs(q + k);
            }
            if (dt == B200_I8) {
#pragma unroll
                for (int k = 0; k < kVec; ++k) out[k] = raw_of<R>((int32_t)(int8_t)h[k]);
            } else {
#pragma unroll
                for (int k = 0; k < kVec; ++k) out[k] = (R)h[k];
            }
            break;
        }
    }
}

template <typename R>
__device__ __forceinline__ void store_vec4(void* p, int dt, int64_t off, bool vec, int nvalid, const R in[kVec]) {
    const bool fast = vec && nvalid == kVec;
    switch (dt) {
        case B200_F32: case B200_I32: case B200_U32: {
            uint32_t* q = reinterpret_cast<uint32_t*>(p) + off;
            if (fast) __stcs(reinterpret_cast<uint4*>(q), make_uint4((uint32_t)in[0], (uint32_t)in[1], (uint32_t)in[2], (uint32_t)in[3]));
            else {
#pragma unroll
                for (int k = 0; k < kVec; ++k) if (k < nvalid) __stcs(q + k, (uint32_t)in[k]);
            }
            break;
        }
        case B200_F64: case B200_I64: case B200_U64: {
            unsigned long long* q = reinterpret_cast<unsigned long long*>(p) + off;
            if (fast) {
                __stcs(reinterpret_cast<ulonglong2*>(q), make_ulonglong2((unsigned long long)in[0], (unsigned long long)in[1]));
                __stcs(reinterpret_cast<ulonglong2*>(q) + 1, make_ulonglong2((unsigned long long)in[2], (unsigned long long)in[3]));
            } else {
#pragma unroll
                for (int k = 0; k < kVec; ++k) if (k < nvalid) __stcs(q + k, (unsigned long long)in[k]);
            }
            break;
        }
        case B200_F16: case B200_BF16: case B200_I16: case B200_U16: {
            uint32_t h[kVec];
            if (dt == B200_F16) {
#pragma unroll
                for (int k = 0; k < kVec; ++k) h[k] = __half_as_ushort(__float2half_rn(as_c<float>(in[k])));
            } else if (dt == B200_BF16) {
#pragma unroll
                for (int k = 0; k < kVec; ++k) h[k] = __bfloat16_as_ushort(__float2bfloat16_rn(as_c<float>(in[k])));
            } else {
#pragma unroll
                for (int k = 0; k < kVec; ++k) h[k] = (uint32_t)in[k] & 0xffffu;
            }
            uint16_t* q = reinterpret_cast<uint16_t*>(p) + off;
            if (fast) __stcs(reinterpret_cast<uint2*>(q), make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16)));
            else {
#pragma unroll
                for (int k = 0; k < kVec; ++k) if (k < nvalid) q[k] = (uint16_t)h[k];
            }
            break;
        }
        default: {
            uint8_t* q = reinterpret_cast<uint8_t*>(p) + off;
            if (fast) *reinterpret_cast<uint32_t*>(q) = ((uint32_t)in[0] & 0xff) | (((uint32_t)in[1] & 0xff) << 8) | (((uint32_t)in[2] & 0xff) << 16) | (((uint32_t)in[3] & 0xff) << 24);
            else {
#pragma unroll
                for (int k = 0; k < kVec; ++k) if (k < nvalid) q[k] = (uint8_t)in[k];
            }
            break;
        }
    }
}

// Rounds / wraps a whole register vector to a narrow element type (one switch per vector).
template <typename R>
__device__ __forceinline__ void narrow_vec(int dt, R v[kVec]) {
    switch (dt) {
        case B200_F16:
#pragma unroll
            for (int k = 0; k < kVec; ++k) v[k] = raw_of<R>(__half2float(__float2half_rn(as_c<float>(v[k]))));
            break;
        case B200_BF16:
#pragma unroll
            for (int k = 0; k < kVec; ++k) v[k] = raw_of<R>(__bfloat162float(__float2bfloat16_rn(as_c<float>(v[k]))));
            break;
        case B200_I8:
#pragma unroll
            for (int k = 0; k < kVec; ++k) v[k] = raw_of<R>((int32_t)(int8_t)as_c<int32_t>(v[k]));
            break;
        case B200_I16:
#pragma unroll
            for (int k = 0; k < kVec; ++k) v[k] = raw_of<R>((int32_t)(int16_t)as_c<int32_t>(v[k]));
            break;
        case B200_U8:
#pragma unroll
            for (int k = 0; k < kVec; ++k) v[k] = raw_of<R>(as_c<uint32_t>(v[k]) & 0xffu);
            break;
        case B200_U16:
#pragma unroll
            for (int k = 0; k < kVec; ++k) v[k] = raw_of<R>(as_c<uint32_t>(v[k]) & 0xffffu);
            break;
        case B200_BOOL:
#pragma unroll
            for (int k = 0; k < kVec; ++k) v[k] = raw_of<R>(as_c<uint32_t>(v[k]) & 1u);
            break;
        default: break;
    }
}

// ---- conversions between classes (rare: one nested switch) ---------------------------------------
template <typename S, typename D, typename R>
__device__ __forceinline__ void convert_class(R* c) {
#pragma unroll
    for (int k = 0; k < kVec; ++k) c[k] = raw_of<R>((D)as_c<S>(c[k]));
}

template <typename S, bool WIDE, typename R>
__device__ __forceinline__ void convert_from(int dst_class, R* c) {
    switch (dst_class) {
        case CF32: convert_class<S, float>(c); break;
        case CI32: convert_class<S, int32_t>(c); break;
        case CU32: convert_class<S, uint32_t>(c); break;
        default:
            if constexpr (WIDE) {
                if (dst_class == CF64) convert_class<S, double>(c);
                else if (dst_class == CI64) convert_class<S, int64_t>(c);
                else convert_class<S, uint64_t>(c);
            }
            break;
    }
}

template <bool WIDE, typename R>
__device__ __forceinline__ void exec_convert(int arg, R* c) {
    const int src = arg >> 4, dst = arg & 15;
    const int sc = dtype_class(src), dc = dtype_class(dst);
    if (sc != dc) {
        switch (sc) {
            case CF32: convert_from<float, WIDE>(dc, c); break;
            case CI32: convert_from<int32_t, WIDE>(dc, c); break;
            case CU32: convert_from<uint32_t, WIDE>(dc, c); break;
            default:
                if constexpr (WIDE) {
                    if (sc == CF64) convert_from<double, WIDE>(dc, c);
                    else if (sc == CI64) convert_from<int64_t, WIDE>(dc, c);
                    else convert_from<uint64_t, WIDE>(dc, c);
                }
                break;
        }
    }
    if (dtype_is_narrow(dst)) narrow_vec<R>(dst, c);
}

// Offset of index-space element `lin` inside leaf `L` (general strides / broadcast dims).
__device__ __forceinline__ int64_t leaf_offset(const ProgramDesc& P, const LeafDesc& L, int64_t lin) {
    int64_t off = 0;
    for (int d = 0; d < P.ndim; ++d) {
        const int64_t e = P.shape[d];
        const int64_t q = lin / e;
        off += (lin - q * e) * L.stride[d];
        lin = q;
    }
    return off;
}

// Where the evaluator takes its instruction stream from.  DynamicCode: the program travels in the
// kernel parameter and every instruction is decoded at run time (the interpreter).  A run-time
// compiled kernel instead supplies a type with the same members as compile-time constants
// (is_static = true); the loops below then unroll, every switch folds and what is left is
// straight-line code for that one expression - same helpers, same roundings, same results.
struct DynamicCode {
    static constexpr bool is_static = false;
    static constexpr int ninstr = 0, nleaves = 0, linear = 0, vec_ok = 0, out_dtype = 0;
    static constexpr int redop = 0, acc_dtype = 0, full = 0;      // reductions only (reduce_program.cuh)
    static constexpr unsigned char hcode[2] = {0, 0};
    static constexpr unsigned char leaf_dtype[1] = {0};
    static constexpr unsigned char leaf_scalar[1] = {0};
};

template <typename R, typename S = DynamicCode>
__device__ __forceinline__ void fetch_leaf(const ProgramDesc& P, int k, const int64_t lin[kVec], int nvalid, R out[kVec]) {
    const LeafDesc& L = P.leaves[k];
    const int dt = S::is_static ? (int)S::leaf_dtype[S::is_static ? k : 0] : L.dtype;
    const bool scalar = S::is_static ? S::leaf_scalar[S::is_static ? k : 0] != 0 : L.is_scalar != 0;
    const bool linear = S::is_static ? S::linear != 0 : P.linear != 0;
    const bool vec_ok = S::is_static ? S::vec_ok != 0 : P.vec_ok != 0;
    if (scalar) {
#pragma unroll
        for (int j = 0; j < kVec; ++j) out[j] = (R)L.scalar;
        return;
    }
    if (linear) {
        load_vec4<R>(L.ptr, dt, lin[0], vec_ok, nvalid, out);
    } else {
        const int bytes = dtype_bytes(dt);
#pragma unroll
        for (int j = 0; j < kVec; ++j)
            out[j] = (j < nvalid) ? decode<R>(dt, load_bits(L.ptr, bytes, leaf_offset(P, L, lin[j]))) : (R)0;
    }
}

// Evaluates the program for the index-space elements lin[0..nvalid).  In linear mode lin[] must
// be consecutive and lin[0] a multiple of kVec.
template <bool WIDE, typename S = DynamicCode>
__device__ __forceinline__ void eval_program(const ProgramDesc& P, const int64_t lin[kVec], int nvalid,
                                             typename RawOf<WIDE>::type result[kVec]) {
    using R = typename RawOf<WIDE>::type;
    const int nleaves = S::is_static ? S::nleaves : P.nleaves;
    // Issue the loads of the first array leaves before decoding anything, so that they overlap.
    R pre[kPrefetch][kVec];
#pragma unroll
    for (int k = 0; k < kPrefetch; ++k) {
        if (k < nleaves) fetch_leaf<R, S>(P, k, lin, nvalid, pre[k]);
    }
    // s0 is the top of the stack; a push moves every slot one down, a pop one up
    R s0[kVec], s1[kVec], s2[kVec], s3[kVec], s4[kVec];
#pragma unroll
    for (int j = 0; j < kVec; ++j) s0[j] = s1[j] = s2[j] = s3[j] = s4[j] = 0;
#define B200_SHIFT_DOWN() _Pragma("unroll") for (int j = 0; j < kVec; ++j) { s4[j] = s3[j]; s3[j] = s2[j]; s2[j] = s1[j]; s1[j] = s0[j]; }
#define B200_POP1() _Pragma("unroll") for (int j = 0; j < kVec; ++j) { s1[j] = s2[j]; s2[j] = s3[j]; s3[j] = s4[j]; }
#define B200_POP2() _Pragma("unroll") for (int j = 0; j < kVec; ++j) { s1[j] = s3[j]; s2[j] = s4[j]; }
#define B200_UN(C, EXPR) { _Pragma("unroll") for (int j = 0; j < kVec; ++j) { const C x = as_c<C>(s0[j]); s0[j] = raw_of<R>(EXPR); } } break;
#define B200_BIN(C, EXPR) { _Pragma("unroll") for (int j = 0; j < kVec; ++j) { const C x = as_c<C>(s1[j]); const C y = as_c<C>(s0[j]); s0[j] = raw_of<R>(EXPR); } B200_POP1() } break;
#define B200_TER(C, EXPR) { _Pragma("unroll") for (int j = 0; j < kVec; ++j) { const C x = as_c<C>(s2[j]); const C y = as_c<C>(s1[j]); const C z = as_c<C>(s0[j]); s0[j] = raw_of<R>(EXPR); } B200_POP2() } break;
#define B200_CLASS_CASES(CID, C)                                                          \
    case kHOps + CID * kNumOps + 0: B200_BIN(C, Arith<C>::add(x, y))                      \
    case kHOps + CID * kNumOps + 1: B200_BIN(C, Arith<C>::sub(x, y))                      \
    case kHOps + CID * kNumOps + 2: B200_BIN(C, Arith<C>::mul(x, y))                      \
    case kHOps + CID * kNumOps + 3: B200_BIN(C, Arith<C>::div(x, y))                      \
    case kHOps + CID * kNumOps + 4: B200_TER(C, Arith<C>::muladd(x, y, z))                \
    case kHOps + CID * kNumOps + 5: B200_UN(C, Arith<C>::abs(x))                          \
    case kHOps + CID * kNumOps + 6: B200_UN(C, Arith<C>::mul(x, x))                       \
    case kHOps + CID * kNumOps + 7: B200_UN(C, Arith<C>::exp(x))                          \
    case kHOps + CID * kNumOps + 8: B200_BIN(C, Arith<C>::max(x, y))                      \
    case kHOps + CID * kNumOps + 9: B200_BIN(C, Arith<C>::min(x, y))                      \
    case kHOps + CID * kNumOps + 10: B200_UN(C, Arith<C>::neg(x))
#define B200_EVAL_STEP \
        const int h = S::is_static ? (int)S::hcode[S::is_static ? 2 * pc : 0] : (int)P.hcode[2 * pc]; \
        const int arg = S::is_static ? (int)S::hcode[S::is_static ? 2 * pc + 1 : 1] : (int)P.hcode[2 * pc + 1]; \
        switch (h) { \
            case kHPre0: B200_SHIFT_DOWN() _Pragma("unroll") for (int j = 0; j < kVec; ++j) s0[j] = pre[0][j]; break; \
            case kHPre1: B200_SHIFT_DOWN() _Pragma("unroll") for (int j = 0; j < kVec; ++j) s0[j] = pre[1][j]; break; \
            case kHPre2: B200_SHIFT_DOWN() _Pragma("unroll") for (int j = 0; j < kVec; ++j) s0[j] = pre[2][j]; break; \
            case kHPre3: B200_SHIFT_DOWN() _Pragma("unroll") for (int j = 0; j < kVec; ++j) s0[j] = pre[3][j]; break; \
            case kHLeafMem: B200_SHIFT_DOWN() fetch_leaf<R, S>(P, arg, lin, nvalid, s0); break; \
            case kHConvert: exec_convert<WIDE, R>(arg, s0); break; \
            B200_CLASS_CASES(CF32, float) \
            B200_CLASS_CASES(CI32, int32_t) \
            B200_CLASS_CASES(CU32, uint32_t) \
            default: \
                if constexpr (WIDE) { \
                    switch (h) { \
                        B200_CLASS_CASES(CF64, double) \
                        B200_CLASS_CASES(CI64, int64_t) \
                        B200_CLASS_CASES(CU64, uint64_t) \
                        default: break; \
                    } \
                } \
                break; \
        } \
        /* operators on narrow element types re-round / re-wrap their result (operand = that dtype) */ \
        if (h >= kHOps && arg != 0xff) narrow_vec<R>(arg, s0);
    if constexpr (S::is_static) {
#pragma unroll
        for (int pc = 0; pc < S::ninstr; ++pc) { B200_EVAL_STEP }
    } else {
#pragma unroll 1
        for (int pc = 0; pc < P.ninstr; ++pc) { B200_EVAL_STEP }
    }
#undef B200_EVAL_STEP
#undef B200_CLASS_CASES
#undef B200_TER
#undef B200_BIN
#undef B200_UN
#undef B200_POP2
#undef B200_POP1
#undef B200_SHIFT_DOWN
#pragma unroll
    for (int j = 0; j < kVec; ++j) result[j] = s0[j];
}

// The broadcast loop over an arbitrary program: one vector of kVec elements per thread and step.
// Instantiated with DynamicCode inside the library (ew_program_kernel, the interpreter) and with
// a constant program by the run-time compiler (jit.cu wraps it in an extern "C" kernel).
template <bool WIDE, typename S = DynamicCode>
__device__ __forceinline__ void ew_program_body(const ProgramDesc& P, const LeafDesc& O, int64_t n) {
    using R = typename RawOf<WIDE>::type;
    const int64_t nvec = (n + kVec - 1) / kVec;
    const bool out_linear = S::is_static ? S::linear != 0 : P.linear != 0;
    const bool vec_ok = S::is_static ? S::vec_ok != 0 : P.vec_ok != 0;
    const int out_dtype = S::is_static ? (int)S::out_dtype : O.dtype;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
        int64_t lin[kVec];
#pragma unroll
        for (int j = 0; j < kVec; ++j) lin[j] = v * kVec + j;
        const int64_t left = n - v * kVec;
        const int nvalid = left < kVec ? (int)left : kVec;
        R res[kVec];
        eval_program<WIDE, S>(P, lin, nvalid, res);
        if (out_linear) {
            store_vec4<R>(const_cast<void*>(O.ptr), out_dtype, lin[0], vec_ok, nvalid, res);
        } else {
            const int bytes = dtype_bytes(out_dtype);
#pragma unroll
            for (int j = 0; j < kVec; ++j)
                if (j < nvalid) store_bits(const_cast<void*>(O.ptr), bytes, leaf_offset(P, O, lin[j]), encode<R>(out_dtype, res[j]));
        }
    }
}

template <bool WIDE>
__global__ void __launch_bounds__(256, WIDE ? 2 : 3)
ew_program_kernel(const __grid_constant__ ProgramDesc P, const __grid_constant__ LeafDesc O, int64_t n) {
    ew_program_body<WIDE, DynamicCode>(P, O, n);
}

#endif  // __CUDACC__

}  // namespace b200
