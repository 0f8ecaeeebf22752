// Fused elementwise broadcast: out[I] = program(leaves[I]...).
//
// Takes the place of the kernel GPUArrays generates for a Broadcasted{ROCArrayStyle} tree
// (style selection in src/broadcast.jl:3-30 of the reference).  Instead of JIT-compiling one
// kernel per expression type, the tree arrives as a postfix program over a fixed operator set
// and is either matched against hard-wired streaming kernels (a*x+y, x*y+exp(-|z|)) or run by
// the register-stack evaluator of program.cuh.  Every path streams each operand exactly once
// with 128-bit accesses: the algorithmic traffic is sizeof(T) per array leaf plus sizeof(T)
// for the destination, per element.
#include "program.cuh"

#include <cstring>
#include <type_traits>
#include <vector>

namespace b200 {

// ---- host: scalar conversions -------------------------------------------------------------------
static float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ff;
    uint32_t f;
    if (exp == 0) {
        if (man == 0) f = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400));
            f = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
        }
    } else if (exp == 31) f = sign | 0x7f800000u | (man << 13);
    else f = sign | ((exp + 127 - 15) << 23) | (man << 13);
    float out;
    memcpy(&out, &f, 4);
    return out;
}

uint64_t scalar_to_class(int32_t dt, uint64_t bits) {
    switch (dt) {
        case B200_F16: { float f = half_bits_to_float((uint16_t)bits); uint32_t u; memcpy(&u, &f, 4); return u; }
        case B200_BF16: return (uint64_t)((uint32_t)(bits & 0xffff) << 16);
        case B200_I8: return (uint32_t)(int32_t)(int8_t)bits;
        case B200_I16: return (uint32_t)(int32_t)(int16_t)bits;
        case B200_U8: case B200_BOOL: return bits & 0xff;
        case B200_U16: return bits & 0xffff;
        case B200_F32: case B200_I32: case B200_U32: return bits & 0xffffffffu;
        default: return bits;
    }
}

// Host-side conversion of a scalar between element types (class representation in and out), with
// the same rounding as the device CONVERT: used to fold `convert(T, scalar)` at compile time so
// that e.g. `2 .* x` with an Int64 literal and a Float32 array still takes a streaming kernel.
static uint16_t float_to_half_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
    uint32_t man = x & 0x7fffffu;
    if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        const int shift = 14 - exp;
        uint32_t h = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1))) ++h;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((uint32_t)exp << 10) | (man >> 13);
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
    return (uint16_t)(sign | h);
}

static uint64_t convert_scalar_class(int src, int dst, uint64_t cls) {
    double d = 0;
    int64_t i = 0;
    uint64_t u = 0;
    const int sc = dtype_class(src), dc = dtype_class(dst);
    const bool src_float = sc == CF32 || sc == CF64;
    if (sc == CF32) { uint32_t b = (uint32_t)cls; float f; memcpy(&f, &b, 4); d = f; }
    else if (sc == CF64) memcpy(&d, &cls, 8);
    else if (sc == CI32) { i = (int32_t)(uint32_t)cls; u = (uint64_t)i; d = (double)i; }
    else if (sc == CI64) { i = (int64_t)cls; u = (uint64_t)i; d = (double)i; }
    else if (sc == CU32) { u = (uint32_t)cls; i = (int64_t)u; d = (double)u; }
    else { u = cls; i = (int64_t)u; d = (double)u; }
    if (src_float) { i = (int64_t)d; u = (uint64_t)i; }
    uint64_t out = 0;
    switch (dc) {
        case CF32: {
            float f = (sc == CF32 || sc == CF64) ? (float)d : (sc == CU64 ? (float)u : (float)i);
            if (dst == B200_F16) f = half_bits_to_float(float_to_half_bits(f));
            uint32_t b;
            memcpy(&b, &f, 4);
            if (dst == B200_BF16) {
                const uint32_t lsb = (b >> 16) & 1u;
                if ((b & 0x7f800000u) != 0x7f800000u) b += 0x7fffu + lsb;
                b &= 0xffff0000u;
            }
            out = b;
            break;
        }
        case CF64: { double v = src_float ? d : (sc == CU64 ? (double)u : (double)i); memcpy(&out, &v, 8); break; }
        case CI32: out = (uint32_t)(int32_t)i; break;
        case CI64: out = (uint64_t)i; break;
        case CU32: out = (uint32_t)u; break;
        default: out = u; break;
    }
    return scalar_to_class(dst, dst == B200_F16 || dst == B200_BF16 ? class_to_storage(dst, out) : out);
}

uint64_t class_to_storage(int32_t dt, uint64_t cls) {
    switch (dt) {
        case B200_F16: { uint32_t b = (uint32_t)cls; float f; memcpy(&f, &b, 4); return float_to_half_bits(f); }
        case B200_BF16: return (cls >> 16) & 0xffff;
        default: return cls;
    }
}

// ---- host: program validation ---------------------------------------------------------------------
int32_t compile_program(const int64_t* shape, int32_t ndim, const b200_leaf* leaves, int32_t nleaves,
                        const uint8_t* program, int32_t ninstr, int32_t final_dtype, Compiled* out) {
    if (ndim < 0 || ndim > B200_MAX_DIMS) return fail(B200_INVALID_ARG, "program: ndim %d outside [0,%d]", ndim, B200_MAX_DIMS);
    if (nleaves < 0 || nleaves > B200_MAX_LEAVES) return fail(B200_INVALID_ARG, "program: %d leaves (at most %d)", nleaves, B200_MAX_LEAVES);
    if (ninstr <= 0 || ninstr > B200_MAX_PROGRAM) return fail(B200_INVALID_ARG, "program: %d instructions (1..%d)", ninstr, B200_MAX_PROGRAM);
    if (!program || (nleaves > 0 && !leaves)) return fail(B200_INVALID_ARG, "program: null pointer");
    memset(out, 0, sizeof *out);
    ProgramDesc& P = out->P;
    P.ndim = ndim;
    P.nleaves = nleaves;
    int64_t numel = 1;
    for (int d = 0; d < ndim; ++d) { P.shape[d] = shape[d]; numel *= shape[d]; }
    bool linear = true, vec_ok = true;
    bool wide = false;
    for (int k = 0; k < nleaves; ++k) {
        const b200_leaf& lf = leaves[k];
        LeafDesc& L = P.leaves[k];
        if (dtype_size(lf.t.dtype) == 0) return fail(B200_UNSUPPORTED, "leaf %d: unknown dtype %d", k, lf.t.dtype);
        L.dtype = lf.t.dtype;
        L.is_scalar = lf.is_scalar ? 1 : 0;
        if (dtype_class(L.dtype) == CF64 || dtype_class(L.dtype) == CI64 || dtype_class(L.dtype) == CU64) wide = true;
        if (lf.is_scalar) {
            L.scalar = scalar_to_class(L.dtype, lf.scalar);
            continue;
        }
        B200_TRY(check_tensor(&lf.t, "broadcast leaf"));
        if (lf.t.ndim > ndim) return fail(B200_INVALID_ARG, "leaf %d has %d dims, index space has %d", k, lf.t.ndim, ndim);
        L.ptr = lf.t.ptr;
        int64_t expect = 1;
        bool dense = true;
        for (int d = 0; d < ndim; ++d) {
            int64_t e = d < lf.t.ndim ? lf.t.shape[d] : 1;
            int64_t s = d < lf.t.ndim ? lf.t.stride[d] : 0;
            if (e != shape[d] && e != 1) return fail(B200_INVALID_ARG, "leaf %d: extent %lld in dim %d does not broadcast to %lld", k, (long long)e, d, (long long)shape[d]);
            if (e == 1) s = 0;
            L.stride[d] = s;
            if (shape[d] != 1) { if (s != expect) dense = false; }
            expect *= shape[d];
        }
        out->n_array_leaves++;
        if (!dense) linear = false;
        if (reinterpret_cast<uintptr_t>(L.ptr) % (dtype_size(L.dtype) * kVec) != 0) vec_ok = false;
    }
    // abstract interpretation: stack of dtypes
    int32_t stack[kMaxStack + 1];
    int sp = 0;
    int nout = 0;
    auto emit = [&](int op, int arg) { P.code[2 * nout] = (uint8_t)op; P.code[2 * nout + 1] = (uint8_t)arg; ++nout; };
    for (int pc = 0; pc < ninstr; ++pc) {
        const int op = program[2 * pc], arg = program[2 * pc + 1];
        switch (op) {
            case B200_OP_LEAF:
                if (arg >= nleaves) return fail(B200_INVALID_ARG, "instruction %d: leaf %d does not exist", pc, arg);
                if (sp >= kMaxStack) return fail(B200_UNSUPPORTED, "program needs a value stack deeper than %d", kMaxStack);
                stack[sp++] = P.leaves[arg].dtype;
                emit(op, arg);
                break;
            case B200_OP_CONVERT: {
                if (sp < 1) return fail(B200_INVALID_ARG, "instruction %d: empty stack", pc);
                if (arg >= B200_DTYPE_COUNT) return fail(B200_UNSUPPORTED, "instruction %d: unknown dtype %d", pc, arg);
                const int src = stack[sp - 1];
                if (src != arg) {
                    // convert(T, scalar) is folded here: the scalar leaf is replaced by a converted copy
                    const bool prev_is_scalar_leaf = nout > 0 && P.code[2 * (nout - 1)] == B200_OP_LEAF &&
                                                     P.leaves[P.code[2 * (nout - 1) + 1]].is_scalar;
                    if (prev_is_scalar_leaf && P.nleaves < B200_MAX_LEAVES && arg != B200_BOOL) {
                        const LeafDesc& old = P.leaves[P.code[2 * (nout - 1) + 1]];
                        LeafDesc& nw = P.leaves[P.nleaves];
                        nw = LeafDesc{};
                        nw.dtype = arg;
                        nw.is_scalar = 1;
                        nw.scalar = convert_scalar_class(old.dtype, arg, old.scalar);
                        P.code[2 * (nout - 1) + 1] = (uint8_t)P.nleaves;
                        ++P.nleaves;
                        const int c = dtype_class(arg);
                        if (c == CF64 || c == CI64 || c == CU64) wide = true;
                    } else {
                        emit(op, (src << 4) | arg);
                    }
                }
                stack[sp - 1] = arg;
                break;
            }
            case B200_OP_ABS: case B200_OP_ABS2: case B200_OP_EXP: case B200_OP_NEG:
                if (sp < 1) return fail(B200_INVALID_ARG, "instruction %d: empty stack", pc);
                if (stack[sp - 1] != arg) return fail(B200_INVALID_ARG, "instruction %d: operand dtype %d differs from the instruction's %d", pc, stack[sp - 1], arg);
                if (op == B200_OP_EXP && !dtype_is_float(arg)) return fail(B200_UNSUPPORTED, "exp needs a floating-point operand");
                if (arg == B200_BOOL) return fail(B200_UNSUPPORTED, "arithmetic on Bool values must be converted first");
                emit(op, arg);
                break;
            case B200_OP_ADD: case B200_OP_SUB: case B200_OP_MUL: case B200_OP_DIV:
            case B200_OP_MAX: case B200_OP_MIN:
                if (sp < 2) return fail(B200_INVALID_ARG, "instruction %d: needs two operands", pc);
                if (stack[sp - 1] != arg || stack[sp - 2] != arg) return fail(B200_INVALID_ARG, "instruction %d: operand dtypes (%d,%d) differ from the instruction's %d", pc, stack[sp - 2], stack[sp - 1], arg);
                if (op == B200_OP_DIV && !dtype_is_float(arg)) return fail(B200_UNSUPPORTED, "/ needs floating-point operands (Base converts integers first)");
                if (arg == B200_BOOL) return fail(B200_UNSUPPORTED, "arithmetic on Bool values must be converted first");
                --sp;
                emit(op, arg);
                break;
            case B200_OP_MULADD:
                if (sp < 3) return fail(B200_INVALID_ARG, "instruction %d: needs three operands", pc);
                if (stack[sp - 1] != arg || stack[sp - 2] != arg || stack[sp - 3] != arg) return fail(B200_INVALID_ARG, "instruction %d: operand dtypes differ from the instruction's %d", pc, arg);
                if (arg == B200_BOOL) return fail(B200_UNSUPPORTED, "arithmetic on Bool values must be converted first");
                sp -= 2;
                emit(op, arg);
                break;
            default:
                return fail(B200_UNSUPPORTED, "instruction %d: unknown opcode %d", pc, op);
        }
        if (op != B200_OP_LEAF && arg < B200_DTYPE_COUNT) {
            int c = dtype_class(op == B200_OP_CONVERT ? arg : stack[sp - 1]);
            if (c == CF64 || c == CI64 || c == CU64) wide = true;
        }
    }
    if (sp != 1) return fail(B200_INVALID_ARG, "program leaves %d values on the stack (expected 1)", sp);
    if (final_dtype >= 0 && stack[0] != final_dtype) {
        if (final_dtype >= B200_DTYPE_COUNT) return fail(B200_UNSUPPORTED, "unknown result dtype %d", final_dtype);
        emit(B200_OP_CONVERT, (stack[0] << 4) | final_dtype);
        int c = dtype_class(final_dtype);
        if (c == CF64 || c == CI64 || c == CU64) wide = true;
        stack[0] = final_dtype;
    }
    // width of the evaluator: only what the final program really touches counts
    auto is_wide = [](int dt) { const int c = dtype_class(dt); return c == CF64 || c == CI64 || c == CU64; };
    wide = false;
    for (int pc = 0; pc < nout; ++pc) {
        const int o = P.code[2 * pc], a = P.code[2 * pc + 1];
        if (o == B200_OP_LEAF) wide = wide || is_wide(P.leaves[a].dtype);
        else if (o == B200_OP_CONVERT) wide = wide || is_wide(a >> 4) || is_wide(a & 15);
        else wide = wide || is_wide(a);
    }
    // device code: one handler number per instruction
    for (int pc = 0; pc < nout; ++pc) {
        const int o = P.code[2 * pc], a = P.code[2 * pc + 1];
        int h, arg = a;
        if (o == B200_OP_LEAF) h = (a < kPrefetch) ? kHPre0 + a : kHLeafMem;
        else if (o == B200_OP_CONVERT) h = kHConvert;
        else {
            h = kHOps + dtype_class(a) * kNumOps + (o - B200_OP_ADD);
            arg = dtype_is_narrow(a) ? a : 0xff;
        }
        P.hcode[2 * pc] = (uint8_t)h;
        P.hcode[2 * pc + 1] = (uint8_t)arg;
    }
    P.ninstr = nout;
    P.linear = linear ? 1 : 0;
    P.vec_ok = (linear && vec_ok) ? 1 : 0;
    out->result_dtype = stack[0];
    out->wide = wide;
    (void)numel;
    return B200_OK;
}

// ---- device: hard-wired streaming kernels --------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    using C = float;
    static __device__ __forceinline__ float up(float v) { return v; }
    static __device__ __forceinline__ float down(float v) { return v; }
    static __device__ __forceinline__ float rnd(float v) { return v; }
};
template <> struct Elem<double> {
    using C = double;
    static __device__ __forceinline__ double up(double v) { return v; }
    static __device__ __forceinline__ double down(double v) { return v; }
    static __device__ __forceinline__ double rnd(double v) { return v; }
};
template <> struct Elem<__half> {
    using C = float;
    static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ float rnd(float v) { return __half2float(__float2half_rn(v)); }
};
template <> struct Elem<__nv_bfloat16> {
    using C = float;
    static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float rnd(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

template <> struct Elem<int32_t> {
    using C = int32_t;
    static __device__ __forceinline__ int32_t up(int32_t v) { return v; }
    static __device__ __forceinline__ int32_t down(int32_t v) { return v; }
    static __device__ __forceinline__ int32_t rnd(int32_t v) { return v; }
};
template <> struct Elem<int64_t> {
    using C = int64_t;
    static __device__ __forceinline__ int64_t up(int64_t v) { return v; }
    static __device__ __forceinline__ int64_t down(int64_t v) { return v; }
    static __device__ __forceinline__ int64_t rnd(int64_t v) { return v; }
};

// One operator of the fixed set applied to arrays and at most one scalar: f(x), x o y, x o s,
// s o x.  The operator is a run-time value; it is switched on once per 16-byte vector.
enum { MODE_UNARY = 0, MODE_AA = 1, MODE_AS = 2, MODE_SA = 3 };
template <typename T>
struct OneOpF {
    int op, mode;
    typename Elem<T>::C s;
    template <int V>
    __device__ __forceinline__ Vec<T, V> vec(const Vec<T, V>& a, const Vec<T, V>& b) const {
        using E = Elem<T>;
        using C = typename E::C;
        using A = Arith<C>;
        Vec<T, V> r;
#define B200_EW(EXPR)                                                         \
    _Pragma("unroll") for (int k = 0; k < V; ++k) {                           \
        const C x = (mode == MODE_SA) ? s : E::up(a.v[k]);                    \
        const C y = (mode == MODE_AS) ? s : (mode == MODE_SA ? E::up(a.v[k]) : E::up(b.v[k])); \
        (void)y;                                                              \
        r.v[k] = E::down(EXPR);                                               \
    }                                                                         \
    break;
        switch (op) {
            case B200_OP_ADD: B200_EW(A::add(x, y))
            case B200_OP_SUB: B200_EW(A::sub(x, y))
            case B200_OP_MUL: B200_EW(A::mul(x, y))
            case B200_OP_DIV: B200_EW(A::div(x, y))
            case B200_OP_MAX: B200_EW(A::max(x, y))
            case B200_OP_MIN: B200_EW(A::min(x, y))
            case B200_OP_ABS: B200_EW(A::abs(x))
            case B200_OP_ABS2: B200_EW(E::rnd(A::mul(x, x)))
            case B200_OP_EXP: B200_EW(A::exp(x))
            case B200_OP_NEG: B200_EW(A::neg(x))
            default: r = a; break;
        }
#undef B200_EW
        return r;
    }
    __device__ __forceinline__ T operator()(T x, T y, T) const {
        Vec<T, 1> a{{x}}, b{{y}};
        return vec<1>(a, b).v[0];
    }
};

// z = a*x + y, multiply and add rounded separately (Base does not contract `a .* x .+ y`).
template <typename T>
struct AxpyF {
    typename Elem<T>::C a;
    __device__ __forceinline__ T operator()(T x, T y, T) const {
        using E = Elem<T>;
        using A = Arith<typename E::C>;
        typename E::C p = E::rnd(A::mul(a, E::up(x)));
        return E::down(A::add(p, E::up(y)));
    }
};
// r = x*y + exp(-abs(z))
template <typename T>
struct MulAddExpNegAbsF {
    __device__ __forceinline__ T operator()(T x, T y, T z) const {
        using E = Elem<T>;
        using A = Arith<typename E::C>;
        typename E::C p = E::rnd(A::mul(E::up(x), E::up(y)));
        typename E::C e = E::rnd(A::exp(A::neg(A::abs(E::up(z)))));
        return E::down(A::add(p, e));
    }
};

template <typename F, typename = void> struct HasVec : std::false_type {};
template <typename T> struct HasVec<OneOpF<T>, void> : std::true_type {};

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;

template <typename T, typename F, int NIN>
__global__ void __launch_bounds__(kEwThreads)
ew_stream_kernel(T* out, const T* in0, const T* in1, const T* in2, F f, int64_t n, int vec_ok) {
    constexpr int V = 16 / sizeof(T);
    constexpr int64_t TILE = (int64_t)kEwThreads * kEwUnroll * V;
    const int64_t ntiles = (n + TILE - 1) / TILE;
    using VT = Vec<T, V>;
    grid_dependency_wait();
    grid_dependency_release();
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int64_t base = tile * TILE;
        if (vec_ok && base + TILE <= n) {
            VT a[kEwUnroll], b[kEwUnroll], c[kEwUnroll];
#pragma unroll
            for (int u = 0; u < kEwUnroll; ++u) {
                const int64_t vi = base / V + (int64_t)u * kEwThreads + threadIdx.x;
                a[u] = __builtin_bit_cast(VT, __ldcs(reinterpret_cast<const uint4*>(in0) + vi));
                if (NIN > 1) b[u] = __builtin_bit_cast(VT, __ldcs(reinterpret_cast<const uint4*>(in1) + vi));
                if (NIN > 2) c[u] = __builtin_bit_cast(VT, __ldcs(reinterpret_cast<const uint4*>(in2) + vi));
            }
#pragma unroll
            for (int u = 0; u < kEwUnroll; ++u) {
                const int64_t vi = base / V + (int64_t)u * kEwThreads + threadIdx.x;
                VT r;
                if constexpr (HasVec<F>::value) {
                    r = f.template vec<V>(a[u], NIN > 1 ? b[u] : a[u]);
                } else {
#pragma unroll
                    for (int k = 0; k < V; ++k)
                        r.v[k] = f(a[u].v[k], NIN > 1 ? b[u].v[k] : a[u].v[k], NIN > 2 ? c[u].v[k] : a[u].v[k]);
                }
                __stcs(reinterpret_cast<uint4*>(out) + vi, __builtin_bit_cast(uint4, r));
            }
        } else {
            const int64_t end = base + TILE < n ? base + TILE : n;
            for (int64_t i = base + threadIdx.x; i < end; i += kEwThreads) {
                T x = in0[i];
                T y = NIN > 1 ? in1[i] : x;
                T z = NIN > 2 ? in2[i] : x;
                out[i] = f(x, y, z);
            }
        }
    }
}

template <typename T, typename F, int NIN>
static void launch_stream(b200_stream_t st, void* out, const void* a, const void* b, const void* c, F f, int64_t n) {
    constexpr int V = 16 / sizeof(T);
    const int64_t TILE = (int64_t)kEwThreads * kEwUnroll * V;
    const int64_t tiles = (n + TILE - 1) / TILE;
    // One tile per block and the hardware block scheduler, not a persistent wave: blocks that
    // start as others retire spread reads and writes evenly over time, where a resident wave moves
    // in lock step (all loading, then all storing).  Measured on B200: 30.9 us against 34.7 us at
    // 2^24 Float32 (axpy), 2.40 ms against 2.49 ms at 2^30 (three inputs).
    const unsigned grid = (unsigned)(tiles < 1 ? 1 : (tiles > 0x7fffffff ? 0x7fffffff : tiles));
    auto al = [](const void* p) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    int vec_ok = al(out) && al(a) && al(b) && al(c);
    launch_overlapped(ew_stream_kernel<T, F, NIN>, grid, kEwThreads, 0, st->s,
                      (T*)out, (const T*)a, (const T*)b, (const T*)c, f, n, vec_ok);
}

// ---- host: pattern matching on the compiled program ----------------------------------------------------
struct Node { int op, arg, kid[3], nk; };

static int build_tree(const ProgramDesc& P, std::vector<Node>& nodes) {
    std::vector<int> stk;
    for (int pc = 0; pc < P.ninstr; ++pc) {
        Node nd{P.code[2 * pc], P.code[2 * pc + 1], {-1, -1, -1}, 0};
        int need = 0;
        switch (nd.op) {
            case B200_OP_LEAF: need = 0; break;
            case B200_OP_CONVERT: case B200_OP_ABS: case B200_OP_ABS2: case B200_OP_EXP: case B200_OP_NEG: need = 1; break;
            case B200_OP_MULADD: need = 3; break;
            default: need = 2; break;
        }
        for (int k = need - 1; k >= 0; --k) { nd.kid[k] = stk.back(); stk.pop_back(); }
        nd.nk = need;
        nodes.push_back(nd);
        stk.push_back((int)nodes.size() - 1);
    }
    return stk.back();
}

template <typename T>
static typename Elem<T>::C scalar_as(uint64_t cls) {
    using C = typename Elem<T>::C;
    if constexpr (std::is_same<C, float>::value) { uint32_t u = (uint32_t)cls; float f; memcpy(&f, &u, 4); return f; }
    else if constexpr (std::is_same<C, double>::value) { double d; memcpy(&d, &cls, 8); return d; }
    else if constexpr (std::is_same<C, int32_t>::value) return (int32_t)(uint32_t)cls;
    else return (int64_t)cls;
}

template <typename T>
static bool try_fixed(b200_stream_t st, const Compiled& C, const std::vector<Node>& N, int root, void* out, int64_t n) {
    const ProgramDesc& P = C.P;
    auto is_arr = [&](int i) { return i >= 0 && N[i].op == B200_OP_LEAF && !P.leaves[N[i].arg].is_scalar; };
    auto is_sc = [&](int i) { return i >= 0 && N[i].op == B200_OP_LEAF && P.leaves[N[i].arg].is_scalar; };
    auto ptr = [&](int i) { return P.leaves[N[i].arg].ptr; };
    const Node& r = N[root];
    // one operator over arrays and at most one scalar
    if (r.nk == 1 && r.op != B200_OP_CONVERT && is_arr(r.kid[0])) {
        if (r.op == B200_OP_EXP && !std::is_floating_point<typename Elem<T>::C>::value) return false;
        OneOpF<T> f{r.op, MODE_UNARY, typename Elem<T>::C(0)};
        launch_stream<T, OneOpF<T>, 1>(st, out, ptr(r.kid[0]), nullptr, nullptr, f, n);
        return true;
    }
    if (r.nk == 2) {
        const int p = r.kid[0], q = r.kid[1];
        if (r.op == B200_OP_DIV && !std::is_floating_point<typename Elem<T>::C>::value) return false;
        if (is_arr(p) && is_arr(q)) {
            OneOpF<T> f{r.op, MODE_AA, typename Elem<T>::C(0)};
            launch_stream<T, OneOpF<T>, 2>(st, out, ptr(p), ptr(q), nullptr, f, n);
            return true;
        }
        if (is_arr(p) && is_sc(q)) {
            OneOpF<T> f{r.op, MODE_AS, scalar_as<T>(P.leaves[N[q].arg].scalar)};
            launch_stream<T, OneOpF<T>, 1>(st, out, ptr(p), nullptr, nullptr, f, n);
            return true;
        }
        if (is_sc(p) && is_arr(q)) {
            OneOpF<T> f{r.op, MODE_SA, scalar_as<T>(P.leaves[N[p].arg].scalar)};
            launch_stream<T, OneOpF<T>, 1>(st, out, ptr(q), nullptr, nullptr, f, n);
            return true;
        }
    }
    if (!std::is_floating_point<typename Elem<T>::C>::value) return false;
    if (r.op != B200_OP_ADD) return false;
    for (int side = 0; side < 2; ++side) {
        const int m = r.kid[side], o = r.kid[1 - side];
        if (m < 0 || N[m].op != B200_OP_MUL) continue;
        const int p = N[m].kid[0], q = N[m].kid[1];
        // a*x + y
        if (is_arr(o) && ((is_sc(p) && is_arr(q)) || (is_arr(p) && is_sc(q)))) {
            const int s = is_sc(p) ? p : q, x = is_sc(p) ? q : p;
            AxpyF<T> f{scalar_as<T>(P.leaves[N[s].arg].scalar)};
            launch_stream<T, AxpyF<T>, 2>(st, out, ptr(x), ptr(o), nullptr, f, n);
            return true;
        }
        // x*y + exp(-abs(z))
        if (is_arr(p) && is_arr(q) && N[o].op == B200_OP_EXP) {
            const int ng = N[o].kid[0];
            if (N[ng].op != B200_OP_NEG) continue;
            const int ab = N[ng].kid[0];
            if (N[ab].op != B200_OP_ABS || !is_arr(N[ab].kid[0])) continue;
            launch_stream<T, MulAddExpNegAbsF<T>, 3>(st, out, ptr(p), ptr(q), ptr(N[ab].kid[0]), MulAddExpNegAbsF<T>{}, n);
            return true;
        }
    }
    return false;
}

// ---- permuted operands ------------------------------------------------------------------------------------
// An operand whose unit-stride dimension is not the first long dimension of the index space (a
// transposed matrix, a PermutedDimsArray) would be read across its lines - 32 bytes fetched per
// element used.  Such operands are copied into dense form first, through shared-memory tiles over
// the pair (a, b): a = first long dimension of the index space (unit stride in the copy),
// b = the operand's own unit-stride dimension.  Reads run along b, writes along a, both in whole
// lines; all other dimensions are batch.  One tile per block.
struct PermutePlan {
    int32_t ndim, a, b;
    int64_t shape[B200_MAX_DIMS];
    int64_t sstride[B200_MAX_DIMS];     // operand strides (elements); sstride[b] == 1
    int64_t dstride[B200_MAX_DIMS];     // dense strides of the copy; dstride[a] == 1
    int64_t tiles_a, tiles_b, nbatch;
};

template <typename E, int TILE>
__global__ void __launch_bounds__(256) permute_copy_kernel(E* dst, const E* src, const __grid_constant__ PermutePlan pl) {
    __shared__ E tile[TILE][TILE + 1];
    constexpr int ROWS = 256 / TILE;
    const int tx = threadIdx.x % TILE, ty = threadIdx.x / TILE;
    const int64_t m = pl.shape[pl.a], n = pl.shape[pl.b];
    const int64_t sa = pl.sstride[pl.a], db = pl.dstride[pl.b];
    const int64_t per_batch = pl.tiles_a * pl.tiles_b;
    grid_dependency_wait();
    for (int64_t t = blockIdx.x; t < per_batch * pl.nbatch; t += gridDim.x) {
        int64_t batch = t / per_batch;
        const int64_t in_batch = t - batch * per_batch;
        const int64_t i0 = (in_batch % pl.tiles_a) * TILE, j0 = (in_batch / pl.tiles_a) * TILE;
        int64_t soff = 0, doff = 0;
        for (int d = 0; d < pl.ndim; ++d) {
            if (d == pl.a || d == pl.b) continue;
            const int64_t e = pl.shape[d];
            const int64_t q = batch / e;
            const int64_t c = batch - q * e;
            soff += c * pl.sstride[d];
            doff += c * pl.dstride[d];
            batch = q;
        }
#pragma unroll
        for (int r = ty; r < TILE; r += ROWS) {
            const int64_t i = i0 + r, j = j0 + tx;
            if (i < m && j < n) tile[r][tx] = src[soff + i * sa + j];
        }
        __syncthreads();
#pragma unroll
        for (int r = ty; r < TILE; r += ROWS) {
            const int64_t i = i0 + tx, j = j0 + r;
            if (i < m && j < n) dst[doff + i + j * db] = tile[tx][r];
        }
        __syncthreads();
    }
}

// Does `t`, seen in the index space `shape`, call for the tiled copy?  It must cover the index
// space (no broadcast along a long dimension), its unit-stride dimension b must differ from the
// first long dimension a, and both must be long enough for tiles to pay.
static bool permuted_operand(const b200_tensor& t, const int64_t* shape, int32_t ndim, PermutePlan* pl) {
    int a = -1, b = -1;
    int64_t numel = 1;
    for (int d = 0; d < ndim; ++d) {
        if (shape[d] <= 1) continue;
        if (d >= t.ndim || t.shape[d] != shape[d] || t.stride[d] == 0) return false;
        if (a < 0) a = d;
        if (t.stride[d] == 1 && b < 0) b = d;
        numel *= shape[d];
    }
    if (a < 0 || b < 0 || a == b || t.stride[a] == 1) return false;
    if (shape[a] < 8 || shape[b] < 8 || numel < (1 << 14)) return false;
    *pl = PermutePlan{};
    pl->ndim = ndim; pl->a = a; pl->b = b;
    int64_t expect = 1;
    pl->nbatch = 1;
    for (int d = 0; d < ndim; ++d) {
        pl->shape[d] = shape[d];
        pl->sstride[d] = (d < t.ndim && shape[d] > 1) ? t.stride[d] : 0;
        pl->dstride[d] = expect;
        expect *= shape[d];
        if (d != a && d != b) pl->nbatch *= shape[d];
    }
    return true;
}

static void launch_permute_copy(b200_stream_t st, void* dst, const void* src, int bytes, PermutePlan pl) {
    const int tile = bytes == 8 ? 32 : 64;
    pl.tiles_a = (pl.shape[pl.a] + tile - 1) / tile;
    pl.tiles_b = (pl.shape[pl.b] + tile - 1) / tile;
    const int64_t tiles = pl.tiles_a * pl.tiles_b * pl.nbatch;
    const unsigned grid = (unsigned)(tiles > 0x7fffffff ? 0x7fffffff : tiles);
    switch (bytes) {
        case 1: launch_overlapped(permute_copy_kernel<uint8_t, 64>, grid, 256, 0, st->s, (uint8_t*)dst, (const uint8_t*)src, pl); break;
        case 2: launch_overlapped(permute_copy_kernel<uint16_t, 64>, grid, 256, 0, st->s, (uint16_t*)dst, (const uint16_t*)src, pl); break;
        case 4: launch_overlapped(permute_copy_kernel<uint32_t, 64>, grid, 256, 0, st->s, (uint32_t*)dst, (const uint32_t*)src, pl); break;
        default: launch_overlapped(permute_copy_kernel<uint64_t, 32>, grid, 256, 0, st->s, (uint64_t*)dst, (const uint64_t*)src, pl); break;
    }
}

// Byte range [lo, hi) an operand with these strides touches.
static void operand_span(const b200_tensor& t, const PermutePlan& pl, uintptr_t* lo, uintptr_t* hi) {
    int64_t last = 0;
    for (int d = 0; d < pl.ndim; ++d) if (pl.shape[d] > 1) last += (pl.shape[d] - 1) * pl.sstride[d];
    *lo = reinterpret_cast<uintptr_t>(t.ptr);
    *hi = *lo + (size_t)(last + 1) * dtype_size(t.dtype);
}

// `fixed` receives the leaves to use: permuted operands replaced by dense copies in the stream's
// scratch.  Without room for the copies the leaves stay as they are (the strided path works).
// With `pool_temp` the copies live in one stream-ordered pool allocation that the caller frees on the
// stream after its launches (for operators that use the stream's scratch themselves).
int32_t densify_permuted_leaves(b200_stream_t st, const int64_t* shape, int32_t ndim, const b200_leaf* leaves,
                                int32_t nleaves, b200_leaf* fixed, void** pool_temp) {
    size_t total = 0;
    PermutePlan plan[B200_MAX_LEAVES];
    bool take[B200_MAX_LEAVES];
    int64_t numel = 1;
    for (int d = 0; d < ndim; ++d) numel *= shape[d];
    for (int k = 0; k < nleaves; ++k) {
        fixed[k] = leaves[k];
        take[k] = !leaves[k].is_scalar && leaves[k].t.ptr && dtype_size(leaves[k].t.dtype) > 0 &&
                  permuted_operand(leaves[k].t, shape, ndim, &plan[k]);
        if (take[k]) total += ((size_t)numel * dtype_size(leaves[k].t.dtype) + 255) / 256 * 256;
    }
    if (total == 0) return B200_OK;
    void* scr = nullptr;
    if (pool_temp) {
        if (b200_malloc_async(&scr, total, st) != B200_OK) return B200_OK;
        *pool_temp = scr;
    } else if (scratch(st, total, &scr) != B200_OK) {
        return B200_OK;
    }
    unsigned char* p = reinterpret_cast<unsigned char*>(scr);
    for (int k = 0; k < nleaves; ++k) {
        if (!take[k]) continue;
        const b200_tensor& t = leaves[k].t;
        const int bytes = (int)dtype_size(t.dtype);
        launch_permute_copy(st, p, t.ptr, bytes, plan[k]);
        fixed[k].t.ptr = p;
        fixed[k].t.ndim = ndim;
        for (int d = 0; d < ndim; ++d) { fixed[k].t.shape[d] = shape[d]; fixed[k].t.stride[d] = plan[k].dstride[d]; }
        p += ((size_t)numel * bytes + 255) / 256 * 256;
    }
    return B200_OK;
}

}  // namespace b200

using namespace b200;

// Destination descriptor and the layout flags that depend on it.
static void destination_layout(const b200_tensor* out, Compiled* C, LeafDesc* O) {
    O->ptr = out->ptr;
    O->dtype = out->dtype;
    for (int d = 0; d < out->ndim; ++d) O->stride[d] = out->shape[d] == 1 ? 0 : out->stride[d];
    if (!tensor_is_contiguous(out)) C->P.linear = 0;
    if (!C->P.linear || reinterpret_cast<uintptr_t>(out->ptr) % (dtype_size(out->dtype) * kVec) != 0) C->P.vec_ok = 0;
}

extern "C" int32_t b200_broadcast_prepare(const b200_tensor* out, const b200_leaf* leaves, int32_t nleaves,
                                          const uint8_t* program, int32_t ninstr) {
    B200_TRY(check_tensor(out, "broadcast destination"));
    Compiled C;
    B200_TRY(compile_program(out->shape, out->ndim, leaves, nleaves, program, ninstr, out->dtype, &C));
    LeafDesc O{};
    destination_layout(out, &C, &O);
    return jit_prepare(C, out->dtype);
}

extern "C" int32_t b200_broadcast(b200_stream_t st, const b200_tensor* out, const b200_leaf* leaves,
                                  int32_t nleaves, const uint8_t* program, int32_t ninstr) {
    B200_TRY(enter(st));
    StreamGuard guard(st);
    B200_TRY(check_tensor(out, "broadcast destination"));
    const int64_t n = tensor_numel(out);
    Compiled C;
    B200_TRY(compile_program(out->shape, out->ndim, leaves, nleaves, program, ninstr, out->dtype, &C));
    if (n == 0) return B200_OK;
    if (!C.P.linear && leaves && nleaves > 0 && nleaves <= B200_MAX_LEAVES) {
        // a plain copy of a permuted operand goes straight into a dense destination
        PermutePlan pp;
        if (ninstr == 1 && program[0] == B200_OP_LEAF && !leaves[program[1]].is_scalar && leaves[program[1]].t.dtype == out->dtype &&
            tensor_is_contiguous(out) && permuted_operand(leaves[program[1]].t, out->shape, out->ndim, &pp)) {
            const b200_tensor& src = leaves[program[1]].t;
            uintptr_t s0, s1;
            operand_span(src, pp, &s0, &s1);
            const uintptr_t o0 = reinterpret_cast<uintptr_t>(out->ptr), o1 = o0 + (size_t)n * dtype_size(out->dtype);
            if (s1 <= o0 || o1 <= s0) {           // source and destination apart (A .= A' goes through the copy below)
                launch_permute_copy(st, out->ptr, src.ptr, (int)dtype_size(src.dtype), pp);
                return finish(st, "b200_broadcast");
            }
        }
        b200_leaf fixed[B200_MAX_LEAVES];
        B200_TRY(densify_permuted_leaves(st, out->shape, out->ndim, leaves, nleaves, fixed, nullptr));
        B200_TRY(compile_program(out->shape, out->ndim, fixed, nleaves, program, ninstr, out->dtype, &C));
    }
    for (int d = 0; d < out->ndim; ++d)
        if (out->shape[d] > 1 && out->stride[d] == 0) return fail(B200_INVALID_ARG, "broadcast destination has a zero stride");

    LeafDesc O{};
    destination_layout(out, &C, &O);

    // Hard-wired kernels: every array leaf dense, same dtype as the destination, no conversions.
    if (C.P.linear) {
        bool uniform = true;
        for (int pc = 0; pc < C.P.ninstr; ++pc) {
            if (C.P.code[2 * pc] == B200_OP_CONVERT) uniform = false;
            if (C.P.code[2 * pc] == B200_OP_LEAF && C.P.leaves[C.P.code[2 * pc + 1]].dtype != out->dtype) uniform = false;
        }
        if (uniform) {
            std::vector<Node> nodes;
            int root = build_tree(C.P, nodes);
            bool done = false;
            switch (out->dtype) {
                case B200_F32: done = try_fixed<float>(st, C, nodes, root, out->ptr, n); break;
                case B200_F64: done = try_fixed<double>(st, C, nodes, root, out->ptr, n); break;
                case B200_F16: done = try_fixed<__half>(st, C, nodes, root, out->ptr, n); break;
                case B200_BF16: done = try_fixed<__nv_bfloat16>(st, C, nodes, root, out->ptr, n); break;
                case B200_I32: done = try_fixed<int32_t>(st, C, nodes, root, out->ptr, n); break;
                case B200_I64: done = try_fixed<int64_t>(st, C, nodes, root, out->ptr, n); break;
                default: break;
            }
            if (done) return finish(st, "b200_broadcast");
        }
    }

    // any other tree: the evaluator specialised for this expression at run time if possible,
    // else the interpreter
    const int specialised = jit_broadcast(st, C, O, n);
    if (specialised > 0) return finish(st, "b200_broadcast");
    if (specialised < 0)
        return fail(B200_UNSUPPORTED, "first use of this broadcast expression inside a stream capture: its kernel has to "
                    "be compiled and loaded, run the expression once before capturing");
    const int64_t nvec = (n + kVec - 1) / kVec;
    const int64_t chunks = (nvec + 255) / 256;
    if (C.wide) ew_program_kernel<true><<<balanced_grid(chunks, resident_blocks(ew_program_kernel<true>, 256, 0, st->dev)), 256, 0, st->s>>>(C.P, O, n);
    else ew_program_kernel<false><<<balanced_grid(chunks, resident_blocks(ew_program_kernel<false>, 256, 0, st->dev)), 256, 0, st->s>>>(C.P, O, n);
    return finish(st, "b200_broadcast");
}
