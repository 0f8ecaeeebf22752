// Internal declarations shared by the translation units of libb200arrays.so.
#pragma once

// Under run-time compilation (NVRTC, which defines __CUDACC_RTC__) only the device-side half of
// this header is seen: the specialised broadcast kernels are built from the very same sources.
#ifndef __CUDACC_RTC__
#include <cuda_runtime.h>
#endif
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>
#ifndef __CUDACC_RTC__
#include <mutex>
#include <string>
#include <vector>
#endif

#include "../../include/b200arrays.h"

#ifndef __CUDACC_RTC__
// ---- host-side handles ---------------------------------------------------------------------
struct b200_stream_s {
    int          dev;
    cudaStream_t s;
    bool         owned;
    // Scratch owned by the stream: operators launched on one stream run in order, so one
    // buffer per stream can be reused by every call without extra synchronisation.
    void*        scratch;
    size_t       scratch_bytes;
    // A captured graph keeps the scratch address it saw: once an operator asked for scratch
    // during a capture the buffer is never freed while the stream lives (it moves to `retired`
    // if a later call needs a larger one).
    bool         scratch_in_graph;
    std::vector<void*> retired;
    // Descriptor words of the one-pass scan: a buffer that only that kernel writes, every word
    // tagged with the number of the launch that wrote it (`scan_epoch`), so that words left by
    // earlier launches read as "empty" and no launch has to clear them first.
    void*        scan_state = nullptr;
    size_t       scan_state_bytes = 0;
    uint32_t     scan_epoch = 0;
    bool         scan_state_in_graph = false;
    // Serialises host threads that issue operators on this stream: scratch handed to one call
    // must stay valid until that call has enqueued its kernels.
    std::recursive_mutex mu;
};

// Held by an operator from validation to its last launch.
struct StreamGuard {
    explicit StreamGuard(b200_stream_t st) : lk(st->mu) {}
    std::lock_guard<std::recursive_mutex> lk;
};

struct b200_event_s {
    int         dev;
    cudaEvent_t e;
};

// Peer exchange for fused reduce + all-reduce (one process per GPU): every rank owns a small
// buffer of slots that all ranks can write over NVLink; `bufs[r]` is rank r's buffer as mapped
// into THIS process (own buffer for r == rank).
constexpr int kMaxPeers = 8;
struct PeerSlot {
    unsigned long long value;    // accumulator bits
    unsigned long long seq;      // sequence number of the collective that wrote `value`
};
struct PeerCtx {
    int32_t   nranks;            // 0: no exchange, plain local result
    int32_t   rank;
    uint64_t  seq;               // this collective's number (1, 2, ...); parity selects the slot bank
    uint32_t  max_polls;
    int32_t*  err_word;
    PeerSlot* bufs[kMaxPeers];   // each: [2 banks][kMaxPeers] slots
};

namespace b200 {

// Thread-local error text; returns `code` so call sites can `return fail(...)`.
int32_t fail(int32_t code, const char* fmt, ...);
int32_t cuda_fail(cudaError_t e, const char* what);

#define B200_CUDA(expr)                                                  \
    do {                                                                 \
        cudaError_t _e = (expr);                                         \
        if (_e != cudaSuccess) return ::b200::cuda_fail(_e, #expr);      \
    } while (0)

#define B200_TRY(expr)                                                   \
    do {                                                                 \
        int32_t _s = (expr);                                             \
        if (_s != B200_OK) return _s;                                    \
    } while (0)

// Makes the stream's device current; validates the handle.
int32_t enter(b200_stream_t st);
// Returns at least `bytes` of stream-owned scratch (256-byte aligned).  The first
// kCounterBytes of every scratch buffer hold ticket counters that are zero between kernels
// (the last block to take a ticket resets it); `counters` receives that region.
constexpr size_t kCounterBytes = 64 * 1024;
int32_t scratch(b200_stream_t st, size_t bytes, void** out, unsigned int** counters = nullptr);
// Descriptor storage for the one-pass scan (see b200_stream_s::scan_state): at least `bytes` after
// a 256-byte header whose first word is the tile ticket (zero between launches).  `epoch` receives
// this launch's tag (1 .. 2^30-1).  `*must_clear` is set when the stream is being captured: a
// replayed graph repeats its tag, so such a launch clears header and descriptors itself first.
constexpr size_t kScanStateHeader = 256;
int32_t scan_state(b200_stream_t st, size_t bytes, void** out, uint32_t* epoch, bool* must_clear);
// One line per operator call on stderr when the environment has B200_LOG=debug.
void log_debug(const char* fmt, ...);
// Device pointer of this device's latched error word (kernels store a status code there).
int32_t* device_error_word(int dev);
// Called by every operator after its launches: launch-error check + optional blocking mode.
int32_t finish(b200_stream_t st, const char* what);
int sm_count(int dev);

// Blocks per SM of a kernel as the occupancy calculator gives them, remembered per (kernel, block
// size, dynamic shared memory, device): the query costs about a microsecond, a fifth of the host
// side of a small operator call.
int cached_blocks_per_sm(const void* kernel, int threads, size_t dyn_smem, int dev);
// Blocks of `kernel` that the whole device keeps resident at once (SMs x blocks per SM).
template <typename Kernel>
inline int64_t resident_blocks(Kernel kernel, int threads, size_t dyn_smem, int dev) {
    return (int64_t)cached_blocks_per_sm(reinterpret_cast<const void*>(kernel), threads, dyn_smem, dev) * sm_count(dev);
}
// Grid for a block-stride loop over `items` equal work items: every block runs the same number
// of iterations (up to rounding) and all blocks are resident together - no partly filled wave.
inline unsigned balanced_grid(int64_t items, int64_t resident) {
    if (items <= 0) return 1;
    const int64_t iters = (items + resident - 1) / resident;
    return (unsigned)((items + iters - 1) / iters);
}

// Launch that may overlap the tail of the kernel in front of it on the same stream (programmatic
// dependent launch): the blocks of this kernel are placed on SMs as the earlier kernel's blocks
// retire and wait in grid_dependency_wait() - which MUST be the kernel's first statement - until
// that kernel has completed and its writes are visible.  Saves the launch gap between dependent
// kernels, which is a tenth of the run time of a 64 MiB operator.  B200_OVERLAP_LAUNCHES=0 in the
// environment turns it off (plain stream order).
bool overlap_launches_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t dyn_smem, cudaStream_t s,
                                     Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = dyn_smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = overlap_launches_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel known only by handle (run-time compiled code), arguments as an array.
inline cudaError_t launch_overlapped_handle(const void* kernel, unsigned grid, unsigned block, void** args, cudaStream_t s) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = overlap_launches_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelExC(&cfg, kernel, args);
}

inline size_t dtype_size(int32_t dt) {
    switch (dt) {
        case B200_F16: case B200_BF16: case B200_I16: case B200_U16: return 2;
        case B200_F32: case B200_I32: case B200_U32: return 4;
        case B200_F64: case B200_I64: case B200_U64: return 8;
        case B200_I8: case B200_U8: case B200_BOOL: return 1;
        default: return 0;
    }
}
inline bool dtype_is_float(int32_t dt) { return dt >= B200_F16 && dt <= B200_F64; }
inline bool dtype_is_signed_int(int32_t dt) { return dt >= B200_I8 && dt <= B200_I64; }
inline bool dtype_is_unsigned_int(int32_t dt) { return dt >= B200_U8 && dt <= B200_BOOL; }

inline int64_t tensor_numel(const b200_tensor* t) {
    int64_t n = 1;
    for (int d = 0; d < t->ndim; ++d) n *= t->shape[d];
    return n;
}
// Dense column-major (stride[0]==1, stride[d]==stride[d-1]*shape[d-1]); extents of 1 are free.
inline bool tensor_is_contiguous(const b200_tensor* t) {
    int64_t expect = 1;
    for (int d = 0; d < t->ndim; ++d) {
        if (t->shape[d] != 1 && t->stride[d] != expect) return false;
        expect *= t->shape[d];
    }
    return true;
}
int32_t check_tensor(const b200_tensor* t, const char* name);
// Fills the kernel-side view of a peer group for its next collective (advances the sequence).
int32_t peer_next_context(b200_peer_t peer, b200_stream_t st, PeerCtx* out);

}  // namespace b200
#endif  // !__CUDACC_RTC__

// ---- device-side helpers --------------------------------------------------------------------
#ifdef __CUDACC__
namespace b200 {

// Device side of launch_overlapped: nothing of the kernel may touch global memory before the wait;
// the second call lets the NEXT kernel's blocks take the SM slots this grid frees as it drains.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 16-byte vector of T for 128-bit global accesses.
template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
    T v[N];
};

// Streaming global accesses: inputs are read once, outputs written once.
template <typename V>
__device__ __forceinline__ V ld_stream(const V* p) {
    return __ldcs(p);
}
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    return __ldcs(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void st_stream16(void* p, uint4 v) {
    __stcs(reinterpret_cast<uint4*>(p), v);
}

// L2 residency control for data that is read twice: the first read asks L2 to keep the lines
// (evict-last), the second read and all streaming stores mark theirs evict-first.
__device__ __forceinline__ uint64_t l2_policy_keep() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_stream() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint4 ld_policy16(const uint4* ptr, uint64_t policy) {
    uint4 v;
    asm volatile("ld.global.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr), "l"(policy));
    return v;
}
__device__ __forceinline__ void st_policy16(uint4* ptr, uint4 v, uint64_t policy) {
    asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;"
                 ::"l"(ptr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(policy) : "memory");
}

// 16-byte asynchronous copy global -> shared (bypasses registers and L1), grouped by commit/wait.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async16_policy(void* smem_dst, const void* gmem_src, uint64_t policy) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem_src), "l"(policy) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Records a device-side failure in the device's latched error word (pinned host memory that
// the host inspects at the next synchronisation).  Spinning kernels poll it on their slow
// path so that one timed-out wait ends every other wait quickly.
__device__ __forceinline__ void latch_error(int32_t* word, int32_t code) {
    *(volatile int32_t*)word = code;
    __threadfence_system();
}
__device__ __forceinline__ bool error_latched(const int32_t* word) {
    return *(volatile const int32_t*)word != 0;
}

// Julia Base.max/min on floats: NaN wins, -0.0 orders below +0.0.
template <typename F>
__device__ __forceinline__ F jl_max(F a, F b) {
    if (a != a) return a;
    if (b != b) return b;
    if (a == b) return signbit(a) ? b : a;
    return a > b ? a : b;
}
template <typename F>
__device__ __forceinline__ F jl_min(F a, F b) {
    if (a != a) return a;
    if (b != b) return b;
    if (a == b) return signbit(a) ? a : b;
    return a < b ? a : b;
}
// Binary32 has the same semantics in one instruction: max.NaN / min.NaN return NaN when either
// input is NaN and order -0.0 below +0.0.
template <>
__device__ __forceinline__ float jl_max<float>(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
template <>
__device__ __forceinline__ float jl_min<float>(float a, float b) {
    float r;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

}  // namespace b200
#endif
