/*
 * b200arrays.h — C ABI of libb200arrays.so: hand-written sm_100a CUDA kernels for the dense
 * data-parallel array path of AMDGPU.jl (fused broadcast, mapreduce with dims, accumulate,
 * sort/sortperm) together with the stream-ordered memory pool and the stream/event runtime
 * those operators sit on.
 *
 * Conventions (they follow the reference's FFI layer: gen/hip/generator.jl:44-70 wraps every
 * driver call in a status check, src/hip/error.jl:143-147 treats "not ready" as a non-error):
 *   - every function returns an int32 status (B200_OK == 0); b200_last_error() gives the text
 *     of the calling thread's most recent failure;
 *   - all array work is asynchronous on the stream handle that is passed in; scalar results are
 *     written to caller-provided device memory, never returned by value;
 *   - the library never calls back into the host language and keeps no pointer to caller-owned
 *     host memory after a call returns (descriptors and programs are consumed before return);
 *   - the library selects the stream's device itself on every entry, so any host thread may
 *     call with any handle (this replaces prepare_state, src/tls.jl:192-199);
 *   - arrays are dense column-major with ELEMENT strides; stride 0 marks a broadcast dimension;
 *     data pointers only need the natural alignment of their element type;
 *   - errors found on the device (a bounded wait that ran out) are latched in a per-device
 *     status word and surface from the next b200_stream_sync / b200_device_sync, the way
 *     throw_if_exception does (src/runtime/hip-execution.jl:58, src/highlevel.jl:40).
 */
#ifndef B200ARRAYS_H
#define B200ARRAYS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------- */
enum {
    B200_OK = 0,
    B200_NOT_READY = 1,        /* stream/event query: work still in flight (not an error)       */
    B200_INVALID_ARG = 2,
    B200_UNSUPPORTED = 3,      /* dtype / op / layout outside the supported set (no CPU fallback)*/
    B200_OOM = 4,              /* pool or hard limit exhausted; caller may collect and retry    */
    B200_CUDA_ERROR = 5,
    B200_NCCL_ERROR = 6,
    B200_LOOKBACK_TIMEOUT = 7, /* a bounded device-side wait gave up; result is invalid         */
    B200_NOT_INITIALISED = 8,
    B200_TOO_LARGE = 9
};

/* ---- element types ------------------------------------------------------------------------ */
enum {
    B200_F16 = 0, B200_BF16 = 1, B200_F32 = 2, B200_F64 = 3,
    B200_I8 = 4,  B200_I16 = 5,  B200_I32 = 6, B200_I64 = 7,
    B200_U8 = 8,  B200_U16 = 9,  B200_U32 = 10, B200_U64 = 11,
    B200_BOOL = 12,
    B200_DTYPE_COUNT = 13
};

/* ---- elementwise program opcodes ---------------------------------------------------------- */
/* A program is a postfix byte string of (opcode, operand) pairs evaluated per output element
 * on a value stack.  LEAF pushes leaf number `operand`; CONVERT converts the top of stack to
 * dtype `operand`; every other opcode pops its inputs and pushes one result, computed in dtype
 * `operand` (inputs must already have that dtype).  16-bit floats compute in binary32 and round
 * after every operation, small integers wrap to their width, as Julia Base does. */
enum {
    B200_OP_LEAF = 0,
    B200_OP_CONVERT = 1,
    B200_OP_ADD = 2, B200_OP_SUB = 3, B200_OP_MUL = 4, B200_OP_DIV = 5,
    B200_OP_MULADD = 6,          /* a*b+c, may be fused (Base.muladd)                           */
    B200_OP_ABS = 7, B200_OP_ABS2 = 8, B200_OP_EXP = 9,
    B200_OP_MAX = 10, B200_OP_MIN = 11,   /* NaN-propagating, -0.0 < +0.0 (Base.max/min)        */
    B200_OP_NEG = 12,
    B200_OP_COUNT = 13
};

/* ---- reduction / scan operators ----------------------------------------------------------- */
enum { B200_RED_ADD = 0, B200_RED_MUL = 1, B200_RED_MAX = 2, B200_RED_MIN = 3, B200_RED_COUNT = 4 };

#define B200_MAX_DIMS 8
#define B200_MAX_LEAVES 8
#define B200_MAX_PROGRAM 64      /* instruction pairs */

typedef struct b200_stream_s* b200_stream_t;
typedef struct b200_event_s*  b200_event_t;
typedef struct b200_comm_s*   b200_comm_t;
typedef struct b200_peer_s*   b200_peer_t;
typedef struct b200_graph_s*      b200_graph_t;
typedef struct b200_graph_exec_s* b200_graph_exec_t;

/* Dense array view.  Mirrors what ROCArray hands to a kernel (src/array.jl:19-39: buffer, dims,
 * byte offset; pointer = base + offset, src/array.jl:353-354). */
typedef struct {
    void*   ptr;
    int32_t dtype;
    int32_t ndim;
    int64_t shape[B200_MAX_DIMS];
    int64_t stride[B200_MAX_DIMS];   /* in elements */
} b200_tensor;

/* Broadcast leaf: an array or a scalar (Ref / number; src/conversions.jl:1-13). For a scalar,
 * t.dtype gives the type and `scalar` holds its bits (little-endian, low bytes used). */
typedef struct {
    b200_tensor t;
    int32_t     is_scalar;
    int32_t     _pad;
    uint64_t    scalar;
} b200_leaf;

typedef struct {
    uint64_t alloc_count, free_count;
    uint64_t alloc_bytes, free_bytes;     /* cumulative */
    uint64_t live_bytes, peak_live_bytes; /* library accounting */
    uint64_t pool_reserved, pool_used;    /* from the CUDA pool attributes */
    uint64_t hard_limit, soft_limit;
} b200_pool_stats_t;

typedef struct {
    char     name[128];
    int32_t  cc_major, cc_minor, sm_count, l2_bytes_mb;
    uint64_t total_mem;
    int32_t  max_smem_per_block, clock_khz;
} b200_props_t;

/* ---- library / device -------------------------------------------------------------------- */
/* replaces AMDGPU.__init__ (src/AMDGPU.jl:153-218) */
int32_t b200_init(void);
/* replaces HIP.devices / ndevices (src/hip/device.jl:112-124) */
int32_t b200_device_count(int32_t* n);
/* replaces HIP.properties / name (src/hip/device.jl:60-110) */
int32_t b200_device_props(int32_t dev, b200_props_t* out);
/* replaces HIP.can_access_peer (src/hip/device.jl:147-151) */
int32_t b200_can_access_peer(int32_t dev, int32_t peer, int32_t* out);
/* replaces status_message / HIPError text (src/hip/error.jl:1-161) */
int32_t b200_last_error(char* buf, size_t n);
const char* b200_status_name(int32_t status);
/* replaces versioninfo (src/utils.jl:44-90) */
int32_t b200_version(int32_t* cuda_runtime, int32_t* cuda_driver, int32_t* lib);
/* replaces AMDGPU.device_synchronize (src/highlevel.jl:63-70) */
int32_t b200_device_sync(int32_t dev);

/* ---- streams and events ------------------------------------------------------------------ */
/* replaces HIPStream(priority) (src/hip/stream.jl:4-36); priority in {-1 high, 0 normal, 1 low}
 * as in the reference (src/hip/stream.jl:17-27) */
int32_t b200_stream_create(int32_t dev, int32_t priority, b200_stream_t* out);
/* wraps a cudaStream_t owned by someone else (a torch stream, the legacy stream = NULL) */
int32_t b200_stream_wrap(int32_t dev, void* cuda_stream, b200_stream_t* out);
/* replaces the HIPStream finalizer hipStreamDestroy (src/hip/stream.jl:29-33) */
int32_t b200_stream_destroy(b200_stream_t st);
/* replaces HIP.synchronize(stream) + throw_if_exception (src/hip/stream.jl:131-143) */
int32_t b200_stream_sync(b200_stream_t st);
/* replaces HIP.isdone(stream) (src/hip/stream.jl:45-55): B200_OK or B200_NOT_READY */
int32_t b200_stream_query(b200_stream_t st);
/* Returns the stream's operator scratch (block partials, radix double buffers, scan descriptors)
 * to the pool, stream ordered; part of reclaim (src/memory.jl:333-344).  Scratch whose address a
 * captured graph holds is kept. */
int32_t b200_stream_release_scratch(b200_stream_t st);
int32_t b200_stream_device(b200_stream_t st, int32_t* dev);
int32_t b200_stream_raw(b200_stream_t st, void** cuda_stream);
/* replaces HIPEvent (src/hip/event.jl:1-75) */
int32_t b200_event_create(int32_t dev, int32_t timing, b200_event_t* out);
int32_t b200_event_destroy(b200_event_t ev);
int32_t b200_event_record(b200_event_t ev, b200_stream_t st);
int32_t b200_event_sync(b200_event_t ev);
int32_t b200_event_query(b200_event_t ev);
/* replaces HIP.elapsed (src/hip/event.jl:71-75): milliseconds between two recorded events */
int32_t b200_event_elapsed_ms(b200_event_t start, b200_event_t stop, float* ms);
/* makes `st` wait for `ev` (replaces HIP.wait(event), src/hip/event.jl:30-36) */
int32_t b200_stream_wait_event(b200_stream_t st, b200_event_t ev);

/* ---- memory pool --------------------------------------------------------------------------- */
/* replaces pool_create + hard/soft limits (src/runtime/memory/hip.jl:4-25, src/memory.jl:37-98);
 * UINT64_MAX = "none" */
int32_t b200_pool_configure(int32_t dev, uint64_t hard_limit, uint64_t soft_limit);
/* replaces HIPBuffer(bytes; stream) → hipMallocFromPoolAsync (src/runtime/memory/hip.jl:38-66);
 * bytes == 0 yields a NULL pointer; B200_OOM is returned (never retried here) so the host can
 * run the collect-and-retry ladder of alloc_or_retry! (src/runtime/memory/utils.jl:1-47) */
int32_t b200_malloc_async(void** ptr, size_t bytes, b200_stream_t st);
/* replaces Mem.free(::HIPBuffer; stream) → hipFreeAsync (src/runtime/memory/hip.jl:82-89) */
int32_t b200_free_async(void* ptr, b200_stream_t st);
/* replaces HIP.trim / reclaim (src/hip/pool.jl:36-40, src/memory.jl:333-344) */
int32_t b200_pool_trim(int32_t dev, size_t keep_bytes);
/* replaces AllocStats / MemoryStats / pool_status (src/memory.jl:103-166,376-404) */
int32_t b200_pool_stats(int32_t dev, b200_pool_stats_t* out);
/* replaces AMDGPU.info / free / total (src/memory.jl:7-35) */
int32_t b200_mem_info(int32_t dev, size_t* free_bytes, size_t* total_bytes);
/* replaces Mem.memcpy! (direction inferred; src/runtime/memory/hip.jl:91-102) */
int32_t b200_memcpy_async(void* dst, const void* src, size_t bytes, b200_stream_t st);
/* replaces Mem.memset! D8/D16/D32 and fill! (src/runtime/memory/hip.jl:107-117,
 * src/array.jl:261-266); width_bytes in {1,2,4,8}, count in elements */
int32_t b200_memset_async(void* dst, uint64_t pattern, int32_t width_bytes, size_t count,
                          b200_stream_t st);
/* replaces HostBuffer (pinned) alloc / free (src/runtime/memory/hip.jl:125-192) */
int32_t b200_host_alloc(void** ptr, size_t bytes);
int32_t b200_host_free(void* ptr);
/* replaces Mem.register / unregister (src/runtime/memory/hip.jl:216-267) */
int32_t b200_host_register(void* ptr, size_t bytes, void** dev_ptr);
int32_t b200_host_unregister(void* ptr);

/* ---- array operators ----------------------------------------------------------------------- */
/* replaces the broadcast kernel GPUArrays launches for a Broadcasted{ROCArrayStyle}
 * (style selection: src/broadcast.jl:3-30): out[I] = program(leaves[I]...) */
int32_t b200_broadcast(b200_stream_t st, const b200_tensor* out, const b200_leaf* leaves,
                       int32_t nleaves, const uint8_t* program, int32_t ninstr);
/* Broadcast expressions outside the hard-wired set run through an evaluator that the library
 * specialises for the expression at run time (the counterpart of the reference compiling each
 * broadcast kernel with GPUCompiler on first use, src/broadcast.jl:3-35 + GPUArrays): the first
 * call with a new expression STRUCTURE (operators, element types, dense/strided) compiles for a
 * few hundred milliseconds, later calls reuse the kernel whatever the pointers, sizes and scalar
 * values.  b200_broadcast_prepare compiles without launching (no device needed; the check_tensor
 * rules of b200_broadcast apply, data is not touched); B200_UNSUPPORTED when the run-time compiler
 * (libnvrtc) is not available - b200_broadcast then interprets the expression on the GPU instead.
 * b200_jit_configure(0) switches specialisation off (env B200_JIT=0 does the same);
 * b200_jit_stats: out[0] kernels compiled, out[1] cache hits, out[2] failures, out[3] enabled. */
int32_t b200_broadcast_prepare(const b200_tensor* out, const b200_leaf* leaves, int32_t nleaves,
                               const uint8_t* program, int32_t ninstr);
int32_t b200_jit_configure(int32_t enable);
int32_t b200_jit_stats(uint64_t out[4]);

/* replaces GPUArrays.mapreducedim!(f, op, R, A; init) (src/kernels/mapreduce.jl:86-173).
 * The map f (possibly a whole broadcast tree) is given as a program over `leaves`; the index
 * space is described by `shape` (ndim entries, that of A); R's shape equals it except for
 * extent 1 in the reduced dimensions.  init == NULL means "R already holds op's neutral
 * element" (src/kernels/mapreduce.jl:60); otherwise init points to one HOST value of R's dtype
 * which is folded in exactly once per output.  Empty A leaves R untouched (:91). */
int32_t b200_mapreduce(b200_stream_t st, const b200_tensor* R, const int64_t* shape, int32_t ndim,
                       const b200_leaf* leaves, int32_t nleaves, const uint8_t* program,
                       int32_t ninstr, int32_t op, const void* init);
/* Validates the same arguments and compiles the kernel that call would need, without launching
 * (no stream, no device): the counterpart of b200_broadcast_prepare for reductions whose map is an
 * expression.  B200_OK also when a kernel that is part of the library serves the call;
 * B200_UNSUPPORTED when the run-time compiler is unavailable (the call itself then interprets). */
int32_t b200_mapreduce_prepare(const b200_tensor* R, const int64_t* shape, int32_t ndim, const b200_leaf* leaves,
                               int32_t nleaves, const uint8_t* program, int32_t ninstr, int32_t op);

/* replaces Base.accumulate!(op, B, A; init, dims) → AK.accumulate! (src/kernels/accumulate.jl:1-8).
 * B and A have equal shape and dtype; dim is 0-based; init is one HOST value of that dtype or
 * NULL (no seed); inclusive != 0 gives B[i] = op(B[i-1], A[i]) seeded by init. B may alias A. */
int32_t b200_accumulate(b200_stream_t st, const b200_tensor* B, const b200_tensor* A, int32_t op,
                        const void* init, int32_t dim, int32_t inclusive);

/* Same scan, seeded by a carry that lives in DEVICE memory (one element of the arrays' type):
 * the sharded scan passes the fold of the lower ranks' totals without a host round trip.  The
 * reference has no counterpart (it has no multi-GPU scan). */
int32_t b200_accumulate_carry(b200_stream_t st, const b200_tensor* B, const b200_tensor* A, int32_t op,
                              const void* carry_dev, int32_t dim, int32_t inclusive);

/* accumulate! for callers that must not allocate once they are running (a process that gave all
 * device memory to its own arena, a plug-in whose host forbids allocations after start-up, a
 * fixed-latency loop).  No counterpart in the reference, which always draws scan temporaries from
 * its pool.  Same arguments and results as b200_accumulate; the scan's bookkeeping lives in a
 * 1 MiB array built into the library (held by every device that loads it), so inputs are
 * limited to 131040 tiles (4096 four-byte / 8192 two-byte elements each) or 43680 tiles of 2048
 * eight-byte elements, one tile at least per scanned column; beyond that B200_TOO_LARGE.  The
 * first call on a device resolves the array's address: issue it at start-up, before any stream
 * capture.  Calls share the array, so calls that could overlap on the GPU must be ordered. */
int32_t b200_accumulate_noalloc(b200_stream_t st, const b200_tensor* B, const b200_tensor* A,
                                int32_t op, const void* init, int32_t dim, int32_t inclusive);

/* replaces Base.sort!(x; rev) → AK.sort! (src/kernels/sorting.jl:1): in place, 1-D contiguous,
 * total order of Base.isless (NaN last, -0.0 < +0.0) */
int32_t b200_sort(b200_stream_t st, const b200_tensor* x, int32_t rev);
/* replaces Base.sortperm!(ix, x; rev) → AK.sortperm! (src/kernels/sorting.jl:2-3): ix is Int64,
 * receives the 1-based stable permutation; x is left untouched */
int32_t b200_sortperm(b200_stream_t st, const b200_tensor* ix, const b200_tensor* x, int32_t rev);

/* replaces the scatter kernel of findall / logical indexing (src/kernels/indexing.jl:8-36).
 * `indices` = cumsum of the Bool mask as Int64 or Int32 (b200_accumulate).  values == NULL: ys (Int64)
 * receives the 1-based linear indices of the true entries; otherwise ys receives values[mask]. */
int32_t b200_compact(b200_stream_t st, const b200_tensor* ys, const b200_tensor* bools,
                     const b200_tensor* indices, const b200_tensor* values);
/* replaces getindex with an integer index vector, y = x[ix] (GPUArrays' vectorised getindex, as
 * used by test/hip_rocarray/sorting.jl:14 `xd[sortperm(xd)]`): indices are 1-based Int64 or Int32,
 * x is read in linear order whatever its shape.  An index outside 1..length(x) latches
 * B200_INVALID_ARG, reported by the next b200_stream_sync; that output element is not written. */
int32_t b200_gather(b200_stream_t st, const b200_tensor* y, const b200_tensor* x, const b200_tensor* ix);
/* replaces _reverse! (src/kernels/reverse.jl:59-87): y = x flipped along the dimensions whose bit
 * is set in dims_mask (bit 0 = first dimension); y and x must not alias. */
int32_t b200_reverse(b200_stream_t st, const b200_tensor* y, const b200_tensor* x, uint32_t dims_mask);

/* replaces rand!/randn! for the synthetic workloads (src/random.jl:30-70): element i of `out`
 * becomes gen(seed, stream_id, first_index + i); dist 0: U[0,1), 1: U[-1,1), 2: N(0,1),
 * 3: integers in [lo,hi], 4: raw low bits.  Counter based, so any slice can be regenerated. */
int32_t b200_fill_random(b200_stream_t st, const b200_tensor* out, int32_t dist, uint64_t seed,
                         uint64_t stream_id, uint64_t first_index, int64_t lo, int64_t hi);

/* ---- graphs (replaces src/hip/graph.jl:16-168: capture, instantiate, launch, update,
 * is_capturing) --------------------------------------------------------------------------- */
/* Every operator above can be captured.  An operator that needs more stream scratch than the
 * stream holds answers B200_UNSUPPORTED inside a capture: run the operation once on that stream
 * first (what @captured does when its first capture fails, src/hip/graph.jl:139-168).  Scratch seen
 * by a capture stays allocated as long as the stream lives.  mode: 0 global, 1 thread local,
 * 2 relaxed (hipStreamCaptureMode). */
int32_t b200_graph_capture_begin(b200_stream_t st, int32_t mode);
/* *out = NULL and an error status when the capture was invalidated */
int32_t b200_graph_capture_end(b200_stream_t st, b200_graph_t* out);
int32_t b200_stream_is_capturing(b200_stream_t st, int32_t* out);
int32_t b200_graph_destroy(b200_graph_t g);
/* allocations captured without their free are released at the next launch of the same graph */
int32_t b200_graph_instantiate(b200_graph_t g, b200_graph_exec_t* out);
int32_t b200_graph_exec_destroy(b200_graph_exec_t e);
int32_t b200_graph_launch(b200_graph_exec_t e, b200_stream_t st);
/* *updated = 1 when `e` now runs `g`; 0 (with B200_OK) when the topologies differ and `e` is unchanged */
int32_t b200_graph_exec_update(b200_graph_exec_t e, b200_graph_t g, int32_t* updated);

/* ---- multi-GPU (one process per GPU) ----------------------------------------------------- */
/* The reference has no collective layer (multi-GPU is one task per device with host copies,
 * docs/src/usage/multitasking.md:37-53); these calls are what the sharded operators add. */
int32_t b200_comm_unique_id(uint8_t id_out[128]);
int32_t b200_comm_init_rank(b200_comm_t* out, int32_t nranks, int32_t rank,
                            const uint8_t id[128], int32_t dev);
int32_t b200_comm_destroy(b200_comm_t comm);
/* Host-side failure detection for the collectives: waits until `st` has drained (st == NULL: looks
 * at the communicator only, once the time is up B200_NOT_READY while NCCL still reports progress),
 * polling ncclCommGetAsyncError meanwhile; an asynchronous error, or `timeout_ms` passing with the
 * stream still busy (a rank that never arrived), aborts the communicator (ncclCommAbort) and
 * returns B200_NCCL_ERROR - after that the communicator only accepts b200_comm_destroy.  Closest
 * relative in the reference: the watchdog on a stream that does not finish, src/hip/stream.jl:99-126.
 * Environment B200_NCCL_LIB names the NCCL library to load instead of libnccl.so.2;
 * b200_comm_init_rank with dev < 0 creates a communicator that is not bound to a device. */
int32_t b200_comm_check(b200_comm_t comm, b200_stream_t st, int32_t timeout_ms);
/* in-place all-reduce of `count` elements of R's dtype on the stream, directly after the kernel
 * that produced them (no host round trip) */
int32_t b200_allreduce(b200_comm_t comm, void* buf, size_t count, int32_t dtype, int32_t op,
                       b200_stream_t st);
/* gathers `count` elements from every rank into recv[rank*count ...] */
int32_t b200_allgather(b200_comm_t comm, const void* send, void* recv, size_t count,
                       int32_t dtype, b200_stream_t st);

/* Self-test of the bounded device-side waits (no counterpart in the reference, whose device-side
 * errors are reported through its exception word, src/device/exceptions.jl:27-66): one scan tile
 * waits for a predecessor that never publishes, gives up after `polls` polls and latches
 * B200_LOOKBACK_TIMEOUT, which the next b200_stream_sync returns.  No fault, no unbounded spin. */
int32_t b200_selftest_wait_timeout(b200_stream_t st, uint32_t polls);

/* Fused reduce + all-reduce over exchange slots that every rank of a group can write (no
 * counterpart in the reference, which has no collective layer).  Every rank calls b200_peer_create,
 * the 64-byte handles are gathered on the host (rank r's handle at handles[64*r]), every rank calls
 * b200_peer_connect.  All ranks must then issue the same sequence of b200_mapreduce_allreduce calls.
 * `transport` says where the slots live:
 *   B200_PEER_HOST  POSIX shared memory registered with the CUDA runtime in every rank; stores and
 *                   polls cross PCIe; no GPU maps another GPU's memory (the handle is the name);
 *   B200_PEER_VMM   one 2 MiB device allocation per rank, exported as a file descriptor and mapped
 *                   by the peers over NVLink - peer access for that allocation only.  The handle
 *                   holds {pid, fd}; a descriptor is only valid inside its process, so either the
 *                   host code passes it over a Unix socket (SCM_RIGHTS) and rewrites pid/fd before
 *                   b200_peer_connect, or the library fetches it with pidfd_getfd (needs the right
 *                   to inspect the exporting process);
 *   B200_PEER_IPC   cudaMalloc + CUDA IPC handle; opening it enables peer access device wide.
 * A group of one rank needs no connect. */
enum { B200_PEER_HOST = 0, B200_PEER_VMM = 1, B200_PEER_IPC = 2 };
int32_t b200_peer_create(int32_t dev, int32_t rank, int32_t nranks, int32_t transport, b200_peer_t* out,
                         uint8_t handle_out[64]);
int32_t b200_peer_connect(b200_peer_t peer, const uint8_t* handles);
/* Call once EVERY rank's b200_peer_connect has returned (the caller knows: one round over its host
 * channel): removes the shared-memory name / closes the exported descriptor, so a process that
 * dies later leaves nothing behind.  Optional; b200_peer_destroy does the same.  No counterpart in
 * the reference. */
int32_t b200_peer_seal(b200_peer_t peer);
/* how often the exchange polls for a peer's partial before it gives up and latches
 * B200_LOOKBACK_TIMEOUT (default 2^26, about ten seconds with the back-off) */
int32_t b200_peer_set_poll_budget(b200_peer_t peer, uint32_t polls);
/* transport of the group and the number of collectives issued so far (either may be NULL) */
int32_t b200_peer_info(b200_peer_t peer, int32_t* transport, uint64_t* seq);
int32_t b200_peer_destroy(b200_peer_t peer);
/* mapreducedim! to ONE element followed by an all-reduce of that element over the peer group,
 * in a single kernel: the block that completes the local reduction stores the partial into every
 * rank's exchange slot and folds all ranks' partials in rank order (identical bits on all ranks).
 * Restricted to a full reduction of one dense array with f in {identity, abs, abs2}; other
 * cases return B200_UNSUPPORTED before anything is exchanged (use b200_mapreduce +
 * b200_allreduce) - that verdict depends on the expression and element types only, so all ranks
 * reach it together.  A rank whose shard is empty takes part with the operator's neutral element.
 * Waits are bounded. */
int32_t b200_mapreduce_allreduce(b200_peer_t peer, b200_stream_t st, const b200_tensor* R,
                                 const int64_t* shape, int32_t ndim, const b200_leaf* leaves,
                                 int32_t nleaves, const uint8_t* program, int32_t ninstr, int32_t op,
                                 const void* init);

#ifdef __cplusplus
}
#endif
#endif /* B200ARRAYS_H */
