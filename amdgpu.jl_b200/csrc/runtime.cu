// Runtime half of libb200arrays.so: device/stream/event handles, the stream-ordered memory
// pool with library-side accounting and limits, copies and fills, and the latched device error
// word.  It stands in for the reference's L2/L4 layers (src/hip/*.jl, src/memory.jl,
// src/runtime/memory/hip.jl) on top of the CUDA runtime.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace b200 {

static thread_local std::string g_last_error;

// B200_LOG: unset/empty = silent, anything = errors, "debug" = also one line per call (the
// reference's @debug lines: src/array.jl:28, src/runtime/memory/hip.jl:58).
static int log_level() {
    static const int level = [] {
        const char* lg = getenv("B200_LOG");
        if (!lg || !lg[0]) return 0;
        return strcmp(lg, "debug") == 0 ? 2 : 1;
    }();
    return level;
}

int32_t fail(int32_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    if (log_level() >= 1) fprintf(stderr, "[b200] error %d: %s\n", code, buf);
    return code;
}

bool overlap_launches_enabled() {
    static const bool on = [] {
        const char* e = getenv("B200_OVERLAP_LAUNCHES");
        return !(e && e[0] == '0');
    }();
    return on;
}

void log_debug(const char* fmt, ...) {
    if (log_level() < 2) return;
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    fprintf(stderr, "[b200] %s\n", buf);
}

int32_t cuda_fail(cudaError_t e, const char* what) {
    // An out-of-memory report is recoverable; clear the sticky-free error state.
    cudaGetLastError();
    if (e == cudaErrorMemoryAllocation) return fail(B200_OOM, "out of memory in %s", what);
    if (e == cudaErrorNotReady) return B200_NOT_READY;
    return fail(B200_CUDA_ERROR, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

// ---- per-device state ------------------------------------------------------------------------
struct DeviceState {
    std::mutex mu;
    bool       ready = false;
    cudaMemPool_t pool = nullptr;
    int32_t*   err_host = nullptr;   // pinned, mapped; kernels store a status code here
    int32_t*   err_dev = nullptr;
    int        sms = 0;
    uint64_t   hard_limit = UINT64_MAX, soft_limit = UINT64_MAX;
    std::unordered_map<void*, size_t> live;
    b200_pool_stats_t stats{};
};

static std::mutex g_mu;
static int g_ndev = -1;
static std::vector<DeviceState*> g_dev;
static bool g_launch_blocking = false;

static int32_t ensure_init() {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_ndev >= 0) return B200_OK;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(B200_NOT_INITIALISED, "no usable CUDA device: %s", cudaGetErrorString(e));
    }
    g_dev.resize(n);
    for (int i = 0; i < n; ++i) g_dev[i] = new DeviceState();
    const char* lb = getenv("B200_LAUNCH_BLOCKING");
    g_launch_blocking = lb && lb[0] && lb[0] != '0';
    g_ndev = n;
    return B200_OK;
}

static int32_t device_state(int dev, DeviceState** out) {
    B200_TRY(ensure_init());
    if (dev < 0 || dev >= g_ndev) return fail(B200_INVALID_ARG, "device %d out of range [0,%d)", dev, g_ndev);
    DeviceState* d = g_dev[dev];
    B200_CUDA(cudaSetDevice(dev));
    std::lock_guard<std::mutex> lk(d->mu);
    if (!d->ready) {
        cudaMemPoolProps props{};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        B200_CUDA(cudaMemPoolCreate(&d->pool, &props));
        uint64_t thr = UINT64_MAX;   // keep freed blocks cached until trimmed (soft limit "none")
        B200_CUDA(cudaMemPoolSetAttribute(d->pool, cudaMemPoolAttrReleaseThreshold, &thr));
        B200_CUDA(cudaHostAlloc((void**)&d->err_host, sizeof(int32_t) * 4, cudaHostAllocMapped));
        memset(d->err_host, 0, sizeof(int32_t) * 4);
        B200_CUDA(cudaHostGetDevicePointer((void**)&d->err_dev, d->err_host, 0));
        B200_CUDA(cudaDeviceGetAttribute(&d->sms, cudaDevAttrMultiProcessorCount, dev));
        d->stats.hard_limit = d->hard_limit;
        d->stats.soft_limit = d->soft_limit;
        d->ready = true;
    }
    *out = d;
    return B200_OK;
}

int32_t enter(b200_stream_t st) {
    if (!st) return fail(B200_INVALID_ARG, "null stream handle");
    DeviceState* d;
    return device_state(st->dev, &d);
}

int32_t* device_error_word(int dev) { return g_dev[dev]->err_dev; }
int sm_count(int dev) { return g_dev[dev]->sms; }

int cached_blocks_per_sm(const void* kernel, int threads, size_t dyn_smem, int dev) {
    struct Key {
        const void* k; int threads; size_t smem; int dev;
        bool operator==(const Key& o) const { return k == o.k && threads == o.threads && smem == o.smem && dev == o.dev; }
    };
    struct Hash {
        size_t operator()(const Key& x) const {
            return std::hash<const void*>()(x.k) ^ (std::hash<size_t>()(x.smem) * 31) ^ ((size_t)x.threads << 20) ^ ((size_t)x.dev << 40);
        }
    };
    static std::mutex mu;
    static std::unordered_map<Key, int, Hash> cache;
    const Key key{kernel, threads, dyn_smem, dev};
    {
        std::lock_guard<std::mutex> lk(mu);
        auto it = cache.find(key);
        if (it != cache.end()) return it->second;
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, dyn_smem) != cudaSuccess || per_sm < 1) {
        cudaGetLastError();
        per_sm = 1;
    }
    std::lock_guard<std::mutex> lk(mu);
    cache[key] = per_sm;
    return per_sm;
}

int32_t finish(b200_stream_t st, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, what);
    log_debug("%s: launched on device %d, stream %p", what, st->dev, (void*)st->s);
    if (g_launch_blocking) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st->s, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) return b200_stream_sync(st);
    }
    return B200_OK;
}

static int32_t pool_alloc(DeviceState* d, void** ptr, size_t bytes, cudaStream_t s, const char* who) {
    *ptr = nullptr;
    if (bytes == 0) return B200_OK;
    {
        std::lock_guard<std::mutex> lk(d->mu);
        if (d->hard_limit != UINT64_MAX && d->stats.live_bytes + bytes > d->hard_limit)
            return fail(B200_OOM, "%s: %zu bytes would exceed the hard memory limit (%llu live, limit %llu)",
                        who, bytes, (unsigned long long)d->stats.live_bytes, (unsigned long long)d->hard_limit);
    }
    cudaError_t e = cudaMallocFromPoolAsync(ptr, bytes, d->pool, s);
    if (e != cudaSuccess) { *ptr = nullptr; return cuda_fail(e, who); }
    log_debug("%s: %zu bytes at %p (stream %p)", who, bytes, *ptr, (void*)s);
    std::lock_guard<std::mutex> lk(d->mu);
    d->live[*ptr] = bytes;
    d->stats.alloc_count++;
    d->stats.alloc_bytes += bytes;
    d->stats.live_bytes += bytes;
    if (d->stats.live_bytes > d->stats.peak_live_bytes) d->stats.peak_live_bytes = d->stats.live_bytes;
    return B200_OK;
}

static int32_t pool_free(DeviceState* d, void* ptr, cudaStream_t s) {
    if (!ptr) return B200_OK;
    {
        std::lock_guard<std::mutex> lk(d->mu);
        auto it = d->live.find(ptr);
        if (it == d->live.end()) return fail(B200_INVALID_ARG, "free of a pointer this pool did not allocate");
        d->stats.free_count++;
        d->stats.free_bytes += it->second;
        d->stats.live_bytes -= it->second;
        d->live.erase(it);
    }
    B200_CUDA(cudaFreeAsync(ptr, s));
    return B200_OK;
}

int32_t scratch(b200_stream_t st, size_t bytes, void** out, unsigned int** counters) {
    DeviceState* d;
    B200_TRY(device_state(st->dev, &d));
    std::lock_guard<std::recursive_mutex> guard(st->mu);
    const size_t need = bytes + kCounterBytes;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    B200_CUDA(cudaStreamIsCapturing(st->s, &cap));
    const bool capturing = cap != cudaStreamCaptureStatusNone;
    if (need > st->scratch_bytes) {
        // growing would put an allocation and a zero-fill of the counters into the graph and leave
        // the stream with an address that only exists inside that graph
        if (capturing)
            return fail(B200_UNSUPPORTED, "this operation needs %zu bytes of stream scratch and the stream holds %zu: "
                        "run it once on this stream before capturing it", need, st->scratch_bytes);
        size_t want = need < (1u << 20) ? (1u << 20) : need + need / 4;
        want = (want + 255) & ~size_t(255);
        if (st->scratch && st->scratch_in_graph) st->retired.push_back(st->scratch);
        else if (st->scratch) B200_TRY(pool_free(d, st->scratch, st->s));
        st->scratch_in_graph = false;
        st->scratch = nullptr;
        st->scratch_bytes = 0;
        B200_TRY(pool_alloc(d, &st->scratch, want, st->s, "operator scratch"));
        st->scratch_bytes = want;
        B200_CUDA(cudaMemsetAsync(st->scratch, 0, kCounterBytes, st->s));
    }
    if (capturing) st->scratch_in_graph = true;
    if (counters) *counters = reinterpret_cast<unsigned int*>(st->scratch);
    *out = reinterpret_cast<char*>(st->scratch) + kCounterBytes;
    return B200_OK;
}

int32_t scan_state(b200_stream_t st, size_t bytes, void** out, uint32_t* epoch, bool* must_clear) {
    DeviceState* d;
    B200_TRY(device_state(st->dev, &d));
    std::lock_guard<std::recursive_mutex> guard(st->mu);
    const size_t need = bytes + kScanStateHeader;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    B200_CUDA(cudaStreamIsCapturing(st->s, &cap));
    const bool capturing = cap != cudaStreamCaptureStatusNone;
    if (need > st->scan_state_bytes) {
        if (capturing)
            return fail(B200_UNSUPPORTED, "this scan needs %zu bytes of descriptor storage and the stream holds %zu: "
                        "run it once on this stream before capturing it", need, st->scan_state_bytes);
        size_t want = need < (size_t(1) << 20) ? (size_t(1) << 20) : need + need / 4;
        want = (want + 255) & ~size_t(255);
        if (st->scan_state && st->scan_state_in_graph) st->retired.push_back(st->scan_state);
        else if (st->scan_state) B200_TRY(pool_free(d, st->scan_state, st->s));
        st->scan_state = nullptr;
        st->scan_state_bytes = 0;
        st->scan_state_in_graph = false;
        B200_TRY(pool_alloc(d, &st->scan_state, want, st->s, "scan descriptors"));
        st->scan_state_bytes = want;
        B200_CUDA(cudaMemsetAsync(st->scan_state, 0, want, st->s));
        st->scan_epoch = 0;
    }
    if (st->scan_epoch >= (1u << 30) - 1) {      // tags wrapped: start over from clean words
        if (capturing) return fail(B200_UNSUPPORTED, "scan descriptor tags wrapped during a capture; run the scan once outside the capture");
        B200_CUDA(cudaMemsetAsync(st->scan_state, 0, st->scan_state_bytes, st->s));
        st->scan_epoch = 0;
    }
    *epoch = ++st->scan_epoch;
    *must_clear = capturing;
    if (capturing) st->scan_state_in_graph = true;
    *out = st->scan_state;
    return B200_OK;
}

int32_t check_tensor(const b200_tensor* t, const char* name) {
    if (!t) return fail(B200_INVALID_ARG, "%s: null tensor descriptor", name);
    if (t->ndim < 0 || t->ndim > B200_MAX_DIMS) return fail(B200_INVALID_ARG, "%s: ndim %d outside [0,%d]", name, t->ndim, B200_MAX_DIMS);
    if (dtype_size(t->dtype) == 0) return fail(B200_UNSUPPORTED, "%s: unknown dtype %d", name, t->dtype);
    int64_t n = 1;
    for (int d = 0; d < t->ndim; ++d) {
        if (t->shape[d] < 0) return fail(B200_INVALID_ARG, "%s: negative extent in dim %d", name, d);
        n *= t->shape[d];
    }
    if (n > 0 && !t->ptr) return fail(B200_INVALID_ARG, "%s: null data pointer", name);
    if (n > 0 && (reinterpret_cast<uintptr_t>(t->ptr) % dtype_size(t->dtype)) != 0)
        return fail(B200_INVALID_ARG, "%s: pointer is not aligned to its element size", name);
    return B200_OK;
}

// ---- fill kernel -------------------------------------------------------------------------------
template <typename T>
__global__ void fill_kernel(T* __restrict__ dst, T value, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    // 16-byte body when the pointer allows it, scalar head/tail otherwise.
    constexpr int V = 16 / sizeof(T);
    uintptr_t a = reinterpret_cast<uintptr_t>(dst);
    size_t head = ((16 - (a & 15)) & 15) / sizeof(T);
    if (head > n) head = n;
    size_t nvec = (n - head) / V;
    Vec<T, V> pack;
#pragma unroll
    for (int k = 0; k < V; ++k) pack.v[k] = value;
    Vec<T, V>* body = reinterpret_cast<Vec<T, V>*>(dst + head);
    for (size_t j = i; j < nvec; j += stride) body[j] = pack;
    size_t done = head + nvec * V;
    for (size_t j = i; j < head; j += stride) dst[j] = value;
    for (size_t j = done + i; j < n; j += stride) dst[j] = value;
}

template <typename T>
static void launch_fill(void* dst, uint64_t pattern, size_t count, b200_stream_t st) {
    T v;
    memcpy(&v, &pattern, sizeof(T));
    size_t per_block = 256 * (16 / sizeof(T)) * 4;
    size_t blocks = (count + per_block - 1) / per_block;
    size_t cap = (size_t)sm_count(st->dev) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    fill_kernel<T><<<(unsigned)blocks, 256, 0, st->s>>>(reinterpret_cast<T*>(dst), v, count);
}

}  // namespace b200

using namespace b200;

// ---- exported: library / device ---------------------------------------------------------------
extern "C" {

int32_t b200_init(void) { return ensure_init(); }

int32_t b200_device_count(int32_t* n) {
    if (!n) return fail(B200_INVALID_ARG, "null output");
    B200_TRY(ensure_init());
    *n = g_ndev;
    return B200_OK;
}

int32_t b200_device_props(int32_t dev, b200_props_t* out) {
    if (!out) return fail(B200_INVALID_ARG, "null output");
    B200_TRY(ensure_init());
    if (dev < 0 || dev >= g_ndev) return fail(B200_INVALID_ARG, "device %d out of range", dev);
    cudaDeviceProp p;
    B200_CUDA(cudaGetDeviceProperties(&p, dev));
    memset(out, 0, sizeof *out);
    strncpy(out->name, p.name, sizeof(out->name) - 1);
    out->cc_major = p.major;
    out->cc_minor = p.minor;
    out->sm_count = p.multiProcessorCount;
    out->l2_bytes_mb = p.l2CacheSize >> 20;
    out->total_mem = p.totalGlobalMem;
    out->max_smem_per_block = (int32_t)p.sharedMemPerBlockOptin;
    int khz = 0;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
    out->clock_khz = khz;
    return B200_OK;
}

int32_t b200_can_access_peer(int32_t dev, int32_t peer, int32_t* out) {
    if (!out) return fail(B200_INVALID_ARG, "null output");
    B200_TRY(ensure_init());
    int v = 0;
    B200_CUDA(cudaDeviceCanAccessPeer(&v, dev, peer));
    *out = v;
    return B200_OK;
}

int32_t b200_last_error(char* buf, size_t n) {
    if (!buf || n == 0) return B200_INVALID_ARG;
    strncpy(buf, g_last_error.c_str(), n - 1);
    buf[n - 1] = 0;
    return B200_OK;
}

const char* b200_status_name(int32_t s) {
    switch (s) {
        case B200_OK: return "B200_OK";
        case B200_NOT_READY: return "B200_NOT_READY";
        case B200_INVALID_ARG: return "B200_INVALID_ARG";
        case B200_UNSUPPORTED: return "B200_UNSUPPORTED";
        case B200_OOM: return "B200_OOM";
        case B200_CUDA_ERROR: return "B200_CUDA_ERROR";
        case B200_NCCL_ERROR: return "B200_NCCL_ERROR";
        case B200_LOOKBACK_TIMEOUT: return "B200_LOOKBACK_TIMEOUT";
        case B200_NOT_INITIALISED: return "B200_NOT_INITIALISED";
        case B200_TOO_LARGE: return "B200_TOO_LARGE";
        default: return "B200_UNKNOWN";
    }
}

int32_t b200_version(int32_t* rt, int32_t* drv, int32_t* lib) {
    int a = 0, b = 0;
    cudaRuntimeGetVersion(&a);
    cudaDriverGetVersion(&b);
    cudaGetLastError();
    if (rt) *rt = a;
    if (drv) *drv = b;
    if (lib) *lib = 100;   // 0.1.0
    return B200_OK;
}

static int32_t check_latched(DeviceState* d) {
    int32_t code = *(volatile int32_t*)d->err_host;
    if (code != 0) {
        *(volatile int32_t*)d->err_host = 0;
        if (code == B200_LOOKBACK_TIMEOUT)
            return fail(code, "a device-side wait ran out of its poll budget (%s); the result of the "
                              "operation that reported it is invalid", b200_status_name(code));
        return fail(code, "a kernel reported %s (for example an index outside its array); the result of "
                          "the operation that reported it is incomplete", b200_status_name(code));
    }
    return B200_OK;
}

int32_t b200_device_sync(int32_t dev) {
    DeviceState* d;
    B200_TRY(device_state(dev, &d));
    B200_CUDA(cudaDeviceSynchronize());
    return check_latched(d);
}

// ---- exported: streams and events ------------------------------------------------------------
int32_t b200_stream_create(int32_t dev, int32_t priority, b200_stream_t* out) {
    if (!out) return fail(B200_INVALID_ARG, "null output");
    DeviceState* d;
    B200_TRY(device_state(dev, &d));
    if (priority < -1 || priority > 1) return fail(B200_INVALID_ARG, "priority must be -1 (high), 0 or 1 (low)");
    int lo = 0, hi = 0;
    B200_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));   // lo = least, hi = greatest (numerically smaller)
    int p = priority < 0 ? hi : (priority > 0 ? lo : (lo + hi) / 2);
    cudaStream_t s;
    B200_CUDA(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, p));
    b200_stream_s* h = new b200_stream_s();
    h->dev = dev; h->s = s; h->owned = true;
    h->scratch = nullptr; h->scratch_bytes = 0; h->scratch_in_graph = false;
    *out = h;
    return B200_OK;
}

int32_t b200_stream_wrap(int32_t dev, void* cuda_stream, b200_stream_t* out) {
    if (!out) return fail(B200_INVALID_ARG, "null output");
    DeviceState* d;
    B200_TRY(device_state(dev, &d));
    b200_stream_s* h = new b200_stream_s();
    h->dev = dev; h->s = (cudaStream_t)cuda_stream; h->owned = false;
    h->scratch = nullptr; h->scratch_bytes = 0; h->scratch_in_graph = false;
    *out = h;
    return B200_OK;
}

int32_t b200_stream_destroy(b200_stream_t st) {
    if (!st) return B200_OK;
    DeviceState* d;
    B200_TRY(device_state(st->dev, &d));
    if (st->scratch) pool_free(d, st->scratch, st->s);
    if (st->scan_state) pool_free(d, st->scan_state, st->s);
    for (void* p : st->retired) pool_free(d, p, st->s);
    if (st->owned) {
        cudaError_t e = cudaStreamDestroy(st->s);   // deferred by the runtime until work drains
        if (e != cudaSuccess) cudaGetLastError();
    }
    delete st;
    return B200_OK;
}

// Hands the stream's operator scratch (reduction partials, radix double buffers, scan descriptors)
// back to the pool, stream ordered; the next operator that needs scratch allocates it again.
// Buffers whose address a captured graph holds stay.
int32_t b200_stream_release_scratch(b200_stream_t st) {
    if (!st) return fail(B200_INVALID_ARG, "null stream handle");
    DeviceState* d;
    B200_TRY(device_state(st->dev, &d));
    std::lock_guard<std::recursive_mutex> guard(st->mu);
    if (st->scratch && !st->scratch_in_graph) {
        B200_TRY(pool_free(d, st->scratch, st->s));
        st->scratch = nullptr;
        st->scratch_bytes = 0;
    }
    if (st->scan_state && !st->scan_state_in_graph) {
        B200_TRY(pool_free(d, st->scan_state, st->s));
        st->scan_state = nullptr;
        st->scan_state_bytes = 0;
        st->scan_epoch = 0;
    }
    return B200_OK;
}

int32_t b200_stream_sync(b200_stream_t st) {
    if (!st) return fail(B200_INVALID_ARG, "null stream handle");
    DeviceState* d;
    B200_TRY(device_state(st->dev, &d));
    B200_CUDA(cudaStreamSynchronize(st->s));
    return check_latched(d);
}

int32_t b200_stream_query(b200_stream_t st) {
    B200_TRY(enter(st));
    cudaError_t e = cudaStreamQuery(st->s);
    if (e == cudaSuccess) return B200_OK;
    if (e == cudaErrorNotReady) { cudaGetLastError(); return B200_NOT_READY; }
    return cuda_fail(e, "cudaStreamQuery");
}

int32_t b200_stream_device(b200_stream_t st, int32_t* dev) {
    if (!st || !dev) return fail(B200_INVALID_ARG, "null argument");
    *dev = st->dev;
    return B200_OK;
}

int32_t b200_stream_raw(b200_stream_t st, void** cuda_stream) {
    if (!st || !cuda_stream) return fail(B200_INVALID_ARG, "null argument");
    *cuda_stream = (void*)st->s;
    return B200_OK;
}

int32_t b200_event_create(int32_t dev, int32_t timing, b200_event_t* out) {
    if (!out) return fail(B200_INVALID_ARG, "null output");
    DeviceState* d;
    B200_TRY(device_state(dev, &d));
    cudaEvent_t e;
    B200_CUDA(cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming));
    *out = new b200_event_s{dev, e};
    return B200_OK;
}

int32_t b200_event_destroy(b200_event_t ev) {
    if (!ev) return B200_OK;
    cudaSetDevice(ev->dev);
    cudaEventDestroy(ev->e);
    cudaGetLastError();
    delete ev;
    return B200_OK;
}

int32_t b200_event_record(b200_event_t ev, b200_stream_t st) {
    if (!ev) return fail(B200_INVALID_ARG, "null event handle");
    B200_TRY(enter(st));
    if (ev->dev != st->dev) return fail(B200_INVALID_ARG, "event and stream live on different devices");
    B200_CUDA(cudaEventRecord(ev->e, st->s));
    return B200_OK;
}

int32_t b200_event_sync(b200_event_t ev) {
    if (!ev) return fail(B200_INVALID_ARG, "null event handle");
    B200_CUDA(cudaSetDevice(ev->dev));
    B200_CUDA(cudaEventSynchronize(ev->e));
    return B200_OK;
}

int32_t b200_event_query(b200_event_t ev) {
    if (!ev) return fail(B200_INVALID_ARG, "null event handle");
    B200_CUDA(cudaSetDevice(ev->dev));
    cudaError_t e = cudaEventQuery(ev->e);
    if (e == cudaSuccess) return B200_OK;
    if (e == cudaErrorNotReady) { cudaGetLastError(); return B200_NOT_READY; }
    return cuda_fail(e, "cudaEventQuery");
}

int32_t b200_event_elapsed_ms(b200_event_t a, b200_event_t b, float* ms) {
    if (!a || !b || !ms) return fail(B200_INVALID_ARG, "null argument");
    B200_CUDA(cudaSetDevice(a->dev));
    B200_CUDA(cudaEventElapsedTime(ms, a->e, b->e));
    return B200_OK;
}

int32_t b200_stream_wait_event(b200_stream_t st, b200_event_t ev) {
    if (!ev) return fail(B200_INVALID_ARG, "null event handle");
    B200_TRY(enter(st));
    B200_CUDA(cudaStreamWaitEvent(st->s, ev->e, 0));
    return B200_OK;
}

// ---- exported: memory -------------------------------------------------------------------------
int32_t b200_pool_configure(int32_t dev, uint64_t hard_limit, uint64_t soft_limit) {
    DeviceState* d;
    B200_TRY(device_state(dev, &d));
    std::lock_guard<std::mutex> lk(d->mu);
    d->hard_limit = hard_limit;
    d->soft_limit = soft_limit;
    d->stats.hard_limit = hard_limit;
    d->stats.soft_limit = soft_limit;
    uint64_t thr = soft_limit;
    B200_CUDA(cudaMemPoolSetAttribute(d->pool, cudaMemPoolAttrReleaseThreshold, &thr));
    return B200_OK;
}

int32_t b200_malloc_async(void** ptr, size_t bytes, b200_stream_t st) {
    if (!ptr) return fail(B200_INVALID_ARG, "null output");
    if (!st) return fail(B200_INVALID_ARG, "null stream handle");
    DeviceState* d;
    B200_TRY(device_state(st->dev, &d));
    return pool_alloc(d, ptr, bytes, st->s, "b200_malloc_async");
}

int32_t b200_free_async(void* ptr, b200_stream_t st) {
    if (!st) return fail(B200_INVALID_ARG, "null stream handle");
    DeviceState* d;
    B200_TRY(device_state(st->dev, &d));
    return pool_free(d, ptr, st->s);
}

int32_t b200_pool_trim(int32_t dev, size_t keep) {
    DeviceState* d;
    B200_TRY(device_state(dev, &d));
    B200_CUDA(cudaMemPoolTrimTo(d->pool, keep));
    return B200_OK;
}

int32_t b200_pool_stats(int32_t dev, b200_pool_stats_t* out) {
    if (!out) return fail(B200_INVALID_ARG, "null output");
    DeviceState* d;
    B200_TRY(device_state(dev, &d));
    uint64_t reserved = 0, used = 0;
    B200_CUDA(cudaMemPoolGetAttribute(d->pool, cudaMemPoolAttrReservedMemCurrent, &reserved));
    B200_CUDA(cudaMemPoolGetAttribute(d->pool, cudaMemPoolAttrUsedMemCurrent, &used));
    std::lock_guard<std::mutex> lk(d->mu);
    *out = d->stats;
    out->pool_reserved = reserved;
    out->pool_used = used;
    return B200_OK;
}

int32_t b200_mem_info(int32_t dev, size_t* free_bytes, size_t* total_bytes) {
    DeviceState* d;
    B200_TRY(device_state(dev, &d));
    size_t f = 0, t = 0;
    B200_CUDA(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return B200_OK;
}

int32_t b200_memcpy_async(void* dst, const void* src, size_t bytes, b200_stream_t st) {
    B200_TRY(enter(st));
    if (bytes == 0) return B200_OK;
    if (!dst || !src) return fail(B200_INVALID_ARG, "null pointer in memcpy");
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, st->s));
    return B200_OK;
}

int32_t b200_memset_async(void* dst, uint64_t pattern, int32_t width, size_t count, b200_stream_t st) {
    B200_TRY(enter(st));
    if (count == 0) return B200_OK;
    if (!dst) return fail(B200_INVALID_ARG, "null pointer in memset");
    if ((reinterpret_cast<uintptr_t>(dst) % width) != 0) return fail(B200_INVALID_ARG, "memset pointer not aligned to width");
    switch (width) {
        case 1: B200_CUDA(cudaMemsetAsync(dst, (int)(pattern & 0xff), count, st->s)); break;
        case 2: launch_fill<uint16_t>(dst, pattern, count, st); break;
        case 4: launch_fill<uint32_t>(dst, pattern, count, st); break;
        case 8: launch_fill<uint64_t>(dst, pattern, count, st); break;
        default: return fail(B200_INVALID_ARG, "memset width must be 1, 2, 4 or 8 bytes");
    }
    return finish(st, "b200_memset_async");
}

int32_t b200_host_alloc(void** ptr, size_t bytes) {
    if (!ptr) return fail(B200_INVALID_ARG, "null output");
    B200_TRY(ensure_init());
    *ptr = nullptr;
    if (bytes == 0) return B200_OK;
    B200_CUDA(cudaHostAlloc(ptr, bytes, cudaHostAllocPortable | cudaHostAllocMapped));
    return B200_OK;
}

int32_t b200_host_free(void* ptr) {
    if (!ptr) return B200_OK;
    B200_CUDA(cudaFreeHost(ptr));
    return B200_OK;
}

int32_t b200_host_register(void* ptr, size_t bytes, void** dev_ptr) {
    if (!ptr) return fail(B200_INVALID_ARG, "null pointer");
    B200_TRY(ensure_init());
    B200_CUDA(cudaHostRegister(ptr, bytes, cudaHostRegisterPortable | cudaHostRegisterMapped));
    if (dev_ptr) B200_CUDA(cudaHostGetDevicePointer(dev_ptr, ptr, 0));
    return B200_OK;
}

int32_t b200_host_unregister(void* ptr) {
    if (!ptr) return B200_OK;
    B200_CUDA(cudaHostUnregister(ptr));
    return B200_OK;
}

}  // extern "C"


// ---- graphs --------------------------------------------------------------------------------------------
// Capture / instantiate / launch / update, the operations of src/hip/graph.jl:16-168.  Every
// operator of this library can be captured: they only enqueue kernels and memsets on the stream
// they are given.  The one host-side state an operator may change is the stream's scratch
// buffer; it cannot grow inside a capture (see scratch()), so an operation is run once before it
// is captured - what the reference's @captured does anyway when its first capture fails.
struct b200_graph_s { int dev; cudaGraph_t g; };
struct b200_graph_exec_s { int dev; cudaGraphExec_t e; };

extern "C" int32_t b200_graph_capture_begin(b200_stream_t st, int32_t mode) {
    B200_TRY(enter(st));
    if (mode < 0 || mode > 2) return fail(B200_INVALID_ARG, "capture mode must be 0 (global), 1 (thread local) or 2 (relaxed)");
    const cudaStreamCaptureMode m = mode == 0 ? cudaStreamCaptureModeGlobal
                                   : mode == 1 ? cudaStreamCaptureModeThreadLocal : cudaStreamCaptureModeRelaxed;
    B200_CUDA(cudaStreamBeginCapture(st->s, m));
    return B200_OK;
}

extern "C" int32_t b200_graph_capture_end(b200_stream_t st, b200_graph_t* out) {
    if (!out) return fail(B200_INVALID_ARG, "null output");
    *out = nullptr;
    B200_TRY(enter(st));
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(st->s, &g);
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (g) cudaGraphDestroy(g);
        return cuda_fail(e, "ending the stream capture (a call that cannot be captured invalidates it)");
    }
    *out = new b200_graph_s{st->dev, g};
    return B200_OK;
}

extern "C" int32_t b200_stream_is_capturing(b200_stream_t st, int32_t* out) {
    if (!out) return fail(B200_INVALID_ARG, "null output");
    B200_TRY(enter(st));
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    B200_CUDA(cudaStreamIsCapturing(st->s, &cap));
    *out = cap != cudaStreamCaptureStatusNone ? 1 : 0;
    return B200_OK;
}

extern "C" int32_t b200_graph_destroy(b200_graph_t g) {
    if (!g) return B200_OK;
    DeviceState* d;
    B200_TRY(device_state(g->dev, &d));
    cudaError_t e = cudaGraphDestroy(g->g);
    delete g;
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphDestroy");
    return B200_OK;
}

extern "C" int32_t b200_graph_instantiate(b200_graph_t g, b200_graph_exec_t* out) {
    if (!g || !out) return fail(B200_INVALID_ARG, "null graph or output");
    DeviceState* d;
    B200_TRY(device_state(g->dev, &d));
    cudaGraphExec_t e = nullptr;
    // allocations captured without their free are released when the graph is launched again
    B200_CUDA(cudaGraphInstantiateWithFlags(&e, g->g, cudaGraphInstantiateFlagAutoFreeOnLaunch));
    *out = new b200_graph_exec_s{g->dev, e};
    return B200_OK;
}

extern "C" int32_t b200_graph_exec_destroy(b200_graph_exec_t e) {
    if (!e) return B200_OK;
    DeviceState* d;
    B200_TRY(device_state(e->dev, &d));
    cudaError_t err = cudaGraphExecDestroy(e->e);
    delete e;
    if (err != cudaSuccess) return cuda_fail(err, "cudaGraphExecDestroy");
    return B200_OK;
}

extern "C" int32_t b200_graph_launch(b200_graph_exec_t e, b200_stream_t st) {
    if (!e) return fail(B200_INVALID_ARG, "null executable graph");
    B200_TRY(enter(st));
    if (st->dev != e->dev) return fail(B200_INVALID_ARG, "graph of device %d launched on a stream of device %d", e->dev, st->dev);
    B200_CUDA(cudaGraphLaunch(e->e, st->s));
    return B200_OK;
}

extern "C" int32_t b200_graph_exec_update(b200_graph_exec_t e, b200_graph_t g, int32_t* updated) {
    if (!e || !g || !updated) return fail(B200_INVALID_ARG, "null argument");
    *updated = 0;
    DeviceState* d;
    B200_TRY(device_state(e->dev, &d));
    cudaGraphExecUpdateResultInfo info{};
    cudaError_t err = cudaGraphExecUpdate(e->e, g->g, &info);
    if (err == cudaSuccess && info.result == cudaGraphExecUpdateSuccess) { *updated = 1; return B200_OK; }
    cudaGetLastError();
    if (err == cudaErrorGraphExecUpdateFailure || err == cudaSuccess) return B200_OK;   // topology differs: not an error, *updated stays 0
    return cuda_fail(err, "cudaGraphExecUpdate");
}
