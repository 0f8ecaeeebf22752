// Collective layer for the sharded operators: one process per GPU, NCCL over NVLink/NVSwitch.
// The reference has no collective backend at all (multi-GPU there is one task per device with
// copies through the host, docs/src/usage/multitasking.md:37-53), so these entry points are
// additions, not replacements.  NCCL is resolved with dlopen at first use: a process that
// already loaded a NCCL (for instance through torch.distributed) shares that copy, and a
// single-GPU user never needs the library to be present.
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>

struct b200_comm_s {
    ncclComm_t comm;
    int dev, rank, nranks;
};

namespace b200 {

struct NcclApi {
    void* handle = nullptr;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclAllReduce) AllReduce = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
    decltype(&ncclCommAbort) CommAbort = nullptr;
};
static NcclApi g_nccl;
static std::mutex g_nccl_mu;

static int32_t load_nccl() {
    std::lock_guard<std::mutex> lk(g_nccl_mu);
    if (g_nccl.handle) return B200_OK;
    // B200_NCCL_LIB names the library to load instead of the system's (a path or a soname)
    const char* names[] = {getenv("B200_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* nm : names) {
        if (!nm || !nm[0]) continue;
        h = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return fail(B200_NCCL_ERROR, "cannot load libnccl.so.2: %s", dlerror());
#define B200_SYM(field, name)                                                         \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name));          \
    if (!g_nccl.field) return fail(B200_NCCL_ERROR, "libnccl lacks symbol %s", name);
    B200_SYM(GetUniqueId, "ncclGetUniqueId")
    B200_SYM(CommInitRank, "ncclCommInitRank")
    B200_SYM(CommDestroy, "ncclCommDestroy")
    B200_SYM(AllReduce, "ncclAllReduce")
    B200_SYM(AllGather, "ncclAllGather")
    B200_SYM(GetErrorString, "ncclGetErrorString")
    B200_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
    B200_SYM(CommAbort, "ncclCommAbort")
#undef B200_SYM
    g_nccl.handle = h;
    return B200_OK;
}

static int32_t nccl_fail(ncclResult_t r, const char* what) {
    return fail(B200_NCCL_ERROR, "NCCL error %d (%s) in %s", (int)r, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?", what);
}
#define B200_NCCL(expr)                                            \
    do {                                                           \
        ncclResult_t _r = (expr);                                  \
        if (_r != ncclSuccess) return nccl_fail(_r, #expr);        \
    } while (0)

static int32_t nccl_dtype(int32_t dt, ncclDataType_t* out) {
    switch (dt) {
        case B200_I8: *out = ncclInt8; break;
        case B200_U8: case B200_BOOL: *out = ncclUint8; break;
        case B200_I32: *out = ncclInt32; break;
        case B200_U32: *out = ncclUint32; break;
        case B200_I64: *out = ncclInt64; break;
        case B200_U64: *out = ncclUint64; break;
        case B200_F16: *out = ncclFloat16; break;
        case B200_BF16: *out = ncclBfloat16; break;
        case B200_F32: *out = ncclFloat32; break;
        case B200_F64: *out = ncclFloat64; break;
        default: return fail(B200_UNSUPPORTED, "collective: element type %d is not supported", dt);
    }
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int32_t b200_comm_unique_id(uint8_t id_out[128]) {
    if (!id_out) return fail(B200_INVALID_ARG, "null output");
    B200_TRY(load_nccl());
    ncclUniqueId id;
    static_assert(sizeof(ncclUniqueId) == 128, "unexpected ncclUniqueId size");
    B200_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(id_out, &id, 128);
    return B200_OK;
}

extern "C" int32_t b200_comm_init_rank(b200_comm_t* out, int32_t nranks, int32_t rank, const uint8_t id[128], int32_t dev) {
    if (!out || !id) return fail(B200_INVALID_ARG, "null argument");
    if (nranks < 1 || rank < 0 || rank >= nranks) return fail(B200_INVALID_ARG, "rank %d outside [0,%d)", rank, nranks);
    B200_TRY(load_nccl());
    if (dev >= 0) B200_CUDA(cudaSetDevice(dev));      // dev < 0: not bound to a device (health checks only)
    ncclUniqueId uid;
    memcpy(&uid, id, 128);
    ncclComm_t c;
    B200_NCCL(g_nccl.CommInitRank(&c, nranks, uid, rank));
    *out = new b200_comm_s{c, dev, rank, nranks};
    return B200_OK;
}

extern "C" int32_t b200_comm_destroy(b200_comm_t comm) {
    if (!comm) return B200_OK;
    if (comm->dev >= 0) cudaSetDevice(comm->dev);
    ncclResult_t r = comm->comm ? g_nccl.CommDestroy(comm->comm) : ncclSuccess;   // an aborted communicator is already gone
    delete comm;
    if (r != ncclSuccess) return nccl_fail(r, "ncclCommDestroy");
    return B200_OK;
}

// Failure detection for the collectives, on the host: NCCL reports a failed peer or transport
// through ncclCommGetAsyncError, and a collective whose peer never arrives simply never ends.
// This call watches both until the stream has drained or `timeout_ms` has passed; on an error or
// a timeout it aborts the communicator (ncclCommAbort: the stuck kernel leaves the GPU, the
// stream becomes usable again) and reports B200_NCCL_ERROR.  Afterwards the communicator only
// accepts b200_comm_destroy.  The reference's closest relative is the one-second watchdog on a
// stream that does not finish (src/hip/stream.jl:99-126).
extern "C" int32_t b200_comm_check(b200_comm_t comm, b200_stream_t st, int32_t timeout_ms) {
    if (!comm) return fail(B200_INVALID_ARG, "null communicator");
    if (!comm->comm) return fail(B200_NCCL_ERROR, "the communicator was aborted");
    if (st) {
        B200_TRY(enter(st));
        if (st->dev != comm->dev) return fail(B200_INVALID_ARG, "stream and communicator live on different devices");
    }
    const auto t0 = std::chrono::steady_clock::now();
    while (true) {
        ncclResult_t async = ncclSuccess;
        ncclResult_t r = g_nccl.CommGetAsyncError(comm->comm, &async);
        if (r != ncclSuccess) async = r;
        if (async != ncclSuccess && async != ncclInProgress) {
            g_nccl.CommAbort(comm->comm);
            comm->comm = nullptr;
            return nccl_fail(async, "a collective in flight (communicator aborted)");
        }
        bool done = true;
        if (st) {
            cudaError_t e = cudaStreamQuery(st->s);
            if (e == cudaErrorNotReady) { cudaGetLastError(); done = false; }
            else if (e != cudaSuccess) return cuda_fail(e, "cudaStreamQuery");
        }
        if (done && async == ncclSuccess) return B200_OK;
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms >= timeout_ms) {
            if (!st && async == ncclInProgress) return B200_NOT_READY;
            g_nccl.CommAbort(comm->comm);
            comm->comm = nullptr;
            return fail(B200_NCCL_ERROR, "collective did not finish within %d ms: a rank is missing or stuck (communicator aborted)", timeout_ms);
        }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
}

extern "C" int32_t b200_allreduce(b200_comm_t comm, void* buf, size_t count, int32_t dtype, int32_t op, b200_stream_t st) {
    if (!comm) return fail(B200_INVALID_ARG, "null communicator");
    if (!comm->comm) return fail(B200_NCCL_ERROR, "the communicator was aborted");
    B200_TRY(enter(st));
    if (st->dev != comm->dev) return fail(B200_INVALID_ARG, "stream and communicator live on different devices");
    if (op < 0 || op >= B200_RED_COUNT) return fail(B200_UNSUPPORTED, "allreduce: unknown operator %d", op);
    ncclDataType_t dt;
    B200_TRY(nccl_dtype(dtype, &dt));
    const ncclRedOp_t ops[4] = {ncclSum, ncclProd, ncclMax, ncclMin};
    B200_NCCL(g_nccl.AllReduce(buf, buf, count, dt, ops[op], comm->comm, st->s));
    return B200_OK;
}

extern "C" int32_t b200_allgather(b200_comm_t comm, const void* send, void* recv, size_t count, int32_t dtype, b200_stream_t st) {
    if (!comm) return fail(B200_INVALID_ARG, "null communicator");
    if (!comm->comm) return fail(B200_NCCL_ERROR, "the communicator was aborted");
    B200_TRY(enter(st));
    if (st->dev != comm->dev) return fail(B200_INVALID_ARG, "stream and communicator live on different devices");
    ncclDataType_t dt;
    B200_TRY(nccl_dtype(dtype, &dt));
    B200_NCCL(g_nccl.AllGather(send, recv, count, dt, comm->comm, st->s));
    return B200_OK;
}
