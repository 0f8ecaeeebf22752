// Exchange buffers for the fused reduce + all-reduce (one process per GPU).
//
// Every rank owns a few hundred bytes of slots that all ranks of the group can write.  The
// reduction kernel's last block stores its partial straight into every rank's slots and reads the
// partials of the others from its own buffer - no separate collective launch, no host round trip.
// Plain one-to-one stores and loads only (system-scope fences, no library kernel on peer memory).
//
// Three transports place the slots differently; the kernel code is the same for all:
//   * B200_PEER_HOST: the slots live in POSIX shared memory that every rank registers with the
//     CUDA runtime (pinned + mapped).  Stores and polls cross PCIe to host memory (a few
//     microseconds); no GPU ever maps another GPU's memory.
//   * B200_PEER_VMM: the slots are ONE 2 MiB device allocation made with the driver's
//     virtual-memory calls and exported as a file descriptor; each peer maps exactly that
//     allocation (NVLink through NVSwitch).  Peer access is granted per mapping, never device wide.
//   * B200_PEER_IPC: cudaMalloc + CUDA IPC handle.  Opening the handle switches peer access on for
//     the whole device (cudaIpcMemLazyEnablePeerAccess).
// The reference has nothing comparable (no collective layer at all).
#include "common.cuh"

#include <cuda.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstdio>
#include <cstring>

namespace {

constexpr size_t kSlotBytes = sizeof(PeerSlot) * 2 * kMaxPeers;
constexpr size_t kHostBytes = 4096;            // one page of shared memory per rank
constexpr uint32_t kVmmMagic = 0x314d4d56u;    // "VMM1"

struct VmmHandle {            // what b200_peer_create writes into handle_out for B200_PEER_VMM
    uint32_t magic;
    int32_t  pid;             // process in which `fd` is valid
    int32_t  fd;
    int32_t  reserved;
    uint64_t bytes;
};
static_assert(sizeof(VmmHandle) <= 64, "handle must fit the 64-byte slot");

struct Mapping {              // one rank's buffer as seen from this process
    PeerSlot* dev = nullptr;  // pointer kernels use
    void*     host = nullptr; // HOST: the mmap'ed page
    CUdeviceptr va = 0;       // VMM: reserved range
    CUmemGenericAllocationHandle mem = 0;
    size_t    bytes = 0;
    bool      live = false;
};

// The driver's virtual-memory entry points, looked up through the runtime (the library does not
// link against libcuda).
struct VmmApi {
    decltype(&cuMemCreate) Create = nullptr;
    decltype(&cuMemRelease) Release = nullptr;
    decltype(&cuMemAddressReserve) Reserve = nullptr;
    decltype(&cuMemAddressFree) Free = nullptr;
    decltype(&cuMemMap) Map = nullptr;
    decltype(&cuMemUnmap) Unmap = nullptr;
    decltype(&cuMemSetAccess) SetAccess = nullptr;
    decltype(&cuMemGetAllocationGranularity) Granularity = nullptr;
    decltype(&cuMemExportToShareableHandle) Export = nullptr;
    decltype(&cuMemImportFromShareableHandle) Import = nullptr;
    bool ok = false;
};

static int32_t vmm_api(VmmApi* api) {
    static VmmApi cached;
    static std::atomic<int> state{0};     // 0 unknown, 1 ready, 2 unavailable
    if (state.load() == 0) {
        VmmApi a;
        bool good = true;
        auto get = [&](const char* name, void** fn) {
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !*fn) {
                cudaGetLastError();
                good = false;
            }
        };
        get("cuMemCreate", (void**)&a.Create);
        get("cuMemRelease", (void**)&a.Release);
        get("cuMemAddressReserve", (void**)&a.Reserve);
        get("cuMemAddressFree", (void**)&a.Free);
        get("cuMemMap", (void**)&a.Map);
        get("cuMemUnmap", (void**)&a.Unmap);
        get("cuMemSetAccess", (void**)&a.SetAccess);
        get("cuMemGetAllocationGranularity", (void**)&a.Granularity);
        get("cuMemExportToShareableHandle", (void**)&a.Export);
        get("cuMemImportFromShareableHandle", (void**)&a.Import);
        a.ok = good;
        cached = a;
        state.store(good ? 1 : 2);
    }
    if (state.load() != 1) return b200::fail(B200_UNSUPPORTED, "the driver's virtual-memory calls (cuMemCreate ...) are not available");
    *api = cached;
    return B200_OK;
}

#define B200_CU(expr)                                                                             \
    do {                                                                                          \
        CUresult _r = (expr);                                                                     \
        if (_r != CUDA_SUCCESS) return b200::fail(B200_CUDA_ERROR, "driver error %d in %s", (int)_r, #expr); \
    } while (0)

static CUmemAllocationProp vmm_prop(int dev) {
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

// Maps `mem` into this process for device `dev` (read + write).
static int32_t vmm_map(const VmmApi& api, int dev, CUmemGenericAllocationHandle mem, size_t bytes, Mapping* m) {
    CUdeviceptr va = 0;
    B200_CU(api.Reserve(&va, bytes, 0, 0, 0));
    CUresult r = api.Map(va, bytes, 0, mem, 0);
    if (r != CUDA_SUCCESS) { api.Free(va, bytes); return b200::fail(B200_CUDA_ERROR, "driver error %d in cuMemMap", (int)r); }
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = dev;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = api.SetAccess(va, bytes, &acc, 1);
    if (r != CUDA_SUCCESS) {
        api.Unmap(va, bytes);
        api.Free(va, bytes);
        return b200::fail(B200_CUDA_ERROR, "driver error %d in cuMemSetAccess (is peer access between the devices possible?)", (int)r);
    }
    m->va = va;
    m->mem = mem;
    m->bytes = bytes;
    m->dev = reinterpret_cast<PeerSlot*>(va);
    m->live = true;
    return B200_OK;
}

static std::atomic<unsigned> g_shm_counter{0};

}  // namespace

struct b200_peer_s {
    int       dev, rank, nranks, transport;
    Mapping   map[kMaxPeers];        // every rank's buffer as seen from this process
    char      shm_name[64];          // HOST: name of this rank's own segment
    int       export_fd;             // VMM: descriptor handed out in the handle (closed at destroy)
    uint64_t  seq;
    uint32_t  max_polls;
};

namespace b200 {

int32_t peer_next_context(b200_peer_t p, b200_stream_t st, PeerCtx* out) {
    if (!st) return fail(B200_INVALID_ARG, "null stream handle");
    if (st->dev != p->dev) return fail(B200_INVALID_ARG, "stream and peer group live on different devices");
    for (int r = 0; r < p->nranks; ++r)
        if (!p->map[r].dev) return fail(B200_NOT_INITIALISED, "peer group is not connected yet (b200_peer_connect)");
    out->nranks = p->nranks;
    out->rank = p->rank;
    out->seq = ++p->seq;
    out->max_polls = p->max_polls;
    out->err_word = device_error_word(p->dev);
    for (int r = 0; r < kMaxPeers; ++r) out->bufs[r] = r < p->nranks ? p->map[r].dev : nullptr;
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int32_t b200_peer_create(int32_t dev, int32_t rank, int32_t nranks, int32_t transport, b200_peer_t* out,
                                    uint8_t handle_out[64]) {
    if (!out || !handle_out) return fail(B200_INVALID_ARG, "null output");
    *out = nullptr;
    if (nranks < 1 || nranks > kMaxPeers || rank < 0 || rank >= nranks)
        return fail(B200_INVALID_ARG, "peer group of %d ranks (at most %d), rank %d", nranks, kMaxPeers, rank);
    if (transport < B200_PEER_HOST || transport > B200_PEER_IPC) return fail(B200_INVALID_ARG, "unknown peer transport %d", transport);
    B200_TRY(b200_init());
    B200_CUDA(cudaSetDevice(dev));
    B200_CUDA(cudaFree(nullptr));             // make sure the device's context exists
    memset(handle_out, 0, 64);
    b200_peer_s* p = new b200_peer_s{};
    p->dev = dev; p->rank = rank; p->nranks = nranks; p->transport = transport;
    p->seq = 0; p->export_fd = -1;
    p->max_polls = 1u << 26;                  // with back-off this is on the order of ten seconds
    Mapping& own = p->map[rank];
    int32_t status = B200_OK;
    if (transport == B200_PEER_HOST) {
        snprintf(p->shm_name, sizeof p->shm_name, "/b200peer-%d-%u-%d", (int)getpid(), g_shm_counter.fetch_add(1), rank);
        const int fd = shm_open(p->shm_name, O_CREAT | O_EXCL | O_RDWR, 0600);
        if (fd < 0) status = fail(B200_CUDA_ERROR, "shm_open(%s) failed: %s", p->shm_name, strerror(errno));
        if (status == B200_OK && ftruncate(fd, (off_t)kHostBytes) != 0) status = fail(B200_CUDA_ERROR, "ftruncate on %s failed: %s", p->shm_name, strerror(errno));
        void* page = MAP_FAILED;
        if (status == B200_OK) {
            page = mmap(nullptr, kHostBytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
            if (page == MAP_FAILED) status = fail(B200_CUDA_ERROR, "mmap of %s failed: %s", p->shm_name, strerror(errno));
        }
        if (fd >= 0) close(fd);
        if (status == B200_OK) {
            memset(page, 0, kHostBytes);
            cudaError_t e = cudaHostRegister(page, kHostBytes, cudaHostRegisterPortable | cudaHostRegisterMapped);
            void* dptr = nullptr;
            if (e == cudaSuccess) e = cudaHostGetDevicePointer(&dptr, page, 0);
            if (e != cudaSuccess) { munmap(page, kHostBytes); status = cuda_fail(e, "registering the exchange page"); }
            else { own.host = page; own.dev = reinterpret_cast<PeerSlot*>(dptr); own.bytes = kHostBytes; own.live = true; }
        }
        if (status != B200_OK && p->shm_name[0]) shm_unlink(p->shm_name);
        if (status == B200_OK) memcpy(handle_out, p->shm_name, strlen(p->shm_name) + 1);
    } else if (transport == B200_PEER_VMM) {
        VmmApi api;
        status = vmm_api(&api);
        if (status == B200_OK) {
            status = [&]() -> int32_t {
                CUmemAllocationProp prop = vmm_prop(dev);
                size_t gran = 0;
                B200_CU(api.Granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM));
                const size_t bytes = (kSlotBytes + gran - 1) / gran * gran;
                CUmemGenericAllocationHandle mem = 0;
                B200_CU(api.Create(&mem, bytes, &prop, 0));
                int32_t s = vmm_map(api, dev, mem, bytes, &own);
                if (s != B200_OK) { api.Release(mem); return s; }
                B200_CUDA(cudaMemset(own.dev, 0, kSlotBytes));
                B200_CUDA(cudaDeviceSynchronize());
                int fd = -1;
                B200_CU(api.Export(&fd, mem, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
                p->export_fd = fd;
                VmmHandle h{kVmmMagic, (int32_t)getpid(), fd, 0, (uint64_t)bytes};
                memcpy(handle_out, &h, sizeof h);
                return B200_OK;
            }();
        }
    } else {
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "unexpected IPC handle size");
        status = [&]() -> int32_t {
            PeerSlot* buf = nullptr;
            B200_CUDA(cudaMalloc((void**)&buf, kSlotBytes));
            own.dev = buf; own.bytes = kSlotBytes; own.live = true;
            B200_CUDA(cudaMemset(buf, 0, kSlotBytes));
            B200_CUDA(cudaDeviceSynchronize());
            cudaIpcMemHandle_t h;
            B200_CUDA(cudaIpcGetMemHandle(&h, buf));
            memcpy(handle_out, &h, 64);
            return B200_OK;
        }();
    }
    if (status != B200_OK) {
        b200_peer_destroy(p);
        return status;
    }
    *out = p;
    return B200_OK;
}

extern "C" int32_t b200_peer_connect(b200_peer_t p, const uint8_t* handles) {
    if (!p || !handles) return fail(B200_INVALID_ARG, "null argument");
    B200_CUDA(cudaSetDevice(p->dev));
    for (int r = 0; r < p->nranks; ++r) {
        if (r == p->rank || p->map[r].dev) continue;
        const uint8_t* hb = handles + 64 * r;
        Mapping& m = p->map[r];
        if (p->transport == B200_PEER_HOST) {
            char name[64];
            memcpy(name, hb, 64);
            name[63] = 0;
            if (strncmp(name, "/b200peer-", 10) != 0) return fail(B200_INVALID_ARG, "handle of rank %d is not a shared-memory name", r);
            const int fd = shm_open(name, O_RDWR, 0600);
            if (fd < 0) return fail(B200_CUDA_ERROR, "shm_open(%s) failed: %s", name, strerror(errno));
            void* page = mmap(nullptr, kHostBytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
            close(fd);
            if (page == MAP_FAILED) return fail(B200_CUDA_ERROR, "mmap of %s failed: %s", name, strerror(errno));
            cudaError_t e = cudaHostRegister(page, kHostBytes, cudaHostRegisterPortable | cudaHostRegisterMapped);
            void* dptr = nullptr;
            if (e == cudaSuccess) e = cudaHostGetDevicePointer(&dptr, page, 0);
            if (e != cudaSuccess) { munmap(page, kHostBytes); return cuda_fail(e, "registering a peer's exchange page"); }
            m.host = page; m.dev = reinterpret_cast<PeerSlot*>(dptr); m.bytes = kHostBytes; m.live = true;
        } else if (p->transport == B200_PEER_VMM) {
            VmmHandle h;
            memcpy(&h, hb, sizeof h);
            if (h.magic != kVmmMagic) return fail(B200_INVALID_ARG, "handle of rank %d is not a virtual-memory export", r);
            VmmApi api;
            B200_TRY(vmm_api(&api));
            int fd = -1;
            if (h.pid == (int32_t)getpid()) {
                fd = dup(h.fd);       // already valid here (passed over a Unix socket by the host code)
                if (fd < 0) return fail(B200_INVALID_ARG, "descriptor %d in the handle of rank %d is not open in this process", h.fd, r);
            } else {
                // fetch the descriptor from the exporting process (needs permission to inspect it)
                const int pidfd = (int)syscall(SYS_pidfd_open, (pid_t)h.pid, 0u);
                if (pidfd >= 0) {
                    fd = (int)syscall(SYS_pidfd_getfd, pidfd, h.fd, 0u);
                    close(pidfd);
                }
                if (fd < 0)
                    return fail(B200_UNSUPPORTED, "cannot take descriptor %d from process %d (%s): pass it over a Unix socket "
                                "(SCM_RIGHTS) and put the received descriptor and this process id into the handle",
                                h.fd, h.pid, strerror(errno));
            }
            CUmemGenericAllocationHandle mem = 0;
            CUresult cr = api.Import(&mem, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            close(fd);
            if (cr != CUDA_SUCCESS) return fail(B200_CUDA_ERROR, "driver error %d in cuMemImportFromShareableHandle", (int)cr);
            int32_t s = vmm_map(api, p->dev, mem, (size_t)h.bytes, &m);
            if (s != B200_OK) { api.Release(mem); return s; }
        } else {
            cudaIpcMemHandle_t h;
            memcpy(&h, hb, 64);
            void* ptr = nullptr;
            B200_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
            m.dev = reinterpret_cast<PeerSlot*>(ptr);
            m.live = true;
        }
    }
    return B200_OK;
}

extern "C" int32_t b200_peer_set_poll_budget(b200_peer_t p, uint32_t polls) {
    if (!p) return fail(B200_INVALID_ARG, "null peer group");
    if (polls == 0) return fail(B200_INVALID_ARG, "the poll budget must be positive");
    p->max_polls = polls;
    return B200_OK;
}

extern "C" int32_t b200_peer_info(b200_peer_t p, int32_t* transport, uint64_t* seq) {
    if (!p) return fail(B200_INVALID_ARG, "null peer group");
    if (transport) *transport = p->transport;
    if (seq) *seq = p->seq;
    return B200_OK;
}

// Every rank has mapped every buffer: the names the mappings were found by are not needed any
// more.  Removing them now means a process that dies later leaves no file in /dev/shm and no open
// descriptor behind; the mappings themselves live until b200_peer_destroy.
extern "C" int32_t b200_peer_seal(b200_peer_t p) {
    if (!p) return fail(B200_INVALID_ARG, "null peer group");
    if (p->transport == B200_PEER_HOST && p->shm_name[0]) {
        shm_unlink(p->shm_name);
        p->shm_name[0] = 0;
    }
    if (p->export_fd >= 0) {
        close(p->export_fd);
        p->export_fd = -1;
    }
    return B200_OK;
}

extern "C" int32_t b200_peer_destroy(b200_peer_t p) {
    if (!p) return B200_OK;
    cudaSetDevice(p->dev);
    cudaDeviceSynchronize();
    VmmApi api;
    const bool have_vmm = p->transport == B200_PEER_VMM && vmm_api(&api) == B200_OK;
    for (int r = 0; r < kMaxPeers; ++r) {
        Mapping& m = p->map[r];
        if (!m.live) continue;
        if (p->transport == B200_PEER_HOST) {
            cudaHostUnregister(m.host);
            munmap(m.host, m.bytes);
        } else if (p->transport == B200_PEER_VMM) {
            if (have_vmm) {
                api.Unmap(m.va, m.bytes);
                api.Free(m.va, m.bytes);
                api.Release(m.mem);
            }
        } else if (r == p->rank) {
            cudaFree(m.dev);
        } else {
            cudaIpcCloseMemHandle(m.dev);
        }
        m = Mapping{};
    }
    if (p->transport == B200_PEER_HOST && p->shm_name[0]) shm_unlink(p->shm_name);
    if (p->export_fd >= 0) close(p->export_fd);
    cudaGetLastError();
    delete p;
    return B200_OK;
}
