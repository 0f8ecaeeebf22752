// Peer exchange buffers for the fused reduce + all-reduce (one process per GPU).
//
// Every rank allocates a few hundred bytes of slots with cudaMalloc, exports them with a CUDA IPC
// handle, and maps the buffers of all other ranks (NVLink peer access through NVSwitch).  The
// reduction kernel's last block then stores its partial straight into every rank's slots and
// reads the partials of the others from its own buffer - no separate collective launch, no host
// round trip.  Plain peer stores and loads only.
// The reference has nothing comparable (no collective layer at all).
#include "common.cuh"

#include <cstring>

struct b200_peer_s {
    int       dev, rank, nranks;
    PeerSlot* local;                 // own buffer: [2 banks][kMaxPeers]
    PeerSlot* mapped[kMaxPeers];     // every rank's buffer as seen from this process
    bool      opened[kMaxPeers];
    uint64_t  seq;
};

namespace b200 {

int32_t peer_next_context(b200_peer_t p, b200_stream_t st, PeerCtx* out) {
    if (!st) return fail(B200_INVALID_ARG, "null stream handle");
    if (st->dev != p->dev) return fail(B200_INVALID_ARG, "stream and peer group live on different devices");
    for (int r = 0; r < p->nranks; ++r)
        if (!p->mapped[r]) return fail(B200_NOT_INITIALISED, "peer group is not connected yet (b200_peer_connect)");
    out->nranks = p->nranks;
    out->rank = p->rank;
    out->seq = ++p->seq;
    out->max_polls = 1u << 26;       // with back-off this is on the order of ten seconds
    out->err_word = device_error_word(p->dev);
    for (int r = 0; r < kMaxPeers; ++r) out->bufs[r] = r < p->nranks ? p->mapped[r] : nullptr;
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int32_t b200_peer_create(int32_t dev, int32_t rank, int32_t nranks, b200_peer_t* out, uint8_t handle_out[64]) {
    if (!out || !handle_out) return fail(B200_INVALID_ARG, "null output");
    if (nranks < 1 || nranks > kMaxPeers || rank < 0 || rank >= nranks)
        return fail(B200_INVALID_ARG, "peer group of %d ranks (at most %d), rank %d", nranks, kMaxPeers, rank);
    B200_TRY(b200_init());
    B200_CUDA(cudaSetDevice(dev));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "unexpected IPC handle size");
    PeerSlot* buf = nullptr;
    const size_t bytes = sizeof(PeerSlot) * 2 * kMaxPeers;
    B200_CUDA(cudaMalloc((void**)&buf, bytes));
    B200_CUDA(cudaMemset(buf, 0, bytes));
    B200_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, buf);
    if (e != cudaSuccess) { cudaFree(buf); return cuda_fail(e, "cudaIpcGetMemHandle"); }
    memcpy(handle_out, &h, 64);
    b200_peer_s* p = new b200_peer_s{};
    p->dev = dev; p->rank = rank; p->nranks = nranks; p->local = buf; p->seq = 0;
    p->mapped[rank] = buf;
    *out = p;
    return B200_OK;
}

extern "C" int32_t b200_peer_connect(b200_peer_t p, const uint8_t* handles) {
    if (!p || !handles) return fail(B200_INVALID_ARG, "null argument");
    B200_CUDA(cudaSetDevice(p->dev));
    for (int r = 0; r < p->nranks; ++r) {
        if (r == p->rank || p->mapped[r]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + 64 * r, 64);
        void* ptr = nullptr;
        B200_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        p->mapped[r] = reinterpret_cast<PeerSlot*>(ptr);
        p->opened[r] = true;
    }
    return B200_OK;
}

extern "C" int32_t b200_peer_destroy(b200_peer_t p) {
    if (!p) return B200_OK;
    cudaSetDevice(p->dev);
    cudaDeviceSynchronize();
    for (int r = 0; r < p->nranks; ++r)
        if (p->opened[r] && p->mapped[r]) cudaIpcCloseMemHandle(p->mapped[r]);
    if (p->local) cudaFree(p->local);
    cudaGetLastError();
    delete p;
    return B200_OK;
}
