/* A stand-in for libnccl used by tests/test_comm_check.py: the entry points libb200arrays.so
 * resolves, with a scripted health state instead of a network.  No GPU, no peers.
 * stub_script(code): what ncclCommGetAsyncError reports from now on (0 success, 7 in progress,
 * 6 remote error ...).  stub_aborts(): how often ncclCommAbort was called. */
#include <string.h>

typedef int ncclResult_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef void* ncclComm_t;

static int g_async = 0;
static int g_aborts = 0;
static int g_destroys = 0;
static int g_comm_storage;

void stub_script(int code) { g_async = code; }
int stub_aborts(void) { return g_aborts; }
int stub_destroys(void) { return g_destroys; }

ncclResult_t ncclGetUniqueId(ncclUniqueId* id) { memset(id, 7, sizeof *id); return 0; }
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank) {
    (void)nranks; (void)id; (void)rank;
    *comm = &g_comm_storage;
    return 0;
}
ncclResult_t ncclCommDestroy(ncclComm_t comm) { (void)comm; ++g_destroys; return 0; }
ncclResult_t ncclCommAbort(ncclComm_t comm) { (void)comm; ++g_aborts; return 0; }
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* async) { (void)comm; *async = g_async; return 0; }
ncclResult_t ncclAllReduce(const void* s, void* r, size_t n, int dt, int op, ncclComm_t c, void* st) {
    (void)s; (void)r; (void)n; (void)dt; (void)op; (void)c; (void)st; return 0;
}
ncclResult_t ncclAllGather(const void* s, void* r, size_t n, int dt, ncclComm_t c, void* st) {
    (void)s; (void)r; (void)n; (void)dt; (void)c; (void)st; return 0;
}
const char* ncclGetErrorString(ncclResult_t r) {
    switch (r) {
        case 0: return "no error";
        case 6: return "remote process exited or there was a network error";
        case 7: return "NCCL operation in progress";
        default: return "stub error";
    }
}
