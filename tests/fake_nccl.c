/* Stand-in for libnccl.so.2 for the host-side failure tests of the gather layer (no GPU, no
 * network).  It plays the other ranks: FAKE_NCCL_MODE = "ok" (everybody joins at once),
 * "late" (joins after 150 ms of polling), "never" (a rank never arrives: the init stays in
 * progress for ever), "fail" (the init reports an asynchronous system error).  It counts the
 * calls so that the test can see that a communicator which timed out was aborted. */
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef void* ncclComm_t;
typedef int ncclResult_t;       /* 0 success, 2 system error, 7 in progress */
typedef struct { size_t size; unsigned magic; unsigned version; int blocking; } fake_config_head;

static int n_init, n_abort, n_destroy, n_poll;
static struct timespec t_init;
static int comm_storage;

static const char* mode(void) { const char* m = getenv("FAKE_NCCL_MODE"); return m ? m : "ok"; }

__attribute__((visibility("default"))) int fake_nccl_count(int which)
{
    return which == 0 ? n_init : which == 1 ? n_abort : which == 2 ? n_destroy : n_poll;
}
__attribute__((visibility("default"))) void fake_nccl_reset(void) { n_init = n_abort = n_destroy = n_poll = 0; }

__attribute__((visibility("default"))) ncclResult_t ncclGetUniqueId(ncclUniqueId* id) { memset(id, 0x5a, sizeof *id); return 0; }

__attribute__((visibility("default"))) ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, void* config)
{
    (void)nranks; (void)id; (void)rank;
    ++n_init;
    if (!config || ((fake_config_head*)config)->blocking != 0) return 4;      /* the library must ask for a non-blocking communicator */
    clock_gettime(CLOCK_MONOTONIC, &t_init);
    *comm = &comm_storage;
    return strcmp(mode(), "ok") == 0 ? 0 : 7;
}

__attribute__((visibility("default"))) ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* st)
{
    (void)comm;
    ++n_poll;
    const char* m = mode();
    if (strcmp(m, "never") == 0) *st = 7;
    else if (strcmp(m, "fail") == 0) *st = 2;
    else if (strcmp(m, "late") == 0) {
        struct timespec now; clock_gettime(CLOCK_MONOTONIC, &now);
        const double ms = (now.tv_sec - t_init.tv_sec) * 1e3 + (now.tv_nsec - t_init.tv_nsec) / 1e6;
        *st = ms < 150.0 ? 7 : 0;
    } else *st = 0;
    return 0;
}

__attribute__((visibility("default"))) ncclResult_t ncclCommAbort(ncclComm_t comm) { (void)comm; ++n_abort; return 0; }
__attribute__((visibility("default"))) ncclResult_t ncclCommDestroy(ncclComm_t comm) { (void)comm; ++n_destroy; return 0; }
__attribute__((visibility("default"))) ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* out, void* config)
{
    (void)comm; (void)color; (void)key; (void)config;
    *out = &comm_storage;
    return 0;
}
__attribute__((visibility("default"))) ncclResult_t ncclGroupStart(void) { return 0; }
__attribute__((visibility("default"))) ncclResult_t ncclGroupEnd(void) { return 0; }
__attribute__((visibility("default"))) ncclResult_t ncclSend(const void* b, size_t n, int t, int p, ncclComm_t c, void* s) { (void)b; (void)n; (void)t; (void)p; (void)c; (void)s; return 0; }
__attribute__((visibility("default"))) ncclResult_t ncclRecv(void* b, size_t n, int t, int p, ncclComm_t c, void* s) { (void)b; (void)n; (void)t; (void)p; (void)c; (void)s; return 0; }
__attribute__((visibility("default"))) ncclResult_t ncclAllGather(const void* a, void* b, size_t n, int t, ncclComm_t c, void* s) { (void)a; (void)b; (void)n; (void)t; (void)c; (void)s; return 0; }
__attribute__((visibility("default"))) const char* ncclGetErrorString(ncclResult_t r) { return r == 2 ? "unhandled system error (stand-in)" : r == 7 ? "in progress" : "stand-in error"; }
