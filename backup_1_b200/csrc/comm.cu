/*
 * Gathering the result blocks of a sharded call over NCCL (one process or thread per GPU).
 *
 * The reference is single-GPU ("supports only single GPU", DECX_cpu/DECX_CPU.cpp:9) and hands
 * its result back whole (srcs/GEMM/CUDA/large_squares/GEMM.h:119-122); nothing here has a
 * counterpart there.  The path needs no exchange to compute: every rank multiplies its own rows
 * of A (or convolves its own images).  Only when the caller wants the whole result on every rank
 * do the blocks travel, and then the transfer is overlapped with the arithmetic: the rank's rows
 * are computed in a few row-panel groups, and while group g+1 is multiplied the finished rows of
 * group g are already on their way to the peers (NCCL send/receive on a side stream, into their
 * final place in the peers' result arrays, through a communicator limited to a few thread blocks so
 * that the GEMM beside it keeps its SMs).  Only the last, small group's transfer is exposed, and it
 * goes through a communicator with many thread blocks.
 *
 * NCCL is loaded at run time (dlopen of libnccl.so.2, or the file DECXB_NCCL_LIB names), so
 * the library has no link-time dependency on it and single-GPU users never load it.  The
 * communicator is created non-blocking: every NCCL call is followed by a poll of
 * ncclCommGetAsyncError under a host-side time limit, after which the communicator is aborted
 * and the entry returns DECXB_ERR_TIMEOUT (a rank that never arrives, a peer that died).  No
 * kernel of this library reads a peer's memory; NCCL moves the bytes into local HBM.
 */
#include "common.h"

#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <thread>

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommSplit)(ncclComm_t, int, int, ncclComm_t*, ncclConfig_t*) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    std::string error;
};

std::mutex g_api_mtx;
std::map<std::string, NcclApi*> g_apis;      /* one per library path, kept for the life of the process */

NcclApi* load_nccl(const char* path_or_null, std::string* err)
{
    const char* env = getenv("DECXB_NCCL_LIB");
    const std::string path = path_or_null && *path_or_null ? path_or_null : (env && *env ? env : "libnccl.so.2");
    std::lock_guard<std::mutex> lock(g_api_mtx);
    auto it = g_apis.find(path);
    if (it != g_apis.end()) return it->second;
    void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
    if (!h) { *err = std::string("cannot load ") + path + ": " + dlerror(); return nullptr; }
    NcclApi* a = new NcclApi();
    a->handle = h;
    bool ok = true;
    auto sym = [&](const char* name) { void* p = dlsym(h, name); if (!p) { ok = false; *err = std::string("missing symbol ") + name + " in " + path; } return p; };
    a->GetUniqueId = reinterpret_cast<decltype(a->GetUniqueId)>(sym("ncclGetUniqueId"));
    a->CommInitRankConfig = reinterpret_cast<decltype(a->CommInitRankConfig)>(sym("ncclCommInitRankConfig"));
    a->CommGetAsyncError = reinterpret_cast<decltype(a->CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    a->CommAbort = reinterpret_cast<decltype(a->CommAbort)>(sym("ncclCommAbort"));
    a->CommDestroy = reinterpret_cast<decltype(a->CommDestroy)>(sym("ncclCommDestroy"));
    a->CommSplit = reinterpret_cast<decltype(a->CommSplit)>(sym("ncclCommSplit"));
    a->GroupStart = reinterpret_cast<decltype(a->GroupStart)>(sym("ncclGroupStart"));
    a->GroupEnd = reinterpret_cast<decltype(a->GroupEnd)>(sym("ncclGroupEnd"));
    a->Send = reinterpret_cast<decltype(a->Send)>(sym("ncclSend"));
    a->Recv = reinterpret_cast<decltype(a->Recv)>(sym("ncclRecv"));
    a->AllGather = reinterpret_cast<decltype(a->AllGather)>(sym("ncclAllGather"));
    a->GetErrorString = reinterpret_cast<decltype(a->GetErrorString)>(sym("ncclGetErrorString"));
    if (!ok) { delete a; return nullptr; }
    g_apis[path] = a;
    return a;
}

}  // namespace

struct decxb_comm {
    NcclApi* api = nullptr;
    ncclComm_t comm = nullptr;          /* wide: many thread blocks per NCCL kernel, for transfers that run alone */
    ncclComm_t narrow = nullptr;        /* few thread blocks, for transfers that run beside a GEMM (split off `comm`) */
    int wide_ctas = 32;
    decxb_ctx* ctx = nullptr;           /* may be NULL in the host-side self-test */
    int world = 0, rank = 0;
    int timeout_ms = 30000;
    int reserve_sms = 8;                /* SMs left to NCCL's kernels while a transfer overlaps a GEMM = blocks of `narrow` */
    bool aborted = false;
    cudaStream_t stream = nullptr;      /* side stream the transfers run on */
    cudaEvent_t ev_ready = nullptr, ev_done = nullptr;
    std::mutex mtx;
    std::string last_error;
};

namespace {

int comm_fail(decxb_comm* c, int status, const std::string& msg)
{
    c->last_error = std::string(decxb_status_string(status)) + ": " + msg;
    if (c->ctx) decxb_set_error(c->ctx, c->last_error);
    return status;
}

/* Polls the communicator until the last NCCL call has left the "in progress" state; aborts the
 * communicator when the time limit passes or NCCL reports an asynchronous error. */
void comm_abort_all(decxb_comm* c)
{
    if (c->narrow) { c->api->CommAbort(c->narrow); c->narrow = nullptr; }
    if (c->comm) { c->api->CommAbort(c->comm); c->comm = nullptr; }
    c->aborted = true;
}

int comm_settle(decxb_comm* c, ncclResult_t call_rc, const char* what, ncclComm_t which = nullptr)
{
    if (call_rc != ncclSuccess && call_rc != ncclInProgress)
        return comm_fail(c, DECXB_ERR_COMM, std::string(what) + ": " + c->api->GetErrorString(call_rc));
    if (!which) which = c->comm;
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        ncclResult_t st = ncclSuccess;
        ncclResult_t q = c->api->CommGetAsyncError(which, &st);
        if (q != ncclSuccess) st = q;
        if (st == ncclSuccess) return DECXB_OK;
        const bool late = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() > c->timeout_ms;
        if (st != ncclInProgress || late) {
            comm_abort_all(c);
            if (st == ncclInProgress)
                return comm_fail(c, DECXB_ERR_TIMEOUT, std::string(what) + " did not complete within " + std::to_string(c->timeout_ms) +
                                                       " ms (a rank that never arrived?); communicator aborted");
            return comm_fail(c, DECXB_ERR_COMM, std::string(what) + ": " + c->api->GetErrorString(st) + "; communicator aborted");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(100));
    }
}

int comm_handshake(decxb_comm* c, const void* id128)
{
    ncclUniqueId id;
    static_assert(sizeof(id) == DECXB_COMM_ID_BYTES, "NCCL unique id size");
    memcpy(&id, id128, sizeof id);
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 0;
    /* Two communicators over the same ranks.  The wide one (DECXB_COMM_WIDE_CTAS thread blocks per NCCL kernel,
     * default 32) serves transfers that run alone.  The narrow one (DECXB_COMM_MAX_CTAS, default 2 per rank, 4 to 16) serves transfers
     * that run beside the persistent GEMM kernel, whose blocks fill whole SMs: every block NCCL takes is an SM the
     * GEMM does without, and a transfer hidden behind a row-panel group has time to spare. */
    const char* envw = getenv("DECXB_COMM_WIDE_CTAS");
    const char* envn = getenv("DECXB_COMM_MAX_CTAS");
    c->wide_ctas = envw && atoi(envw) > 0 && atoi(envw) <= 64 ? atoi(envw) : 32;
    /* measured on config 5: 4 blocks are too slow to hide a group's transfer at 4 ranks, 8 are best there, 16 cost the
     * GEMM more than they save; with twice the ranks a group's GEMM is half as long for about the same bytes */
    int narrow_default = 2 * c->world;
    if (narrow_default < 4) narrow_default = 4;
    if (narrow_default > 16) narrow_default = 16;
    c->reserve_sms = envn && atoi(envn) > 0 && atoi(envn) <= 64 ? atoi(envn) : narrow_default;
    cfg.maxCTAs = c->wide_ctas;
    ncclResult_t rc = c->api->CommInitRankConfig(&c->comm, c->world, id, c->rank, &cfg);
    if (!c->comm && rc != ncclSuccess && rc != ncclInProgress)
        return comm_fail(c, DECXB_ERR_COMM, std::string("ncclCommInitRankConfig: ") + c->api->GetErrorString(rc));
    int st = comm_settle(c, rc, "ncclCommInitRankConfig");
    if (st || c->world == 1) return st;
    ncclConfig_t cfgn = NCCL_CONFIG_INITIALIZER;
    cfgn.blocking = 0;
    cfgn.minCTAs = 1;
    cfgn.maxCTAs = c->reserve_sms;
    rc = c->api->CommSplit(c->comm, 0, c->rank, &c->narrow, &cfgn);
    if (rc != ncclSuccess && rc != ncclInProgress) {
        comm_abort_all(c);
        return comm_fail(c, DECXB_ERR_COMM, std::string("ncclCommSplit: ") + c->api->GetErrorString(rc));
    }
    if ((st = comm_settle(c, rc, "ncclCommSplit"))) return st;              /* the parent reports the split's progress */
    return c->narrow ? comm_settle(c, ncclSuccess, "ncclCommSplit (new communicator)", c->narrow) : DECXB_OK;
}

/* Bounded wait for everything queued on the side stream; aborts the communicator when the limit passes. */
int comm_drain(decxb_comm* c)
{
    if (!c->stream) return DECXB_OK;
    if (cudaEventRecord(c->ev_done, c->stream) != cudaSuccess) { cudaGetLastError(); return comm_fail(c, DECXB_ERR_CUDA, "cudaEventRecord"); }
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t e = cudaEventQuery(c->ev_done);
        if (e == cudaSuccess) return DECXB_OK;
        if (e != cudaErrorNotReady) { cudaGetLastError(); return comm_fail(c, DECXB_ERR_CUDA, std::string("transfer stream: ") + cudaGetErrorString(e)); }
        if (c->comm) {
            ncclResult_t st = ncclSuccess;
            c->api->CommGetAsyncError(c->comm, &st);
            if (st != ncclSuccess && st != ncclInProgress) {
                comm_abort_all(c);
                return comm_fail(c, DECXB_ERR_COMM, std::string("asynchronous NCCL error: ") + c->api->GetErrorString(st) + "; communicator aborted");
            }
        }
        if (std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() > c->timeout_ms) {
            if (c->comm) comm_abort_all(c);
            return comm_fail(c, DECXB_ERR_TIMEOUT, "transfers did not finish within " + std::to_string(c->timeout_ms) + " ms; communicator aborted");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

/* Rows [a, b) of the `rows`-row block of one rank that belong to panel group g of G.  The transfer of
 * the LAST group is the only one nothing overlaps, so the last group is small (a third of an even
 * share) and the others share the rest evenly; boundaries are multiples of 256 rows (whole tiles).
 * A pure function of its arguments, so sender and receivers agree on every panel without talking. */
void panel_range(int64_t rows, int g, int G, int64_t* a, int64_t* b)
{
    auto cut = [&](int k) -> int64_t {
        if (k <= 0) return 0;
        if (k >= G) return rows;
        const int64_t last = rows / (3 * (int64_t)G);
        int64_t c = (rows - last) * k / (G - 1) / 256 * 256;
        return c > rows ? rows : c;
    };
    *a = cut(g); *b = cut(g + 1);
}

/* One exchange: every rank sends units [ua_r, ub_r) of its own block to all peers and receives theirs
 * into place.  `base` is the whole array (same layout on every rank), unit_bytes the size of a unit. */
template <typename RangeFn>
int exchange(decxb_comm* c, ncclComm_t comm, char* base, size_t unit_bytes, int64_t total_units, RangeFn range, cudaStream_t s)
{
    NcclApi* n = c->api;
    int64_t my_f = 0, my_l = 0;
    decxb_shard_range(total_units, c->world, c->rank, &my_f, &my_l);
    int64_t ma = 0, mb = 0;
    range(my_l - my_f, &ma, &mb);
    ncclResult_t rc = n->GroupStart();
    if (rc != ncclSuccess && rc != ncclInProgress) return comm_fail(c, DECXB_ERR_COMM, std::string("ncclGroupStart: ") + n->GetErrorString(rc));
    for (int p = 0; p < c->world && (rc == ncclSuccess || rc == ncclInProgress); ++p) {
        if (p == c->rank) continue;
        int64_t f = 0, l = 0, a = 0, b = 0;
        decxb_shard_range(total_units, c->world, p, &f, &l);
        range(l - f, &a, &b);
        if (mb > ma) rc = n->Send(base + (size_t)(my_f + ma) * unit_bytes, (size_t)(mb - ma) * unit_bytes, ncclChar, p, comm, s);
        if (b > a && (rc == ncclSuccess || rc == ncclInProgress))
            rc = n->Recv(base + (size_t)(f + a) * unit_bytes, (size_t)(b - a) * unit_bytes, ncclChar, p, comm, s);
    }
    ncclResult_t rc2 = n->GroupEnd();
    if (rc != ncclSuccess && rc != ncclInProgress) return comm_settle(c, rc, "ncclSend/ncclRecv", comm);
    return comm_settle(c, rc2, "ncclGroupEnd", comm);
}

int comm_usable(decxb_comm* c)
{
    if (!c) return DECXB_ERR_BAD_PARAM;
    if (!c->comm || c->aborted) return comm_fail(c, DECXB_ERR_COMM, "the communicator was aborted; create a new one");
    if (!c->ctx) return comm_fail(c, DECXB_ERR_NOT_INIT, "communicator without a context");
    return DECXB_OK;
}

}  // namespace

extern "C" int decxb_comm_unique_id(void* id128)
{
    if (!id128) return DECXB_ERR_BAD_PARAM;
    std::string err;
    NcclApi* a = load_nccl(nullptr, &err);
    if (!a) return DECXB_ERR_COMM;
    ncclUniqueId id;
    if (a->GetUniqueId(&id) != ncclSuccess) return DECXB_ERR_COMM;
    memcpy(id128, &id, sizeof id);
    return DECXB_OK;
}

extern "C" int decxb_comm_init(decxb_ctx* ctx, int world, int rank, const void* id128, int timeout_ms, decxb_comm** out)
{
    if (!out) return DECXB_ERR_BAD_PARAM;
    *out = nullptr;
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (world < 1 || rank < 0 || rank >= world || !id128) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "bad world/rank/id");
    std::string err;
    NcclApi* api = load_nccl(nullptr, &err);
    if (!api) return decxb_fail(ctx, DECXB_ERR_COMM, err);
    decxb_comm* c = new decxb_comm();
    c->api = api; c->ctx = ctx; c->world = world; c->rank = rank;
    if (timeout_ms > 0) c->timeout_ms = timeout_ms;
    int lo = 0, hi = 0;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);
    bool ok = cudaStreamCreateWithPriority(&c->stream, cudaStreamNonBlocking, hi) == cudaSuccess
           && cudaEventCreateWithFlags(&c->ev_ready, cudaEventDisableTiming) == cudaSuccess
           && cudaEventCreateWithFlags(&c->ev_done, cudaEventDisableTiming) == cudaSuccess;
    if (!ok) { cudaGetLastError(); decxb_comm_destroy(c); return decxb_fail(ctx, DECXB_ERR_CUDA, "communicator stream/events"); }
    rc = comm_handshake(c, id128);
    if (rc) { decxb_comm_destroy(c); return rc; }
    *out = c;
    return DECXB_OK;
}

extern "C" int decxb_comm_destroy(decxb_comm* c)
{
    if (!c) return DECXB_OK;
    if (c->ctx) decxb_bind(c->ctx);
    if (c->stream) (void)comm_drain(c);
    if (c->narrow) { c->api->CommDestroy(c->narrow); c->narrow = nullptr; }
    if (c->comm) { c->api->CommDestroy(c->comm); c->comm = nullptr; }
    if (c->ev_ready) cudaEventDestroy(c->ev_ready);
    if (c->ev_done) cudaEventDestroy(c->ev_done);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
    return DECXB_OK;
}

extern "C" const char* decxb_comm_last_error(decxb_comm* c) { return c ? c->last_error.c_str() : "null communicator"; }

extern "C" int decxb_comm_set_reserved_sms(decxb_comm* c, int sms)
{
    if (!c || sms < 0 || sms > 64) return DECXB_ERR_BAD_PARAM;
    c->reserve_sms = sms;
    return DECXB_OK;
}

extern "C" int decxb_comm_synchronize(decxb_comm* c)
{
    int rc = comm_usable(c);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(c->mtx);
    if ((rc = decxb_bind(c->ctx))) return rc;
    return comm_drain(c);
}

/* Handshake against the NCCL-like library at `nccl_path` with no CUDA call at all: the host-side
 * half of decxb_comm_init (load, non-blocking init, bounded poll, abort on expiry). */
extern "C" int decxb_comm_selftest_handshake(const char* nccl_path, int world, int rank, const void* id128, int timeout_ms,
                                             char* err, size_t err_len)
{
    std::string msg;
    NcclApi* api = load_nccl(nccl_path, &msg);
    int rc = DECXB_ERR_COMM;
    if (api && id128 && world >= 1 && rank >= 0 && rank < world) {
        decxb_comm c;
        c.api = api; c.world = world; c.rank = rank;
        if (timeout_ms > 0) c.timeout_ms = timeout_ms;
        rc = comm_handshake(&c, id128);
        msg = c.last_error;
        if (c.comm) { api->CommDestroy(c.comm); c.comm = nullptr; }
    } else if (api) { rc = DECXB_ERR_BAD_PARAM; msg = "bad world/rank/id"; }
    if (err && err_len) { strncpy(err, msg.c_str(), err_len - 1); err[err_len - 1] = 0; }
    return rc;
}

namespace {
int allgather_blocks_locked(decxb_comm* c, void* base, size_t unit_bytes, int64_t total_units, cudaStream_t s);
}

extern "C" int decxb_comm_allgather_blocks(decxb_comm* c, void* base, size_t unit_bytes, int64_t total_units, void* stream)
{
    int rc = comm_usable(c);
    if (rc) return rc;
    if (!base || unit_bytes == 0 || total_units < 0) return comm_fail(c, DECXB_ERR_BAD_PARAM, "allgather arguments");
    std::lock_guard<std::mutex> lock(c->mtx);
    if ((rc = decxb_bind(c->ctx))) return rc;
    return allgather_blocks_locked(c, base, unit_bytes, total_units, stream ? (cudaStream_t)stream : c->ctx->stream);
}

namespace {
int allgather_blocks_locked(decxb_comm* c, void* base, size_t unit_bytes, int64_t total_units, cudaStream_t s)
{
    int rc = DECXB_OK;
    /* the transfers run on the side stream after everything queued on `s`, and `s` continues after them */
    if (cudaEventRecord(c->ev_ready, s) != cudaSuccess || cudaStreamWaitEvent(c->stream, c->ev_ready, 0) != cudaSuccess) {
        cudaGetLastError(); return comm_fail(c, DECXB_ERR_CUDA, "event on the compute stream");
    }
    int64_t f = 0, l = 0;
    decxb_shard_range(total_units, c->world, c->rank, &f, &l);
    if (total_units % c->world == 0 && c->world > 1) {
        /* equal blocks: NCCL's own all-gather, in place */
        const size_t count = (size_t)(l - f) * unit_bytes;
        ncclResult_t r = c->api->AllGather(static_cast<char*>(base) + (size_t)f * unit_bytes, base, count, ncclChar, c->comm, c->stream);
        rc = comm_settle(c, r, "ncclAllGather");
    } else if (c->world > 1) {
        rc = exchange(c, c->comm, static_cast<char*>(base), unit_bytes, total_units, [](int64_t n, int64_t* a, int64_t* b) { *a = 0; *b = n; }, c->stream);
    }
    if (rc) return rc;
    if (cudaEventRecord(c->ev_done, c->stream) != cudaSuccess || cudaStreamWaitEvent(s, c->ev_done, 0) != cudaSuccess) {
        cudaGetLastError(); return comm_fail(c, DECXB_ERR_CUDA, "event on the transfer stream");
    }
    return DECXB_OK;
}
}  // namespace

extern "C" int decxb_gemm_f32_rowshard_gather(decxb_ctx* ctx, decxb_comm* c, int mode, int tile, int64_t M, int64_t N, int64_t K,
                                              const float* A_rows, int64_t lda, const float* B, int64_t ldb,
                                              float* D_full, int groups, void* stream)
{
    int rc = comm_usable(c);
    if (rc) return rc;
    if (ctx != c->ctx) return comm_fail(c, DECXB_ERR_BAD_PARAM, "the communicator belongs to another context");
    if (groups < 1 || groups > 64) return comm_fail(c, DECXB_ERR_BAD_PARAM, "groups must be 1..64");
    if (M <= 0 || N <= 0 || K <= 0 || !A_rows || !B || !D_full) return comm_fail(c, DECXB_ERR_BAD_PARAM, "gemm arguments");
    std::lock_guard<std::mutex> lock(c->mtx);
    if ((rc = decxb_bind(ctx))) return rc;
    cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
    int64_t f = 0, l = 0;
    decxb_shard_range(M, c->world, c->rank, &f, &l);
    const int64_t rows = l - f;
    /* B is prepared (split, transposed) once for all groups */
    decxb_prepared_b* pb = nullptr;
    if (rows > 0 && (rc = decxb_gemm_prepare_b(ctx, mode, K, N, B, ldb, s, &pb))) return rc;
    const size_t row_bytes = (size_t)N * sizeof(float);
    cudaEvent_t ev = c->ev_ready;
    for (int g = 0; g < groups && rc == DECXB_OK; ++g) {
        int64_t a = 0, b = 0;
        panel_range(rows, g, groups, &a, &b);
        /* while transfers of earlier groups run, the GEMM leaves a few SMs to NCCL's kernels */
        ctx->reserved_sms = (g > 0 && c->world > 1) ? c->reserve_sms : 0;
        if (b > a)
            rc = decxb_gemm_rows_prepared_b(ctx, mode, tile, b - a, N, K, A_rows + a * lda, lda, pb, nullptr, 0,
                                            D_full + (f + a) * N, N, s);
        ctx->reserved_sms = 0;
        if (rc) break;
        if (c->world == 1) continue;
        if (cudaEventRecord(ev, s) != cudaSuccess || cudaStreamWaitEvent(c->stream, ev, 0) != cudaSuccess) {
            cudaGetLastError(); rc = comm_fail(c, DECXB_ERR_CUDA, "event on the compute stream"); break;
        }
        if (groups == 1 && M % c->world == 0) {
            /* one group of equal blocks: NCCL's own all-gather, in place */
            ncclResult_t r = c->api->AllGather(reinterpret_cast<char*>(D_full) + (size_t)f * row_bytes, D_full, (size_t)rows * row_bytes,
                                               ncclChar, c->comm, c->stream);
            rc = comm_settle(c, r, "ncclAllGather");
        } else {
            /* the last group's transfer runs alone: the wide communicator; the others run beside the next GEMM */
            rc = exchange(c, (g == groups - 1 || !c->narrow) ? c->comm : c->narrow, reinterpret_cast<char*>(D_full), row_bytes, M,
                          [&](int64_t n, int64_t* pa, int64_t* pbb) { panel_range(n, g, groups, pa, pbb); }, c->stream);
        }
    }
    if (pb) decxb_gemm_release_b(ctx, pb, s);
    if (rc) return rc;
    if (c->world > 1 && (cudaEventRecord(c->ev_done, c->stream) != cudaSuccess || cudaStreamWaitEvent(s, c->ev_done, 0) != cudaSuccess)) {
        cudaGetLastError(); return comm_fail(c, DECXB_ERR_CUDA, "event on the transfer stream");
    }
    return DECXB_OK;
}

/* Host-resident operands on several GPUs.  Every rank holds (or can read) the whole B in host memory, but the host's
 * copy bandwidth is shared by all ranks of the box (measured: 55 GB/s for one rank alone, 8 to 36 GB/s per rank when
 * eight copy at once), while NVLink is not: so a rank uploads only its own 1/world of the rows of each column block
 * of B and the ranks all-gather the block on the device; the rest is the single-GPU pipeline (a first row block of A
 * multiplied with the column blocks as they complete, then the other row blocks against the whole prepared B). */
extern "C" int decxb_gemm_f32_rowshard_host(decxb_ctx* ctx, decxb_comm* c, int mode, int tile, int64_t M, int64_t N, int64_t K,
                                            const float* hA_rows, int64_t lda, const float* hB, int64_t ldb,
                                            float* hD_rows, int64_t ldd)
{
    int rc = comm_usable(c);
    if (rc) return rc;
    if (ctx != c->ctx) return comm_fail(c, DECXB_ERR_BAD_PARAM, "the communicator belongs to another context");
    if (M <= 0 || N <= 0 || K <= 0 || !hA_rows || !hB || !hD_rows) return comm_fail(c, DECXB_ERR_BAD_PARAM, "gemm arguments");
    if (lda < K || ldb < N || ldd < N) return comm_fail(c, DECXB_ERR_DIM_MISMATCH, "leading dimension smaller than the row length");
    std::lock_guard<std::mutex> lock(c->mtx);
    if ((rc = decxb_bind(ctx))) return rc;
    int64_t f = 0, l = 0;
    decxb_shard_range(M, c->world, c->rank, &f, &l);
    decxb_b_share share = {};
    share.world = c->world;
    decxb_shard_range(K, c->world, c->rank, &share.k_first, &share.k_last);
    share.user = c;
    share.gather = [](void* user, float* base, size_t unit_bytes, int64_t units, cudaStream_t s) {
        return allgather_blocks_locked((decxb_comm*)user, base, unit_bytes, units, s);
    };
    rc = decxb_gemm_host_pipeline(ctx, mode, tile, l - f, N, K, hA_rows, lda, hB, ldb, nullptr, 0, hD_rows, ldd, &share);
    if (rc) {                                      /* the pipeline drained its own streams; the transfer stream is this layer's */
        cudaStreamSynchronize(c->stream);
        cudaGetLastError();
        c->last_error = decxb_last_error(ctx);
        return rc;
    }
    return comm_drain(c);
}
