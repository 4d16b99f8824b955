/* Context, error text, device arena, copies: the host-side runtime of the decxb library. */
#include "common.h"

#include <string.h>

static const char* kVersion = "decxb 0.1 (sm_100a)";

extern "C" const char* decxb_version(void) { return kVersion; }

extern "C" int decxb_bounds_build(void)
{
#ifdef DECXB_BOUNDS
    return 1;
#else
    return 0;
#endif
}

extern "C" const char* decxb_status_string(int status)
{
    switch (status) {
    case DECXB_OK: return "success";
    case DECXB_ERR_NOT_INIT: return "CUDA should be initialized first";
    case DECXB_ERR_DIM_MISMATCH: return "matrix dims don't match each other";
    case DECXB_ERR_BAD_KERNEL: return "convolution kernel is not supported";
    case DECXB_ERR_BAD_FLAG: return "invalid flag";
    case DECXB_ERR_BAD_PARAM: return "invalid parameter";
    case DECXB_ERR_ALLOC: return "fail to allocate memory on device";
    case DECXB_ERR_CUDA: return "CUDA call failed";
    case DECXB_ERR_NO_DEVICE: return "no CUDA device";
    case DECXB_ERR_ARCH: return "device is not compute capability 10.x (sm_100a code only)";
    case DECXB_ERR_TIMEOUT: return "a bounded device-side wait expired";
    case DECXB_ERR_TOO_LARGE: return "request exceeds a fixed limit";
    case DECXB_ERR_COMM: return "communication library failure";
    case DECXB_ERR_BOUNDS: return "debug bounds check caught an access outside its array";
    default: return "unknown status";
    }
}

void decxb_set_error(decxb_ctx* ctx, const std::string& msg)
{
    if (ctx) ctx->last_error = msg;
}

int decxb_fail(decxb_ctx* ctx, int status, const std::string& msg)
{
    decxb_set_error(ctx, std::string(decxb_status_string(status)) + ": " + msg);
    return status;
}

extern "C" const char* decxb_last_error(decxb_ctx* ctx)
{
    return ctx ? ctx->last_error.c_str() : "null context";
}

int decxb_bind(decxb_ctx* ctx)
{
    if (!ctx || ctx->device < 0) return DECXB_ERR_NOT_INIT;
    DECXB_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return DECXB_OK;
}

extern "C" int decxb_init(int device, decxb_ctx** out)
{
    if (!out) return DECXB_ERR_BAD_PARAM;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) { cudaGetLastError(); return DECXB_ERR_NO_DEVICE; }
    if (device < 0 || device >= n || device >= DECXB_MAX_DEVICES) return DECXB_ERR_BAD_PARAM;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return DECXB_ERR_CUDA;
    if (prop.major != 10) return DECXB_ERR_ARCH;
    decxb_ctx* ctx = new decxb_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    bool ok = cudaSetDevice(device) == cudaSuccess
           && cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) == cudaSuccess
           && cudaStreamCreateWithFlags(&ctx->copy_stream[0], cudaStreamNonBlocking) == cudaSuccess
           && cudaStreamCreateWithFlags(&ctx->copy_stream[1], cudaStreamNonBlocking) == cudaSuccess
           && cudaMalloc((void**)&ctx->d_status, sizeof(decxb_dev_status)) == cudaSuccess
           && cudaMemset(ctx->d_status, 0, sizeof(decxb_dev_status)) == cudaSuccess
           && cudaHostAlloc((void**)&ctx->h_status, sizeof(decxb_dev_status), cudaHostAllocDefault) == cudaSuccess
           && cudaMalloc((void**)&ctx->wave_counters, DECXB_WAVE_SLOTS * sizeof(unsigned long long)) == cudaSuccess
           && cudaMemset(ctx->wave_counters, 0, DECXB_WAVE_SLOTS * sizeof(unsigned long long)) == cudaSuccess;
    if (!ok) { cudaGetLastError(); delete ctx; return DECXB_ERR_CUDA; }
    memset(ctx->h_status, 0, sizeof(decxb_dev_status));
    *out = ctx;
    return DECXB_OK;
}

extern "C" int decxb_destroy(decxb_ctx* ctx)
{
    if (!ctx) return DECXB_OK;
    if (decxb_bind(ctx) == DECXB_OK) {
        cudaDeviceSynchronize();
        decxb_release_cached(ctx);
        for (auto& kv : ctx->arena.live) cudaFree(kv.first);
        for (cudaEvent_t e : ctx->arena.ev_pool) cudaEventDestroy(e);
        cudaFree(ctx->d_status);
        cudaFree(ctx->wave_counters);
        cudaFreeHost(ctx->h_status);
        cudaStreamDestroy(ctx->stream);
        cudaStreamDestroy(ctx->copy_stream[0]);
        cudaStreamDestroy(ctx->copy_stream[1]);
    }
    delete ctx;
    return DECXB_OK;
}

extern "C" int decxb_device(decxb_ctx* ctx) { return ctx ? ctx->device : -1; }
extern "C" void* decxb_stream(decxb_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
extern "C" uint64_t decxb_kernel_launch_count(decxb_ctx* ctx) { return ctx ? ctx->launches.load() : 0; }

extern "C" int decxb_set_wait_limit_ms(decxb_ctx* ctx, int ms)
{
    if (!ctx || ms <= 0) return DECXB_ERR_BAD_PARAM;
    ctx->wait_limit_ns = (long long)ms * 1000000LL;
    return DECXB_OK;
}

extern "C" int decxb_set_tile_group(decxb_ctx* ctx, int tile_rows)
{
    if (!ctx || tile_rows < 1 || tile_rows > 64) return DECXB_ERR_BAD_PARAM;
    ctx->tile_group = tile_rows;
    return DECXB_OK;
}

bool decxb_wave_slot(decxb_ctx* ctx, cudaStream_t s, unsigned long long arrivals, unsigned long long** counter, unsigned long long* base)
{
    std::lock_guard<std::mutex> lock(ctx->wave_mtx);
    int free_slot = -1;
    for (int i = 0; i < DECXB_WAVE_SLOTS; ++i) {
        auto& w = ctx->wave_slots[i];
        if (w.used && w.stream == s) { *counter = ctx->wave_counters + i; *base = w.base; w.base += arrivals; return true; }
        if (!w.used && free_slot < 0) free_slot = i;
    }
    if (free_slot < 0) return false;
    auto& w = ctx->wave_slots[free_slot];
    w.used = true; w.stream = s; w.base = arrivals;
    *counter = ctx->wave_counters + free_slot; *base = 0;
    return true;
}

void decxb_wave_unslot(decxb_ctx* ctx, cudaStream_t s, unsigned long long arrivals)
{
    std::lock_guard<std::mutex> lock(ctx->wave_mtx);
    for (auto& w : ctx->wave_slots) if (w.used && w.stream == s) { w.base -= arrivals; return; }
}

void decxb_wave_reset(decxb_ctx* ctx)
{
    std::lock_guard<std::mutex> lock(ctx->wave_mtx);
    cudaDeviceSynchronize();
    cudaMemset(ctx->wave_counters, 0, DECXB_WAVE_SLOTS * sizeof(unsigned long long));
    for (auto& w : ctx->wave_slots) w = {};
    cudaGetLastError();
}

extern "C" int decxb_set_wave_align(decxb_ctx* ctx, int on)
{
    if (!ctx) return DECXB_ERR_BAD_PARAM;
    ctx->wave_align = on == 2 ? 2 : on ? 1 : 0;
    return DECXB_OK;
}

extern "C" int decxb_set_tile_trace(decxb_ctx* ctx, unsigned long long* dbuf, int tiles_per_cluster)
{
    if (!ctx || tiles_per_cluster < 0) return DECXB_ERR_BAD_PARAM;
    ctx->trace = tiles_per_cluster > 0 ? dbuf : nullptr;
    ctx->trace_tiles = dbuf ? tiles_per_cluster : 0;
    return DECXB_OK;
}

extern "C" int decxb_set_pack_variant(decxb_ctx* ctx, int variant)
{
    if (!ctx || variant < 0 || variant > 2) return DECXB_ERR_BAD_PARAM;
    ctx->pack_variant = variant;
    return DECXB_OK;
}

int decxb_check_dev_status(decxb_ctx* ctx)
{
    DECXB_CUDA_TRY(ctx, cudaMemcpy(ctx->h_status, ctx->d_status, sizeof(decxb_dev_status), cudaMemcpyDeviceToHost));
    if (ctx->h_status->code != DECXB_DEVERR_NONE) {
        char buf[200];
        const bool bounds = ctx->h_status->code == DECXB_DEVERR_BOUNDS;
        if (bounds)
            snprintf(buf, sizeof buf, "bounds check: kernel %d, block %d touched element offset %d outside its array (access skipped)",
                     ctx->h_status->where, ctx->h_status->block, ctx->h_status->detail);
        else
            snprintf(buf, sizeof buf, "device wait gave up: code %d at role/barrier %d, block %d, detail %d",
                     ctx->h_status->code, ctx->h_status->where, ctx->h_status->block, ctx->h_status->detail);
        cudaMemset(ctx->d_status, 0, sizeof(decxb_dev_status));
        if (!bounds) decxb_wave_reset(ctx);       /* a launch that gave up left its wave counter short */
        return decxb_fail(ctx, bounds ? DECXB_ERR_BOUNDS : DECXB_ERR_TIMEOUT, buf);
    }
    return DECXB_OK;
}

extern "C" int decxb_synchronize(decxb_ctx* ctx)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    DECXB_CUDA_TRY(ctx, cudaDeviceSynchronize());
    return decxb_check_dev_status(ctx);
}

/* ---- arena ----------------------------------------------------------------------------
 * Blocks are rounded to 256 B (below 1 MiB) or 2 MiB (above) and cached on free.  A cached
 * block serves a request when it is large enough and not more than twice the request, so a
 * 4 GiB scratch block is never pinned under a 1 KiB request. */
static size_t arena_round(size_t bytes)
{
    if (bytes == 0) bytes = 1;
    const size_t g = bytes < (1u << 20) ? 256 : (size_t)2 << 20;
    return (bytes + g - 1) / g * g;
}

static const cudaStream_t kNoStream = (cudaStream_t)(intptr_t)-1;   /* block is idle: no wait needed */

static int arena_take(decxb_ctx* ctx, size_t bytes, void** dptr, cudaStream_t s, bool stream_ordered)
{
    if (!ctx || !dptr) return DECXB_ERR_BAD_PARAM;
    *dptr = nullptr;
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    const size_t need = arena_round(bytes);
    decxb_arena& a = ctx->arena;
    std::lock_guard<std::mutex> lock(a.mtx);
    /* prefer a block last used on the same stream, else any fitting block */
    auto pick = a.cached.end();
    for (auto it = a.cached.lower_bound(need); it != a.cached.end() && it->first <= need * 2; ++it) {
        if (pick == a.cached.end()) pick = it;
        if (it->second.stream == kNoStream || (stream_ordered && it->second.stream == s)) { pick = it; break; }
    }
    void* p = nullptr; size_t got = 0;
    if (pick != a.cached.end()) {
        decxb_cached_block blk = pick->second;
        got = pick->first;
        a.cached.erase(pick);
        if (blk.stream != kNoStream && !(stream_ordered && blk.stream == s)) {
            if (stream_ordered) cudaStreamWaitEvent(s, blk.ev, 0);
            else cudaEventSynchronize(blk.ev);
        }
        if (blk.ev) a.ev_pool.push_back(blk.ev);
        p = blk.ptr;
        a.bytes_cached -= got;
        a.n_reuses++;
    } else {
        cudaError_t e = cudaMalloc(&p, need);
        if (e != cudaSuccess) {
            /* give cached blocks back and retry once */
            cudaGetLastError();
            cudaDeviceSynchronize();
            for (auto& kv : a.cached) { cudaFree(kv.second.ptr); if (kv.second.ev) a.ev_pool.push_back(kv.second.ev); }
            a.cached.clear(); a.bytes_cached = 0;
            e = cudaMalloc(&p, need);
        }
        if (e != cudaSuccess) {
            cudaGetLastError();
            return decxb_fail(ctx, DECXB_ERR_ALLOC, std::to_string(need) + " bytes");
        }
        got = need;
        a.n_driver_allocs++;
    }
    a.live[p] = got;
    a.bytes_in_use += got;
    if (a.bytes_in_use > a.peak) a.peak = a.bytes_in_use;
    *dptr = p;
    return DECXB_OK;
}

static int arena_give(decxb_ctx* ctx, void* dptr, cudaStream_t s, bool stream_ordered)
{
    if (!ctx) return DECXB_ERR_BAD_PARAM;
    if (!dptr) return DECXB_OK;
    decxb_arena& a = ctx->arena;
    std::lock_guard<std::mutex> lock(a.mtx);
    auto it = a.live.find(dptr);
    if (it == a.live.end()) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "pointer not owned by this arena");
    const size_t sz = it->second;
    a.live.erase(it);
    a.bytes_in_use -= sz;
    decxb_cached_block blk = {dptr, kNoStream, nullptr};
    if (stream_ordered) {
        if (!a.ev_pool.empty()) { blk.ev = a.ev_pool.back(); a.ev_pool.pop_back(); }
        else if (cudaEventCreateWithFlags(&blk.ev, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); blk.ev = nullptr; }
        if (blk.ev && cudaEventRecord(blk.ev, s) == cudaSuccess) blk.stream = s;
        else { cudaGetLastError(); cudaStreamSynchronize(s); }
    }
    a.cached.emplace(sz, blk);
    a.bytes_cached += sz;
    return DECXB_OK;
}

extern "C" int decxb_malloc(decxb_ctx* ctx, size_t bytes, void** dptr) { return arena_take(ctx, bytes, dptr, nullptr, false); }
/* cudaFree would wait for the device; this free does not, so the block remembers an event on the
 * context's compute stream: whoever takes it next waits for the library's own asynchronous work
 * that may still use it.  Work the caller queued on a stream of its own is the caller's to
 * finish before the free. */
extern "C" int decxb_free(decxb_ctx* ctx, void* dptr)
{
    if (!ctx) return DECXB_ERR_BAD_PARAM;
    if (decxb_bind(ctx) != DECXB_OK) return arena_give(ctx, dptr, nullptr, false);
    return arena_give(ctx, dptr, ctx->stream, true);
}
int decxb_malloc_on_stream(decxb_ctx* ctx, size_t bytes, void** dptr, cudaStream_t s) { return arena_take(ctx, bytes, dptr, s, true); }
int decxb_free_on_stream(decxb_ctx* ctx, void* dptr, cudaStream_t s) { return arena_give(ctx, dptr, s, true); }

extern "C" int decxb_release_cached(decxb_ctx* ctx)
{
    if (!ctx) return DECXB_ERR_BAD_PARAM;
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    decxb_arena& a = ctx->arena;
    std::lock_guard<std::mutex> lock(a.mtx);
    cudaDeviceSynchronize();
    for (auto& kv : a.cached) { cudaFree(kv.second.ptr); if (kv.second.ev) a.ev_pool.push_back(kv.second.ev); }
    a.cached.clear();
    a.bytes_cached = 0;
    return DECXB_OK;
}

extern "C" int decxb_arena_get_stats(decxb_ctx* ctx, decxb_arena_stats* out)
{
    if (!ctx || !out) return DECXB_ERR_BAD_PARAM;
    decxb_arena& a = ctx->arena;
    std::lock_guard<std::mutex> lock(a.mtx);
    out->bytes_in_use = a.bytes_in_use; out->bytes_cached = a.bytes_cached; out->peak_bytes_in_use = a.peak;
    out->n_driver_allocs = a.n_driver_allocs; out->n_reuses = a.n_reuses;
    return DECXB_OK;
}

extern "C" int decxb_host_alloc(size_t bytes, void** hptr)
{
    if (!hptr) return DECXB_ERR_BAD_PARAM;
    if (cudaHostAlloc(hptr, bytes ? bytes : 1, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError(); *hptr = nullptr; return DECXB_ERR_ALLOC;
    }
    return DECXB_OK;
}

extern "C" int decxb_host_free(void* hptr)
{
    if (hptr && cudaFreeHost(hptr) != cudaSuccess) { cudaGetLastError(); return DECXB_ERR_CUDA; }
    return DECXB_OK;
}

extern "C" int decxb_memcpy2d(decxb_ctx* ctx, void* dst, size_t dpitch, const void* src, size_t spitch,
                              size_t width, size_t rows, int kind)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    cudaMemcpyKind k = kind == 1 ? cudaMemcpyHostToDevice : kind == 2 ? cudaMemcpyDeviceToHost
                     : kind == 3 ? cudaMemcpyDeviceToDevice : cudaMemcpyDefault;
    if (width == 0 || rows == 0) return DECXB_OK;
    DECXB_CUDA_TRY(ctx, cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, rows, k, ctx->stream));
    DECXB_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return DECXB_OK;
}

extern "C" int decxb_memset(decxb_ctx* ctx, void* dptr, int value, size_t bytes)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    DECXB_CUDA_TRY(ctx, cudaMemsetAsync(dptr, value, bytes, ctx->stream));
    DECXB_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return DECXB_OK;
}

/* ---- per-kernel event timing ------------------------------------------------------------- */
static cudaEvent_t prof_event(decxb_ctx* ctx)
{
    if (!ctx->prof_pool.empty()) { cudaEvent_t e = ctx->prof_pool.back(); ctx->prof_pool.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return e;
}

decxb_launch_scope::decxb_launch_scope(decxb_ctx* c, cudaStream_t st, int k) : ctx(c), s(st), cls(k)
{
    ctx->launches++;
    if (!ctx->profiling) return;
    std::lock_guard<std::mutex> lock(ctx->prof_mtx);
    cudaEvent_t a = prof_event(ctx);
    b = prof_event(ctx);
    if (!a || !b) { b = nullptr; return; }
    cudaEventRecord(a, s);
    ctx->prof_open.push_back({cls, a, b});
}

decxb_launch_scope::~decxb_launch_scope()
{
    if (b) cudaEventRecord(b, s);
}

extern "C" int decxb_profile_enable(decxb_ctx* ctx, int on)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    decxb_profile tmp;
    if ((rc = decxb_profile_read(ctx, &tmp))) return rc;     /* drains open spans */
    std::lock_guard<std::mutex> lock(ctx->prof_mtx);
    ctx->profiling = on != 0;
    if (on) ctx->prof_total = decxb_profile{};
    return DECXB_OK;
}

extern "C" int decxb_profile_read(decxb_ctx* ctx, decxb_profile* out)
{
    if (!out) return DECXB_ERR_BAD_PARAM;
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    DECXB_CUDA_TRY(ctx, cudaDeviceSynchronize());
    std::lock_guard<std::mutex> lock(ctx->prof_mtx);
    for (auto& sp : ctx->prof_open) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, sp.a, sp.b) == cudaSuccess) {
            ctx->prof_total.ms[sp.cls] += ms;
            ctx->prof_total.launches[sp.cls] += 1;
        } else cudaGetLastError();
        ctx->prof_pool.push_back(sp.a); ctx->prof_pool.push_back(sp.b);
    }
    ctx->prof_open.clear();
    *out = ctx->prof_total;
    return DECXB_OK;
}
