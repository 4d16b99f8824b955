/*
 * decxb_gemm_f32_noalloc: the 3xTF32 GEMM for callers that must not allocate device memory.
 *
 * Who needs it: code that runs while another component owns the device allocator - a
 * framework whose caching pool has reserved the whole card (a cudaMalloc would fail or
 * evict), or a latency-critical loop in which cudaMalloc's implicit device-wide
 * synchronisation is not acceptable.  The regular entry point takes its hi/lo operand
 * scratch from the context's arena, which grows with cudaMalloc; this one keeps that scratch
 * in a fixed array that is part of the library image.
 *
 * The array below is part of this library's device code: every device whose CUDA context loads
 * the library's module holds its 64 MiB until the process exits, whether or not this entry is
 * ever called.  With the runtime's default lazy loading that is from the first use of anything in
 * this file on that device; with CUDA_MODULE_LOADING=EAGER it is from the first CUDA call of
 * any kind that the process makes on the device.
 *
 * Loading code also takes device memory, and it happens on first use: the first call on a device
 * loads this module, and the first problem that selects a tile shape not used before in the
 * process loads that kernel and sets its shared-memory attribute.  A caller that is about to
 * hand the whole card to another allocator should therefore make, beforehand, one call per
 * device with each problem shape it will use later (or one per tile shape: N <= 64-wide,
 * 128 x 128, 128 x 256 and 256 x 256 outputs select the four kernels).  After that warm-up a
 * call changes the device's free memory by nothing.
 */
#include "common.h"

#include <string.h>

#define DECXB_NOALLOC_SCRATCH_BYTES ((size_t)64 << 20)   /* 64 MiB per device */

/* hi/lo parts of A ([M][Kp]) followed by hi/lo parts of B transposed ([N][Kp]).  In host code
 * this name is only a handle for cudaGetSymbolAddress, never a pointer to pass to a kernel. */
static __device__ __align__(256) unsigned char g_noalloc_scratch[DECXB_NOALLOC_SCRATCH_BYTES];
/* where bounded device-side waits of the GEMM kernel report that they gave up */
static __device__ __align__(16) decxb_dev_status g_noalloc_status;

namespace {

struct DeviceSlot {
    bool ready = false;
    unsigned char* scratch = nullptr;     /* device address of g_noalloc_scratch on this device */
    decxb_dev_status host_status = {};
    decxb_ctx ctx;                        /* host-side bookkeeping only; owns no device memory */
};
DeviceSlot g_slots[16];
std::mutex g_slot_mtx[16];      /* one per device: calls on different devices do not wait for each other */

/* Puts the calling thread's current device back when the entry point returns. */
struct DeviceRestore {
    int prev = -1;
    DeviceRestore() { if (cudaGetDevice(&prev) != cudaSuccess) { cudaGetLastError(); prev = -1; } }
    ~DeviceRestore() { if (prev >= 0) cudaSetDevice(prev); }
};

void say(char* buf, size_t len, const char* msg)
{
    if (buf && len) { strncpy(buf, msg, len - 1); buf[len - 1] = 0; }
}

/* Once per device, with that device current: resolve the device addresses of the two symbols. */
int setup_device(int device, DeviceSlot** out, char* err, size_t err_len)
{
    DeviceSlot& s = g_slots[device];        /* the caller holds g_slot_mtx[device] */
    if (cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); say(err, err_len, "cudaSetDevice failed"); return DECXB_ERR_NO_DEVICE; }
    if (!s.ready) {
        int major = 0, sms = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
            cudaGetLastError(); say(err, err_len, "cannot query the device"); return DECXB_ERR_CUDA;
        }
        if (major != 10) { say(err, err_len, "device is not compute capability 10.x"); return DECXB_ERR_ARCH; }
        void *p_scratch = nullptr, *p_status = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p_scratch, g_noalloc_scratch);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&p_status, g_noalloc_status);
        if (e != cudaSuccess || !p_scratch || !p_status) {
            cudaGetLastError();
            say(err, err_len, "cudaGetSymbolAddress failed for the static scratch array");
            return DECXB_ERR_CUDA;
        }
        s.scratch = static_cast<unsigned char*>(p_scratch);
        s.ctx.device = device;
        s.ctx.sm_count = sms;
        s.ctx.d_status = static_cast<decxb_dev_status*>(p_status);
        s.ctx.h_status = &s.host_status;
        s.ready = true;
    }
    *out = &s;
    return DECXB_OK;
}

}  // namespace

extern "C" int decxb_gemm_f32_noalloc(int device, int64_t M, int64_t N, int64_t K,
                                      const float* A, int64_t lda, const float* B, int64_t ldb,
                                      const float* C, int64_t ldc, float* D, int64_t ldd,
                                      void* stream, char* err, size_t err_len)
{
    say(err, err_len, "");
    if (M <= 0 || N <= 0 || K <= 0) { say(err, err_len, "gemm dims must be positive"); return DECXB_ERR_BAD_PARAM; }
    if (!A || !B || !D) { say(err, err_len, "null operand"); return DECXB_ERR_BAD_PARAM; }
    if (lda < K || ldb < N || ldd < N || (C && ldc < N)) {
        say(err, err_len, "leading dimension smaller than the row length"); return DECXB_ERR_DIM_MISMATCH;
    }
    const int64_t Kp = decxb_ceil_to(K, 4);
    /* each part starts on a 256-byte boundary */
    const size_t a_part = (size_t)decxb_ceil_to(M * Kp * 4, 256), b_part = (size_t)decxb_ceil_to(N * Kp * 4, 256);
    const size_t need = 2 * a_part + 2 * b_part;
    if (M > (1 << 24) || N > (1 << 24) || K > (1 << 24) || need > DECXB_NOALLOC_SCRATCH_BYTES) {
        if (err && err_len)
            snprintf(err, err_len, "needs %zu bytes of operand scratch (2*(M+N)*ceil4(K)*4) but the static array holds %zu",
                     need, (size_t)DECXB_NOALLOC_SCRATCH_BYTES);
        return DECXB_ERR_TOO_LARGE;
    }
    if (device < 0 || device >= 16) { say(err, err_len, "device index out of range (0..15)"); return DECXB_ERR_BAD_PARAM; }
    DeviceRestore restore;
    /* one call at a time per device on the host side (the entry blocks until D is complete, so
     * calls through this lock never overlap on the GPU either) */
    std::lock_guard<std::mutex> lock(g_slot_mtx[device]);
    DeviceSlot* slot = nullptr;
    int rc = setup_device(device, &slot, err, err_len);
    if (rc) return rc;
    decxb_ctx* ctx = &slot->ctx;
    cudaStream_t s = (cudaStream_t)stream;
    if (s) {
        int sdev = -1;
        if (cudaStreamGetDevice(s, &sdev) != cudaSuccess) { cudaGetLastError(); say(err, err_len, "invalid stream"); return DECXB_ERR_BAD_PARAM; }
        if (sdev != device) { say(err, err_len, "the stream belongs to another device"); return DECXB_ERR_BAD_PARAM; }
    }

    float* a_hi = reinterpret_cast<float*>(slot->scratch);
    float* a_lo = reinterpret_cast<float*>(slot->scratch + a_part);
    float* b_hi = reinterpret_cast<float*>(slot->scratch + 2 * a_part);
    float* b_lo = reinterpret_cast<float*>(slot->scratch + 2 * a_part + b_part);

    /* The array keeps whatever the previous call left.  The operand parts are rewritten in
     * full (pad columns included) by the split kernels below; the status word is the one
     * thing that has to start at zero. */
    if (cudaMemsetAsync(ctx->d_status, 0, sizeof(decxb_dev_status), s) != cudaSuccess) {
        cudaGetLastError(); say(err, err_len, "cudaMemsetAsync failed"); return DECXB_ERR_CUDA;
    }
    if ((rc = decxb_launch_split_rows(ctx, A, M, K, lda, a_hi, a_lo, Kp, M, s)) ||
        (rc = decxb_launch_split_transpose(ctx, B, K, N, ldb, b_hi, b_lo, Kp, 0, s))) {
        say(err, err_len, ctx->last_error.c_str()); return rc;
    }
    decxb_gemm_args g = {};
    g.M = M; g.N = N; g.K = K;
    g.a_hi = a_hi; g.a_lo = a_lo; g.lda = Kp;
    g.b_hi = b_hi; g.b_lo = b_lo; g.ldb = Kp; g.b_rows = N;
    g.C = C; g.ldc = ldc; g.D = D; g.ldd = ldd; g.tile = DECXB_TILE_AUTO;
    if ((rc = decxb_launch_gemm_tn(ctx, g, s))) { say(err, err_len, ctx->last_error.c_str()); return rc; }
    if (cudaStreamSynchronize(s) != cudaSuccess) {
        say(err, err_len, cudaGetErrorString(cudaGetLastError())); return DECXB_ERR_CUDA;
    }
    if (cudaMemcpy(&slot->host_status, ctx->d_status, sizeof(decxb_dev_status), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError(); say(err, err_len, "cannot read the device status word"); return DECXB_ERR_CUDA;
    }
    if (slot->host_status.code != DECXB_DEVERR_NONE) {
        if (err && err_len)
            snprintf(err, err_len, "device wait gave up: code %d at role/barrier %d, block %d", slot->host_status.code,
                     slot->host_status.where, slot->host_status.block);
        return DECXB_ERR_TIMEOUT;
    }
    return DECXB_OK;
}
