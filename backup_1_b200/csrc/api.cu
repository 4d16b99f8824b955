/*
 * C-ABI entry points for GEMM and the im2col convolution: argument checks, scratch from the
 * arena, operand preparation, kernel launches, host staging.  See include/decxb.h.
 */
#include "common.h"

#include <stdlib.h>
#include <vector>

namespace {

/* Scratch blocks of one call, taken from the arena in stream order: a block released at the
 * end of a call can serve the next call on the same stream at once, and a call on another
 * stream waits for it on the device.  No host synchronisation, no allocation in steady state. */
struct Scratch {
    decxb_ctx* ctx;
    cudaStream_t s;
    std::vector<void*> ptrs;
    Scratch(decxb_ctx* c, cudaStream_t st) : ctx(c), s(st) {}
    int get(size_t bytes, void** p)
    {
        int rc = decxb_malloc_on_stream(ctx, bytes, p, s);
        if (rc == DECXB_OK) ptrs.push_back(*p);
        return rc;
    }
    void release()
    {
        for (void* q : ptrs) decxb_free_on_stream(ctx, q, s);
        ptrs.clear();
    }
    ~Scratch() { release(); }
};

bool tma_ok(const float* p, int64_t ld) { return ((uintptr_t)p % 16 == 0) && (ld % 4 == 0); }

/* B operand as the kernel wants it: K-contiguous hi (and lo) parts. */
struct PreparedB { const float* hi; const float* lo; int64_t ld; };

int prepare_b(decxb_ctx* ctx, Scratch& scratch, bool x3, int64_t N, int64_t K,
              const float* B, int64_t ldb, bool b_is_nt, cudaStream_t s, PreparedB* out)
{
    const int64_t Kp = decxb_split_pitch(K);
    int rc;
    if (b_is_nt && !x3 && tma_ok(B, ldb)) { out->hi = B; out->lo = nullptr; out->ld = ldb; return DECXB_OK; }
    float *hi = nullptr, *lo = nullptr;
    if ((rc = scratch.get((size_t)N * Kp * sizeof(float), (void**)&hi))) return rc;
    if (x3 && (rc = scratch.get((size_t)N * Kp * sizeof(float), (void**)&lo))) return rc;
    if (b_is_nt) {
        if (x3) { if ((rc = decxb_launch_split_rows(ctx, B, N, K, ldb, hi, lo, Kp, N, s))) return rc; }
        else    { DECXB_CUDA_TRY(ctx, cudaMemcpy2DAsync(hi, Kp * 4, B, ldb * 4, K * 4, N, cudaMemcpyDeviceToDevice, s)); }
    } else {
        if ((rc = decxb_launch_split_transpose(ctx, B, K, N, ldb, hi, lo, Kp, x3 ? 0 : 1, s))) return rc;
    }
    out->hi = hi; out->lo = lo; out->ld = Kp;
    return DECXB_OK;
}

/* D = A * B (+C) with B already prepared; A is split (3xTF32) or used in place. */
int gemm_prepared(decxb_ctx* ctx, Scratch& scratch, bool x3, int tile, int64_t M, int64_t N, int64_t K,
                  const float* A, int64_t lda, const PreparedB& pb,
                  const float* C, int64_t ldc, float* D, int64_t ldd, cudaStream_t s,
                  const float* bias = nullptr, int act = DECXB_ACT_NONE, bool chunked = false)
{
    const int64_t Kp = decxb_split_pitch(K);
    decxb_gemm_args g = {};
    g.chunked = chunked ? 1 : 0;
    g.M = M; g.N = N; g.K = K; g.C = C; g.ldc = ldc; g.D = D; g.ldd = ldd; g.tile = tile; g.b_rows = N;
    g.b_hi = pb.hi; g.b_lo = pb.lo; g.ldb = pb.ld;
    g.bias = bias; g.act = act;
    int rc;
    if (x3 || !tma_ok(A, lda)) {
        float *hi = nullptr, *lo = nullptr;
        if ((rc = scratch.get((size_t)M * Kp * sizeof(float), (void**)&hi))) return rc;
        if (x3 && (rc = scratch.get((size_t)M * Kp * sizeof(float), (void**)&lo))) return rc;
        if (x3) { if ((rc = decxb_launch_split_rows(ctx, A, M, K, lda, hi, lo, Kp, M, s))) return rc; }
        else    { DECXB_CUDA_TRY(ctx, cudaMemcpy2DAsync(hi, Kp * 4, A, lda * 4, K * 4, M, cudaMemcpyDeviceToDevice, s)); }
        g.a_hi = hi; g.a_lo = lo; g.lda = Kp;
    } else { g.a_hi = A; g.a_lo = nullptr; g.lda = lda; }
    return decxb_launch_gemm_tn(ctx, g, s);
}

/* D = A * op(B) (+C).  b_is_nt: B given as Bt[N][K]. */
int gemm_device(decxb_ctx* ctx, int mode, int tile, int64_t M, int64_t N, int64_t K,
                const float* A, int64_t lda, const float* B, int64_t ldb, bool b_is_nt,
                const float* C, int64_t ldc, float* D, int64_t ldd, cudaStream_t s,
                const float* bias = nullptr, int act = DECXB_ACT_NONE)
{
    if (mode != DECXB_GEMM_3XTF32 && mode != DECXB_GEMM_1XTF32 && mode != DECXB_GEMM_3XTF32_STRICT && mode != DECXB_GEMM_TF32_2XBF16)
        return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "gemm mode");
    if (act < DECXB_ACT_NONE || act > DECXB_ACT_TANH) return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "activation");
    if (M <= 0 || N <= 0 || K <= 0) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "gemm dims must be positive");
    if (!A || !B || !D) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "null operand");
    if (lda < K || ldb < (b_is_nt ? K : N) || ldd < N || (C && ldc < N))
        return decxb_fail(ctx, DECXB_ERR_DIM_MISMATCH, "leading dimension smaller than the row length");
    Scratch scratch(ctx, s);
    if (mode == DECXB_GEMM_TF32_2XBF16) {
        /* hi * hi in TF32, a_lo * b and a * b_lo in bf16: three arrays per operand, 8 bytes per element as in 3xTF32 */
        if (b_is_nt) return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "the TF32 + 2 x bf16 mode takes B as [K][N]");
        const int64_t Kp = decxb_split_pitch(K), K16 = decxb_ceil_to(K, 8);
        float *a_hi = nullptr, *b_hi = nullptr; void *a_lo16 = nullptr, *a_16 = nullptr, *b_lo16 = nullptr, *b_16 = nullptr;
        int rc2;
        if ((rc2 = scratch.get((size_t)M * Kp * 4, (void**)&a_hi)) || (rc2 = scratch.get((size_t)M * K16 * 2, &a_lo16)) ||
            (rc2 = scratch.get((size_t)M * K16 * 2, &a_16)) || (rc2 = scratch.get((size_t)N * Kp * 4, (void**)&b_hi)) ||
            (rc2 = scratch.get((size_t)N * K16 * 2, &b_lo16)) || (rc2 = scratch.get((size_t)N * K16 * 2, &b_16))) return rc2;
        if ((rc2 = decxb_launch_split_rows_bf16(ctx, A, M, K, lda, a_hi, a_lo16, a_16, Kp, K16, s))) return rc2;
        if ((rc2 = decxb_launch_split_transpose_bf16(ctx, B, K, N, ldb, b_hi, b_lo16, b_16, Kp, K16, s))) return rc2;
        decxb_gemm_args g = {};
        g.chunked = 1;
        g.M = M; g.N = N; g.K = K; g.C = C; g.ldc = ldc; g.D = D; g.ldd = ldd; g.tile = tile; g.b_rows = N;
        g.a_hi = a_hi; g.lda = Kp; g.b_hi = b_hi; g.ldb = Kp;
        g.a_16 = a_16; g.a_lo16 = a_lo16; g.b_16 = b_16; g.b_lo16 = b_lo16; g.ld16 = K16;
        g.bias = bias; g.act = act;
        rc2 = decxb_launch_gemm_tn(ctx, g, s);
        scratch.release();
        return rc2;
    }
    /* the strict mode is the 3xTF32 product with K accumulated in chunks (see gemm_tcgen05.cu) */
    const bool strict = mode == DECXB_GEMM_3XTF32_STRICT;
    const bool x3 = mode == DECXB_GEMM_3XTF32 || strict;
    int rc;
    if (x3 && !b_is_nt && (M + N) * K <= ((int64_t)1 << 25)) {
        /* small product: both operand splits in one launch */
        const int64_t Kp = decxb_split_pitch(K);
        float *a_hi = nullptr, *a_lo = nullptr, *b_hi = nullptr, *b_lo = nullptr;
        if ((rc = scratch.get((size_t)M * Kp * 4, (void**)&a_hi)) || (rc = scratch.get((size_t)M * Kp * 4, (void**)&a_lo)) ||
            (rc = scratch.get((size_t)N * Kp * 4, (void**)&b_hi)) || (rc = scratch.get((size_t)N * Kp * 4, (void**)&b_lo))) return rc;
        if (decxb_split_ab_possible(B, ldb, b_hi, b_lo)) {
            if ((rc = decxb_launch_split_ab(ctx, A, M, K, lda, a_hi, a_lo, B, N, ldb, b_hi, b_lo, Kp, s))) return rc;
        } else {
            if ((rc = decxb_launch_split_rows(ctx, A, M, K, lda, a_hi, a_lo, Kp, M, s))) return rc;
            if ((rc = decxb_launch_split_transpose(ctx, B, K, N, ldb, b_hi, b_lo, Kp, 0, s))) return rc;
        }
        decxb_gemm_args g = {};
        g.chunked = strict ? 1 : 0;
        g.M = M; g.N = N; g.K = K; g.C = C; g.ldc = ldc; g.D = D; g.ldd = ldd; g.tile = tile; g.b_rows = N;
        g.a_hi = a_hi; g.a_lo = a_lo; g.lda = Kp; g.b_hi = b_hi; g.b_lo = b_lo; g.ldb = Kp;
        g.bias = bias; g.act = act;
        rc = decxb_launch_gemm_tn(ctx, g, s);
        scratch.release();
        return rc;
    }
    PreparedB pb;
    rc = prepare_b(ctx, scratch, x3, N, K, B, ldb, b_is_nt, s, &pb);
    if (rc == DECXB_OK) rc = gemm_prepared(ctx, scratch, x3, tile, M, N, K, A, lda, pb, C, ldc, D, ldd, s, bias, act, strict);
    scratch.release();
    return rc;
}

/* Events of one host-resident call: upload of chunk i done / compute of chunk i done. */
struct ChunkEvents {
    std::vector<cudaEvent_t> ev;
    cudaEvent_t make()
    {
        cudaEvent_t e = nullptr;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        ev.push_back(e);
        return e;
    }
    ~ChunkEvents() { for (cudaEvent_t e : ev) cudaEventDestroy(e); }
};

/* Makes the two copy streams start after whatever is queued on the compute stream. */
int fence_copy_streams(decxb_ctx* ctx, ChunkEvents& evs)
{
    cudaEvent_t e = evs.make();
    if (!e) return decxb_fail(ctx, DECXB_ERR_CUDA, "cudaEventCreate");
    DECXB_CUDA_TRY(ctx, cudaEventRecord(e, ctx->stream));
    DECXB_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->copy_stream[0], e, 0));
    DECXB_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->copy_stream[1], e, 0));
    return DECXB_OK;
}

int sync_all_streams(decxb_ctx* ctx)
{
    DECXB_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->copy_stream[0]));
    DECXB_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    DECXB_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->copy_stream[1]));
    return DECXB_OK;
}

/* Waits for all three streams whatever each one reports (the error path of the pipelines). */
void drain_all_streams(decxb_ctx* ctx)
{
    cudaStreamSynchronize(ctx->copy_stream[0]);
    cudaStreamSynchronize(ctx->stream);
    cudaStreamSynchronize(ctx->copy_stream[1]);
    cudaGetLastError();
}

cudaStream_t pick_stream(decxb_ctx* ctx, void* stream) { return stream ? (cudaStream_t)stream : ctx->stream; }

/* Host-side fault injection for tests (decxb_inject_pipeline_error): true when the CUDA call
 * about to be made by a host-resident pipeline is the one chosen to fail. */
bool injected_failure(decxb_ctx* ctx)
{
    if (ctx->inject_countdown < 0) return false;
    if (ctx->inject_countdown-- > 0) return false;
    return true;
}

/* A CUDA call inside a host-resident pipeline.  When it fails, copies and kernels are already
 * queued on three streams and use the call's scratch blocks and the caller's host buffers:
 * `fail` (a local of the calling function) drains the streams before the function returns and
 * the scratch goes back to the arena. */
#define PIPE_TRY(expr)                                                                              \
    do {                                                                                           \
        cudaError_t _e = injected_failure(ctx) ? cudaErrorUnknown : (expr);                        \
        if (_e != cudaSuccess) {                                                                   \
            decxb_set_error(ctx, std::string(#expr) + ": " + cudaGetErrorString(_e));             \
            return fail(DECXB_ERR_CUDA);                                                           \
        }                                                                                          \
    } while (0)

}  // namespace

extern "C" int decxb_inject_pipeline_error(decxb_ctx* ctx, int nth_call)
{
    if (!ctx) return DECXB_ERR_BAD_PARAM;
    ctx->inject_countdown = nth_call;
    return DECXB_OK;
}

/* ---- B prepared once, used by many products ------------------------------------------------------
 * Weights are constant across calls in the use this path is for; the hi/lo split and the transposition
 * of B cost a tenth of a large product and a third of a small one.  A handle keeps the prepared
 * (K-contiguous, split) operand in arena memory until it is released. */
struct decxb_prepared_b {
    decxb_ctx* ctx;
    int mode;
    int64_t K, N, ld;
    float *hi, *lo;
};

extern "C" int decxb_gemm_prepare_b(decxb_ctx* ctx, int mode, int64_t K, int64_t N, const float* B, int64_t ldb,
                                    void* stream, decxb_prepared_b** out)
{
    if (!out) return DECXB_ERR_BAD_PARAM;
    *out = nullptr;
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (mode != DECXB_GEMM_3XTF32 && mode != DECXB_GEMM_1XTF32 && mode != DECXB_GEMM_3XTF32_STRICT)
        return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "gemm mode");
    if (K <= 0 || N <= 0 || !B) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "prepare_b arguments");
    if (ldb < N) return decxb_fail(ctx, DECXB_ERR_DIM_MISMATCH, "leading dimension smaller than the row length");
    cudaStream_t s = pick_stream(ctx, stream);
    const bool x3 = mode != DECXB_GEMM_1XTF32;
    const int64_t Kp = decxb_split_pitch(K);
    float *hi = nullptr, *lo = nullptr;
    if ((rc = decxb_malloc_on_stream(ctx, (size_t)N * Kp * sizeof(float), (void**)&hi, s))) return rc;
    if (x3 && (rc = decxb_malloc_on_stream(ctx, (size_t)N * Kp * sizeof(float), (void**)&lo, s))) { decxb_free_on_stream(ctx, hi, s); return rc; }
    if ((rc = decxb_launch_split_transpose(ctx, B, K, N, ldb, hi, lo, Kp, x3 ? 0 : 1, s))) {
        decxb_free_on_stream(ctx, hi, s); if (lo) decxb_free_on_stream(ctx, lo, s);
        return rc;
    }
    *out = new decxb_prepared_b{ctx, mode, K, N, Kp, hi, lo};
    return DECXB_OK;
}

extern "C" int decxb_gemm_release_b(decxb_ctx* ctx, decxb_prepared_b* pb, void* stream)
{
    if (!pb) return DECXB_OK;
    if (!ctx || pb->ctx != ctx) return DECXB_ERR_BAD_PARAM;
    cudaStream_t s = pick_stream(ctx, stream);
    decxb_free_on_stream(ctx, pb->hi, s);
    if (pb->lo) decxb_free_on_stream(ctx, pb->lo, s);
    delete pb;
    return DECXB_OK;
}

/* Rows of D = A * B (+C) with B prepared (internal form shared with the gathering entry). */
int decxb_gemm_rows_prepared_b(decxb_ctx* ctx, int mode, int tile, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                               const decxb_prepared_b* pb, const float* C, int64_t ldc, float* D, int64_t ldd, cudaStream_t s,
                               const float* bias, int act)
{
    if (!pb || pb->ctx != ctx) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "prepared operand of another context");
    if (pb->mode != mode || pb->K != K || pb->N != N) return decxb_fail(ctx, DECXB_ERR_DIM_MISMATCH, "prepared operand does not match the call");
    if (act < DECXB_ACT_NONE || act > DECXB_ACT_TANH) return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "activation");
    if (M <= 0) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "gemm dims must be positive");
    if (!A || !D) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "null operand");
    if (lda < K || ldd < N || (C && ldc < N)) return decxb_fail(ctx, DECXB_ERR_DIM_MISMATCH, "leading dimension smaller than the row length");
    Scratch scratch(ctx, s);
    const bool strict = mode == DECXB_GEMM_3XTF32_STRICT;
    PreparedB p = {pb->hi, pb->lo, pb->ld};
    int rc = gemm_prepared(ctx, scratch, mode != DECXB_GEMM_1XTF32, tile, M, N, K, A, lda, p, C, ldc, D, ldd, s, bias, act, strict);
    scratch.release();
    return rc;
}

extern "C" int decxb_gemm_f32_prepared(decxb_ctx* ctx, int tile, int64_t M, const float* A, int64_t lda,
                                       const decxb_prepared_b* pb, const float* C, int64_t ldc,
                                       const float* bias, int activation, float* D, int64_t ldd, void* stream)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (!pb) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "null prepared operand");
    return decxb_gemm_rows_prepared_b(ctx, pb->mode, tile, M, pb->N, pb->K, A, lda, pb, C, ldc, D, ldd, pick_stream(ctx, stream),
                                      bias, activation);
}

extern "C" int decxb_gemm_f32(decxb_ctx* ctx, int mode, int tile, int64_t M, int64_t N, int64_t K,
                              const float* A, int64_t lda, const float* B, int64_t ldb,
                              const float* C, int64_t ldc, float* D, int64_t ldd, void* stream)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    return gemm_device(ctx, mode, tile, M, N, K, A, lda, B, ldb, false, C, ldc, D, ldd, pick_stream(ctx, stream));
}

extern "C" int decxb_gemm_f32_act(decxb_ctx* ctx, int mode, int tile, int64_t M, int64_t N, int64_t K,
                                  const float* A, int64_t lda, const float* B, int64_t ldb,
                                  const float* C, int64_t ldc, const float* bias, int activation,
                                  float* D, int64_t ldd, void* stream)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    return gemm_device(ctx, mode, tile, M, N, K, A, lda, B, ldb, false, C, ldc, D, ldd, pick_stream(ctx, stream), bias, activation);
}

extern "C" int decxb_gemm_f32_nt(decxb_ctx* ctx, int mode, int tile, int64_t M, int64_t N, int64_t K,
                                 const float* A, int64_t lda, const float* Bt, int64_t ldbt,
                                 const float* C, int64_t ldc, float* D, int64_t ldd, void* stream)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    return gemm_device(ctx, mode, tile, M, N, K, A, lda, Bt, ldbt, true, C, ldc, D, ldd, pick_stream(ctx, stream));
}

extern "C" int decxb_gemm_f32_host(decxb_ctx* ctx, int mode, int tile, int64_t M, int64_t N, int64_t K,
                                   const float* hA, int64_t lda, const float* hB, int64_t ldb,
                                   const float* hC, int64_t ldc, float* hD, int64_t ldd)
{
    return decxb_gemm_host_pipeline(ctx, mode, tile, M, N, K, hA, lda, hB, ldb, hC, ldc, hD, ldd, nullptr);
}

/* How the host-resident product is cut (pure host arithmetic, no CUDA call): column blocks of B in upload order, the
 * pieces of the first row-block of A, the later row-blocks. */
struct HostPlan {
    int64_t rows0 = 0;                                         /* rows of the first row-block */
    std::vector<std::pair<int64_t, int64_t>> col_blocks, pieces, row_blocks;   /* (first, count) */
};

static HostPlan host_plan(int64_t M, int64_t N, int64_t K, int world)
{
    HostPlan pl;
    /* later row-blocks: about 1/8 of M, multiples of 256 rows, at least 512 */
    int64_t rows = decxb_ceil_to(decxb_ceil_div(M, 8), 256);
    if (rows < 512) rows = 512;
    if (rows > M) rows = M;
    /* first row-block: about K rows; column blocks of B: about 1/8 of N, at least 1024 columns */
    int64_t rows0 = decxb_ceil_to(K, 256);
    /* ... but no more rows than the GPU needs to stay busy while B comes up: multiplying rows0 rows with a column
     * block takes 2 rows0 ncol K / F, uploading the block 4 K ncol / BW, equal at rows0 = 2 F / BW, about 10 000 rows
     * at 250 TFLOP/s and 50 GB/s, whatever the sizes.  (With K = 32768 the first block was the whole of A: 80 ms of
     * upload with the GPU idle.) */
    int64_t cap0 = 10240;
    /* shares of B arrive `world` times as fast, over a host link that the ranks of the box share (measured per rank:
     * about 0.9 of the rate of a rank alone at 2 ranks, 0.5 at 4 and 8) */
    if (world > 1) {
        double slow = 0.6 + 0.25 * world;
        if (slow > 2.0) slow = 2.0;
        cap0 = decxb_ceil_to((int64_t)(10240.0 * slow / world), 256);
    }
    if (cap0 < 1024) cap0 = 1024;
    if (rows0 > cap0) rows0 = cap0;
    if (rows0 < rows) rows0 = rows;
    if (rows0 > M) rows0 = M;
    int64_t ncol = decxb_ceil_to(decxb_ceil_div(N, 8), 256);
    if (ncol < 1024) ncol = 1024;
    if (N < 2048 || ncol > N) ncol = N;
    pl.rows0 = rows0;
    /* the first column blocks are narrower (a quarter, then half of the regular width): less to wait for before the
     * first product; likewise the last row blocks of the second phase, whose results nothing hides on their way home */
    int64_t w = ncol / 4 >= 1024 && ncol % 4 == 0 ? ncol / 4 : ncol;
    for (int64_t c0 = 0; c0 < N;) {
        const int64_t nc = N - c0 < w ? N - c0 : w;
        pl.col_blocks.push_back({c0, nc});
        c0 += nc;
        if (w < ncol) w *= 2;
    }
    /* the first row-block goes up in up to four pieces, each multiplied with the first column block as it lands */
    int64_t piece = decxb_ceil_to(decxb_ceil_div(rows0 > 0 ? rows0 : 1, 4), 256);
    if (piece < 512) piece = 512;
    for (int64_t r0 = 0; r0 < rows0; r0 += piece) pl.pieces.push_back({r0, rows0 - r0 < piece ? rows0 - r0 : piece});
    int64_t r0 = rows0;
    while (r0 < M) {
        int64_t nr = M - r0;
        if (nr > rows) nr = rows;                                    /* regular blocks ... */
        else if (nr >= 2048 && nr % 512 == 0) nr /= 2;               /* ... then halves of what is left, down to 1024 rows */
        pl.row_blocks.push_back({r0, nr});
        r0 += nr;
    }
    return pl;
}

extern "C" int decxb_gemm_host_plan(int64_t M, int64_t N, int64_t K, int world, int64_t* kind_first_count, int capacity)
{
    if (M < 0 || N <= 0 || K <= 0 || world < 1 || capacity < 0 || (capacity > 0 && !kind_first_count)) return -1;
    const HostPlan pl = host_plan(M, N, K, world);
    int n = 0;
    auto put = [&](int64_t kind, const std::pair<int64_t, int64_t>& b) {
        if (n < capacity) { kind_first_count[3 * n] = kind; kind_first_count[3 * n + 1] = b.first; kind_first_count[3 * n + 2] = b.second; }
        ++n;
    };
    for (const auto& b : pl.col_blocks) put(0, b);
    for (const auto& b : pl.pieces) put(1, b);
    for (const auto& b : pl.row_blocks) put(2, b);
    return n;
}

/* The host-resident product.  With `share` (several ranks, every one of which can read the whole B in host memory)
 * a column block of B is kept contiguous on the device, this rank uploads only rows [k_first, k_last) of it and
 * share->gather completes it from the peers; M may then be 0 (a rank without rows still contributes its rows of B). */
int decxb_gemm_host_pipeline(decxb_ctx* ctx, int mode, int tile, int64_t M, int64_t N, int64_t K,
                             const float* hA, int64_t lda, const float* hB, int64_t ldb,
                             const float* hC, int64_t ldc, float* hD, int64_t ldd, const decxb_b_share* share)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (M < 0 || (M == 0 && !share) || N <= 0 || K <= 0) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "gemm dims must be positive");
    if (!hA || !hB || !hD) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "null operand");
    if (lda < K || ldb < N || ldd < N || (hC && ldc < N))
        return decxb_fail(ctx, DECXB_ERR_DIM_MISMATCH, "leading dimension smaller than the row length");
    if (mode != DECXB_GEMM_3XTF32 && mode != DECXB_GEMM_1XTF32 && mode != DECXB_GEMM_3XTF32_STRICT)
        return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "gemm mode");
    /* Three streams: uploads, compute, downloads.  (The reference does the three phases one
     * after the other on one stream, GEMM.h:106-123.)
     * Phase 1: a first, narrow column block of B goes up, then the first row-block of A in
     * pieces, each multiplied with that column block as it lands, then the rest of B in column
     * blocks; every column block is prepared and multiplied with the row-block as soon as it
     * has landed, and its piece of the result starts its way back while the next column block
     * is still in flight.
     * Phase 2: the remaining row-blocks of A (and C) go up, each multiplied with the whole
     * prepared B as it lands while the previous result block downloads. */
    cudaStream_t s = ctx->stream, up = ctx->copy_stream[0], down = ctx->copy_stream[1];
    Scratch scratch(ctx, s);
    ChunkEvents evs;
    const bool strict = mode == DECXB_GEMM_3XTF32_STRICT;
    const bool x3 = mode == DECXB_GEMM_3XTF32 || strict;
    const int64_t Kp = decxb_split_pitch(K), Np = decxb_ceil_to(N, 4);
    float *dA, *dB, *dC = nullptr, *dD, *b_hi = nullptr, *b_lo = nullptr;
    const int64_t Ma = M > 0 ? M : 1;
    if ((rc = scratch.get((size_t)Ma * Kp * 4, (void**)&dA))) return rc;
    if ((rc = scratch.get((size_t)K * Np * 4, (void**)&dB))) return rc;
    if ((rc = scratch.get((size_t)Ma * Np * 4, (void**)&dD))) return rc;
    if (hC && (rc = scratch.get((size_t)Ma * Np * 4, (void**)&dC))) return rc;
    if ((rc = scratch.get((size_t)N * Kp * 4, (void**)&b_hi))) return rc;
    if (x3 && (rc = scratch.get((size_t)N * Kp * 4, (void**)&b_lo))) return rc;
    if ((rc = fence_copy_streams(ctx, evs))) return rc;
    const HostPlan plan = host_plan(M, N, K, share ? share->world : 1);
    const int64_t rows0 = plan.rows0;
    const auto& col_blocks = plan.col_blocks;
    const auto& row_blocks = plan.row_blocks;

    auto fail = [&](int code) { drain_all_streams(ctx); return code; };
    float *a0_hi = dA, *a0_lo = nullptr;
    if (x3 && rows0 > 0 &&
        ((rc = scratch.get((size_t)rows0 * Kp * 4, (void**)&a0_hi)) || (rc = scratch.get((size_t)rows0 * Kp * 4, (void**)&a0_lo)))) return rc;
    /* a column block of B: up (whole, or this rank's rows of it, completed by the peers), split and transposed */
    auto stage_b_block = [&](int64_t c0, int64_t nc) -> int {
        cudaEvent_t e_up = evs.make();
        if (!e_up) return fail(decxb_fail(ctx, DECXB_ERR_CUDA, "cudaEventCreate"));
        /* whole B: the column block in place in the K x Np array; shares: the block on its own, K rows of nc floats,
         * so that the rows the peers send are contiguous */
        float* blk = share ? dB + K * c0 : dB + c0;
        const int64_t blk_ld = share ? decxb_ceil_to(nc, 4) : Np;
        if (!share) PIPE_TRY(cudaMemcpy2DAsync(blk, blk_ld * 4, hB + c0, ldb * 4, nc * 4, K, cudaMemcpyHostToDevice, up));
        else if (share->k_last > share->k_first)
            PIPE_TRY(cudaMemcpy2DAsync(blk + share->k_first * blk_ld, blk_ld * 4, hB + share->k_first * ldb + c0, ldb * 4, nc * 4,
                                       share->k_last - share->k_first, cudaMemcpyHostToDevice, up));
        PIPE_TRY(cudaEventRecord(e_up, up));
        PIPE_TRY(cudaStreamWaitEvent(s, e_up, 0));
        int r = DECXB_OK;
        if (share && (r = share->gather(share->user, blk, (size_t)blk_ld * 4, K, s))) return fail(r);
        if (M == 0) return DECXB_OK;
        /* columns c0.. of B are rows c0.. of the prepared (K-contiguous) operand */
        if ((r = decxb_launch_split_transpose(ctx, blk, K, nc, blk_ld, b_hi + c0 * Kp, x3 ? b_lo + c0 * Kp : nullptr, Kp,
                                              x3 ? 0 : 1, s))) return fail(r);
        return DECXB_OK;
    };
    /* rows [r0, r0 + nr) of the first row block times a column block, and that piece of the result on its way home */
    auto first_block_product = [&](int64_t r0, int64_t nr, int64_t c0, int64_t nc) -> int {
        cudaEvent_t e_done = evs.make();
        if (!e_done) return fail(decxb_fail(ctx, DECXB_ERR_CUDA, "cudaEventCreate"));
        decxb_gemm_args g = {};
        g.M = nr; g.N = nc; g.K = K;
        g.a_hi = a0_hi + r0 * Kp; g.a_lo = x3 ? a0_lo + r0 * Kp : nullptr; g.lda = Kp;
        g.b_hi = b_hi + c0 * Kp; g.b_lo = x3 ? b_lo + c0 * Kp : nullptr; g.ldb = Kp; g.b_rows = nc;
        g.C = dC ? dC + r0 * Np + c0 : nullptr; g.ldc = Np; g.D = dD + r0 * Np + c0; g.ldd = Np;
        g.tile = tile; g.chunked = strict ? 1 : 0;
        int r = decxb_launch_gemm_tn(ctx, g, s);
        if (r) return fail(r);
        PIPE_TRY(cudaEventRecord(e_done, s));
        PIPE_TRY(cudaStreamWaitEvent(down, e_done, 0));
        PIPE_TRY(cudaMemcpy2DAsync(hD + r0 * ldd + c0, ldd * 4, dD + r0 * Np + c0, Np * 4, nc * 4, nr, cudaMemcpyDeviceToHost, down));
        return DECXB_OK;
    };
    /* The first column block of B goes up first, then the first row block of A in up to four pieces: each piece is
     * split and multiplied with that column block as it lands, so the arithmetic starts a quarter of the way into
     * the row block's upload instead of at its end. */
    const int64_t nc0 = col_blocks[0].second;
    if ((rc = stage_b_block(0, nc0))) return rc;
    for (const auto& pc : plan.pieces) {
        const int64_t r0 = pc.first, nr = pc.second;
        cudaEvent_t e_up = evs.make();
        if (!e_up) return fail(decxb_fail(ctx, DECXB_ERR_CUDA, "cudaEventCreate"));
        PIPE_TRY(cudaMemcpy2DAsync(dA + r0 * Kp, Kp * 4, hA + r0 * lda, lda * 4, K * 4, nr, cudaMemcpyHostToDevice, up));
        if (hC) PIPE_TRY(cudaMemcpy2DAsync(dC + r0 * Np, Np * 4, hC + r0 * ldc, ldc * 4, N * 4, nr, cudaMemcpyHostToDevice, up));
        PIPE_TRY(cudaEventRecord(e_up, up));
        PIPE_TRY(cudaStreamWaitEvent(s, e_up, 0));
        if (x3 && (rc = decxb_launch_split_rows(ctx, dA + r0 * Kp, nr, K, Kp, a0_hi + r0 * Kp, a0_lo + r0 * Kp, Kp, nr, s))) return fail(rc);
        if ((rc = first_block_product(r0, nr, 0, nc0))) return rc;
    }
    for (size_t bi = 1; bi < col_blocks.size(); ++bi) {
        const int64_t c0 = col_blocks[bi].first, nc = col_blocks[bi].second;
        if ((rc = stage_b_block(c0, nc))) return rc;
        if (rows0 > 0 && (rc = first_block_product(0, rows0, c0, nc))) return rc;
    }
    PreparedB pb = {b_hi, b_lo, Kp};
    for (const auto& rbk : row_blocks) {
        const int64_t r0 = rbk.first, nr = rbk.second;
        cudaEvent_t e_up = evs.make(), e_done = evs.make();
        if (!e_up || !e_done) return fail(decxb_fail(ctx, DECXB_ERR_CUDA, "cudaEventCreate"));
        PIPE_TRY(cudaMemcpy2DAsync(dA + r0 * Kp, Kp * 4, hA + r0 * lda, lda * 4, K * 4, nr, cudaMemcpyHostToDevice, up));
        if (hC) PIPE_TRY(cudaMemcpy2DAsync(dC + r0 * Np, Np * 4, hC + r0 * ldc, ldc * 4, N * 4, nr, cudaMemcpyHostToDevice, up));
        PIPE_TRY(cudaEventRecord(e_up, up));
        PIPE_TRY(cudaStreamWaitEvent(s, e_up, 0));
        rc = gemm_prepared(ctx, scratch, x3, tile, nr, N, K, dA + r0 * Kp, Kp, pb, dC ? dC + r0 * Np : nullptr, Np,
                           dD + r0 * Np, Np, s, nullptr, DECXB_ACT_NONE, strict);
        if (rc) return fail(rc);
        PIPE_TRY(cudaEventRecord(e_done, s));
        PIPE_TRY(cudaStreamWaitEvent(down, e_done, 0));
        PIPE_TRY(cudaMemcpy2DAsync(hD + r0 * ldd, ldd * 4, dD + r0 * Np, Np * 4, N * 4, nr, cudaMemcpyDeviceToHost, down));
    }
    if ((rc = sync_all_streams(ctx))) return rc;
    scratch.release();
    return decxb_check_dev_status(ctx);
}

/* ---- fp16 GEMM ------------------------------------------------------------------------------- */
namespace {
int gemm_f16_device(decxb_ctx* ctx, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda, const void* B, int64_t ldb,
                    const void* C, int64_t ldc, void* D, int64_t ldd, cudaStream_t s)
{
    if (M <= 0 || N <= 0 || K <= 0) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "gemm dims must be positive");
    if (!A || !B || !D) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "null operand");
    if (lda < K || ldb < N || ldd < N || (C && ldc < N))
        return decxb_fail(ctx, DECXB_ERR_DIM_MISMATCH, "leading dimension smaller than the row length");
    Scratch scratch(ctx, s);
    const int64_t Kp = decxb_ceil_to(K, 8);
    decxb_gemm_f16_args g = {};
    g.M = M; g.N = N; g.K = K; g.C = C; g.ldc = ldc; g.D = D; g.ldd = ldd; g.act = DECXB_ACT_NONE;
    int rc;
    void* bt = nullptr;
    if ((rc = scratch.get((size_t)N * Kp * 2, &bt))) return rc;
    if ((rc = decxb_launch_transpose_f16(ctx, B, K, N, ldb, bt, Kp, s))) return rc;
    g.Bt = bt; g.ldbt = Kp;
    if (((uintptr_t)A % 16) || (lda % 8)) {            /* TMA cannot address it: repack with a pitch of ceil8(K) */
        void* a2 = nullptr;
        if ((rc = scratch.get((size_t)M * Kp * 2, &a2))) return rc;
        DECXB_CUDA_TRY(ctx, cudaMemcpy2DAsync(a2, Kp * 2, A, lda * 2, K * 2, M, cudaMemcpyDeviceToDevice, s));
        g.A = a2; g.lda = Kp;
    } else { g.A = A; g.lda = lda; }
    rc = decxb_launch_gemm_f16_tn(ctx, g, s);
    scratch.release();
    return rc;
}
}  // namespace

extern "C" int decxb_gemm_f16(decxb_ctx* ctx, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                              const void* B, int64_t ldb, const void* C, int64_t ldc, void* D, int64_t ldd, void* stream)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    return gemm_f16_device(ctx, M, N, K, A, lda, B, ldb, C, ldc, D, ldd, pick_stream(ctx, stream));
}

extern "C" int decxb_gemm_f16_host(decxb_ctx* ctx, int64_t M, int64_t N, int64_t K, const void* hA, int64_t lda,
                                   const void* hB, int64_t ldb, const void* hC, int64_t ldc, void* hD, int64_t ldd)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (M <= 0 || N <= 0 || K <= 0) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "gemm dims must be positive");
    if (!hA || !hB || !hD) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "null operand");
    if (lda < K || ldb < N || ldd < N || (hC && ldc < N))
        return decxb_fail(ctx, DECXB_ERR_DIM_MISMATCH, "leading dimension smaller than the row length");
    /* Three streams, as in the fp32 entry: B goes up first and is transposed once, then A (and C) in row blocks
     * of about an eighth of M: upload, product and the result's way home overlap.  (The reference stages the three
     * phases one after the other, GEMM.h:106-123.) */
    cudaStream_t s = ctx->stream, up = ctx->copy_stream[0], down = ctx->copy_stream[1];
    Scratch scratch(ctx, s);
    ChunkEvents evs;
    const int64_t Kp = decxb_ceil_to(K, 8), Np = decxb_ceil_to(N, 8);
    char *dA, *dB, *dC = nullptr, *dD, *bt;
    if ((rc = scratch.get((size_t)M * Kp * 2, (void**)&dA))) return rc;
    if ((rc = scratch.get((size_t)K * Np * 2, (void**)&dB))) return rc;
    if ((rc = scratch.get((size_t)M * Np * 2, (void**)&dD))) return rc;
    if (hC && (rc = scratch.get((size_t)M * Np * 2, (void**)&dC))) return rc;
    if ((rc = scratch.get((size_t)N * Kp * 2, (void**)&bt))) return rc;
    if ((rc = fence_copy_streams(ctx, evs))) return rc;
    auto fail = [&](int code) { drain_all_streams(ctx); return code; };
    cudaEvent_t e_b = evs.make();
    if (!e_b) return decxb_fail(ctx, DECXB_ERR_CUDA, "cudaEventCreate");
    PIPE_TRY(cudaMemcpy2DAsync(dB, Np * 2, hB, ldb * 2, N * 2, K, cudaMemcpyHostToDevice, up));
    PIPE_TRY(cudaEventRecord(e_b, up));
    PIPE_TRY(cudaStreamWaitEvent(s, e_b, 0));
    if ((rc = decxb_launch_transpose_f16(ctx, dB, K, N, Np, bt, Kp, s))) return fail(rc);
    int64_t rows = decxb_ceil_to(decxb_ceil_div(M, 8), 256);
    if (rows < 1024) rows = 1024;
    if (rows > M) rows = M;
    const char *hA8 = (const char*)hA, *hC8 = (const char*)hC;
    char* hD8 = (char*)hD;
    for (int64_t r0 = 0; r0 < M; r0 += rows) {
        const int64_t nr = M - r0 < rows ? M - r0 : rows;
        cudaEvent_t e_up = evs.make(), e_done = evs.make();
        if (!e_up || !e_done) return fail(decxb_fail(ctx, DECXB_ERR_CUDA, "cudaEventCreate"));
        PIPE_TRY(cudaMemcpy2DAsync(dA + r0 * Kp * 2, Kp * 2, hA8 + r0 * lda * 2, lda * 2, K * 2, nr, cudaMemcpyHostToDevice, up));
        if (hC) PIPE_TRY(cudaMemcpy2DAsync(dC + r0 * Np * 2, Np * 2, hC8 + r0 * ldc * 2, ldc * 2, N * 2, nr, cudaMemcpyHostToDevice, up));
        PIPE_TRY(cudaEventRecord(e_up, up));
        PIPE_TRY(cudaStreamWaitEvent(s, e_up, 0));
        decxb_gemm_f16_args g = {};
        g.M = nr; g.N = N; g.K = K;
        g.A = dA + r0 * Kp * 2; g.lda = Kp;               /* pitch ceil8(K): every row block starts on a 16-byte boundary */
        g.Bt = bt; g.ldbt = Kp;
        g.C = dC ? dC + r0 * Np * 2 : nullptr; g.ldc = Np;
        g.D = dD + r0 * Np * 2; g.ldd = Np;
        g.act = DECXB_ACT_NONE;
        if ((rc = decxb_launch_gemm_f16_tn(ctx, g, s))) return fail(rc);
        PIPE_TRY(cudaEventRecord(e_done, s));
        PIPE_TRY(cudaStreamWaitEvent(down, e_done, 0));
        PIPE_TRY(cudaMemcpy2DAsync(hD8 + r0 * ldd * 2, ldd * 2, dD + r0 * Np * 2, Np * 2, N * 2, nr, cudaMemcpyDeviceToHost, down));
    }
    if ((rc = sync_all_streams(ctx))) return rc;
    scratch.release();
    return decxb_check_dev_status(ctx);
}

/* ---- batched GEMM over arrays of equally sized matrices -------------------------------------- */
/* All matrices of the batch in ONE launch: the operands are split into stacked hi/lo arrays in
 * which every matrix occupies whole tiles, and the kernel's tile index runs over (matrix, tile). */
static int gemm_batched_device(decxb_ctx* ctx, int mode, int tile, int64_t batch, int64_t M, int64_t N, int64_t K,
                               const float* A, int64_t lda, int64_t strideA, const float* B, int64_t ldb, int64_t strideB,
                               const float* C, int64_t ldc, int64_t strideC, float* D, int64_t ldd, int64_t strideD,
                               cudaStream_t s)
{
    if (mode != DECXB_GEMM_3XTF32 && mode != DECXB_GEMM_1XTF32 && mode != DECXB_GEMM_3XTF32_STRICT)
        return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "gemm mode");
    if (batch < 0 || M <= 0 || N <= 0 || K <= 0) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "gemm dims must be positive");
    if (batch == 0) return DECXB_OK;
    if (!A || !B || !D) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "null operand");
    if (lda < K || ldb < N || ldd < N || (C && ldc < N))
        return decxb_fail(ctx, DECXB_ERR_DIM_MISMATCH, "leading dimension smaller than the row length");
    if (batch == 1)
        return gemm_device(ctx, mode, tile, M, N, K, A, lda, B, ldb, false, C, ldc, D, ldd, s);
    const bool strict = mode == DECXB_GEMM_3XTF32_STRICT;
    const bool x3 = mode == DECXB_GEMM_3XTF32 || strict;
    if (tile == DECXB_TILE_AUTO) tile = decxb_pick_tile(ctx, M, N, batch);
    int tm = 128, tn = 128;
    decxb_tile_shape(tile, &tm, &tn);
    const int64_t Kp = decxb_split_pitch(K), m_pad = decxb_ceil_to(M, tm), n_pad = decxb_ceil_to(N, tn);
    Scratch scratch(ctx, s);
    float *a_hi = nullptr, *a_lo = nullptr, *b_hi = nullptr, *b_lo = nullptr;
    int rc;
    if ((rc = scratch.get((size_t)batch * m_pad * Kp * 4, (void**)&a_hi))) return rc;
    if ((rc = scratch.get((size_t)batch * n_pad * Kp * 4, (void**)&b_hi))) return rc;
    if (x3) {
        if ((rc = scratch.get((size_t)batch * m_pad * Kp * 4, (void**)&a_lo))) return rc;
        if ((rc = scratch.get((size_t)batch * n_pad * Kp * 4, (void**)&b_lo))) return rc;
    }
    if ((rc = decxb_launch_split_rows(ctx, A, M, K, lda, a_hi, a_lo, Kp, m_pad, s, batch, strideA, x3 ? 0 : 1))) return rc;
    if ((rc = decxb_launch_split_transpose(ctx, B, K, N, ldb, b_hi, b_lo, Kp, x3 ? 0 : 1, s, batch, strideB, n_pad))) return rc;
    decxb_gemm_args g = {};
    g.M = M; g.N = N; g.K = K;
    g.a_hi = a_hi; g.a_lo = a_lo; g.lda = Kp;
    g.b_hi = b_hi; g.b_lo = b_lo; g.ldb = Kp; g.b_rows = n_pad;
    g.C = C; g.ldc = ldc; g.D = D; g.ldd = ldd; g.tile = tile;
    g.nbatch = batch; g.m_pad = m_pad; g.n_pad = n_pad; g.d_batch_stride = strideD; g.c_batch_stride = strideC;
    g.chunked = strict ? 1 : 0;
    rc = decxb_launch_gemm_tn(ctx, g, s);
    scratch.release();
    return rc;
}

extern "C" int decxb_gemm_f32_batched(decxb_ctx* ctx, int mode, int tile, int64_t batch, int64_t M, int64_t N, int64_t K,
                                      const float* A, int64_t lda, int64_t strideA,
                                      const float* B, int64_t ldb, int64_t strideB,
                                      const float* C, int64_t ldc, int64_t strideC,
                                      float* D, int64_t ldd, int64_t strideD, void* stream)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    return gemm_batched_device(ctx, mode, tile, batch, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC,
                               D, ldd, strideD, pick_stream(ctx, stream));
}

extern "C" int decxb_gemm_f32_batched_host(decxb_ctx* ctx, int mode, int tile, int64_t batch, int64_t M, int64_t N, int64_t K,
                                           const float* hA, int64_t lda, int64_t strideA,
                                           const float* hB, int64_t ldb, int64_t strideB,
                                           const float* hC, int64_t ldc, int64_t strideC,
                                           float* hD, int64_t ldd, int64_t strideD)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (batch < 0 || M <= 0 || N <= 0 || K <= 0) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "gemm dims must be positive");
    if (batch == 0) return DECXB_OK;
    if (!hA || !hB || !hD) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "null operand");
    if (lda < K || ldb < N || ldd < N || (hC && ldc < N))
        return decxb_fail(ctx, DECXB_ERR_DIM_MISMATCH, "leading dimension smaller than the row length");
    /* A ring of three device slots, each holding a GROUP of matrices (about 32 MiB of operands, so
     * small matrices still fill the GPU: a group is one batched launch).  Group i is uploaded
     * while group i-1 is multiplied and the results of group i-2 travel back (the reference
     * pipelines the same three phases, one matrix at a time, GEMM3_macros.h:140-248). */
    constexpr int SLOTS = 3;
    cudaStream_t s = ctx->stream, up = ctx->copy_stream[0], down = ctx->copy_stream[1];
    Scratch scratch(ctx, s);
    ChunkEvents evs;
    const int64_t Kp = decxb_ceil_to(K, 4), Np = decxb_ceil_to(N, 4);
    const int64_t per_matrix = (M * Kp + K * Np + M * Np) * 4;
    int64_t group = ((int64_t)32 << 20) / per_matrix;
    if (group < 1) group = 1;
    if (group > batch) group = batch;
    const int64_t ngroups = decxb_ceil_div(batch, group);
    const int nslots = ngroups < SLOTS ? (int)ngroups : SLOTS;
    float *dA[SLOTS], *dB[SLOTS], *dC[SLOTS] = {nullptr, nullptr, nullptr}, *dD[SLOTS];
    for (int k = 0; k < nslots; ++k) {
        if ((rc = scratch.get((size_t)group * M * Kp * 4, (void**)&dA[k]))) return rc;
        if ((rc = scratch.get((size_t)group * K * Np * 4, (void**)&dB[k]))) return rc;
        if ((rc = scratch.get((size_t)group * M * Np * 4, (void**)&dD[k]))) return rc;
        if (hC && (rc = scratch.get((size_t)group * M * Np * 4, (void**)&dC[k]))) return rc;
    }
    if ((rc = fence_copy_streams(ctx, evs))) return rc;
    auto fail = [&](int code) { drain_all_streams(ctx); return code; };
    std::vector<cudaEvent_t> e_done(ngroups, nullptr), e_down(ngroups, nullptr);
    for (int64_t gi = 0; gi < ngroups; ++gi) {
        const int k = (int)(gi % nslots);
        const int64_t i0 = gi * group, nb = batch - i0 < group ? batch - i0 : group;
        cudaEvent_t e_up = evs.make();
        e_done[gi] = evs.make(); e_down[gi] = evs.make();
        if (!e_up || !e_done[gi] || !e_down[gi]) return fail(decxb_fail(ctx, DECXB_ERR_CUDA, "cudaEventCreate"));
        if (gi >= nslots) PIPE_TRY(cudaStreamWaitEvent(up, e_done[gi - nslots], 0));      /* operands of the slot consumed */
        for (int64_t j = 0; j < nb; ++j) {
            PIPE_TRY(cudaMemcpy2DAsync(dA[k] + j * M * Kp, Kp * 4, hA + (i0 + j) * strideA, lda * 4, K * 4, M, cudaMemcpyHostToDevice, up));
            PIPE_TRY(cudaMemcpy2DAsync(dB[k] + j * K * Np, Np * 4, hB + (i0 + j) * strideB, ldb * 4, N * 4, K, cudaMemcpyHostToDevice, up));
            if (hC) PIPE_TRY(cudaMemcpy2DAsync(dC[k] + j * M * Np, Np * 4, hC + (i0 + j) * strideC, ldc * 4, N * 4, M, cudaMemcpyHostToDevice, up));
        }
        PIPE_TRY(cudaEventRecord(e_up, up));
        PIPE_TRY(cudaStreamWaitEvent(s, e_up, 0));
        if (gi >= nslots) PIPE_TRY(cudaStreamWaitEvent(s, e_down[gi - nslots], 0));       /* result slot drained */
        rc = gemm_batched_device(ctx, mode, tile, nb, M, N, K, dA[k], Kp, M * Kp, dB[k], Np, K * Np,
                                 dC[k], Np, M * Np, dD[k], Np, M * Np, s);
        if (rc) return fail(rc);
        PIPE_TRY(cudaEventRecord(e_done[gi], s));
        PIPE_TRY(cudaStreamWaitEvent(down, e_done[gi], 0));
        for (int64_t j = 0; j < nb; ++j)
            PIPE_TRY(cudaMemcpy2DAsync(hD + (i0 + j) * strideD, ldd * 4, dD[k] + j * M * Np, Np * 4, N * 4, M, cudaMemcpyDeviceToHost, down));
        PIPE_TRY(cudaEventRecord(e_down[gi], down));
    }
    if ((rc = sync_all_streams(ctx))) return rc;
    scratch.release();
    return decxb_check_dev_status(ctx);
}

/* ---- convolution ------------------------------------------------------------------------ */
extern "C" int decxb_conv_geometry(int64_t W, int64_t H, int64_t depth, int64_t kW, int64_t kH, int64_t N,
                                   int flag, decxb_conv_geom* g)
{
    if (!g) return DECXB_ERR_BAD_PARAM;
    if (W <= 0 || H <= 0 || depth <= 0 || kW <= 0 || kH <= 0 || N <= 0) return DECXB_ERR_BAD_PARAM;
    if (kW / 2 > 8 || kH / 2 > 8) return DECXB_ERR_BAD_KERNEL;   /* the reference's fixed apron of 8 */
    if (flag == DECXB_CONV_ZERO_COMPENSATE) { g->out_w = W; g->out_h = H; }
    else if (flag == DECXB_CONV_NO_COMPENSATE) {
        g->out_w = W - (kW / 2) * 2; g->out_h = H - (kH / 2) * 2;
        if (g->out_w <= 0 || g->out_h <= 0) return DECXB_ERR_BAD_KERNEL;
    } else return DECXB_ERR_BAD_FLAG;
    g->eq_w = decxb_ceil_to(g->out_w, 4);
    g->M = g->eq_w * g->out_h;
    g->Kp = kW * kH * decxb_ceil_to(depth, 4);
    g->Np = decxb_ceil_to(N, 4);
    return DECXB_OK;
}

extern "C" int decxb_im2col_pack_f32(decxb_ctx* ctx, const float* src, int64_t W, int64_t H, int64_t depth,
                                     int64_t kW, int64_t kH, int flag, float* i2c, int64_t batch,
                                     int64_t src_stride, int64_t i2c_stride, void* stream)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (!src || !i2c) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "null tensor");
    return decxb_launch_pack(ctx, src, W, H, depth, kW, kH, flag, i2c, batch, src_stride, i2c_stride, pick_stream(ctx, stream));
}

/* Filter bank prepared once (gathered into the filter matrix of the chosen algorithm, split into hi/lo). */
struct decxb_prepared_filters {
    decxb_ctx* ctx;
    int mode, algo;
    int64_t kW, kH, depth, N, ld;      /* ld: columns of the filter matrix */
    float *hi, *lo;
};

namespace {

int conv_device(decxb_ctx* ctx, int mode, int algo, int flag,
                const float* src, int64_t W, int64_t H, int64_t depth,
                const float* filters, int64_t kW, int64_t kH, int64_t N,
                float* dst, int64_t batch, int64_t src_stride, int64_t dst_stride, cudaStream_t s,
                const float* bias = nullptr, int act = DECXB_ACT_NONE, const decxb_prepared_filters* pf = nullptr)
{
    if (mode != DECXB_GEMM_3XTF32 && mode != DECXB_GEMM_1XTF32 && mode != DECXB_GEMM_3XTF32_STRICT)
        return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "gemm mode");
    if (act < DECXB_ACT_NONE || act > DECXB_ACT_TANH) return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "activation");
    if (algo != DECXB_CONV_EXPLICIT && algo != DECXB_CONV_IMPLICIT) return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "conv algo");
    if (!src || (!filters && !pf) || !dst) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "null tensor");
    decxb_conv_geom g;
    int rc = decxb_conv_geometry(W, H, depth, kW, kH, N, flag, &g);
    if (rc) return decxb_fail(ctx, rc, "convolution geometry");
    if (batch <= 0) return DECXB_OK;
    const int64_t dp = decxb_ceil_to(depth, 4), wp = decxb_ceil_to(W, 4);
    if (src_stride == 0) src_stride = H * wp * dp;
    if (dst_stride == 0) dst_stride = g.M * g.Np;
    const bool strict = mode == DECXB_GEMM_3XTF32_STRICT;
    const bool x3 = mode == DECXB_GEMM_3XTF32 || strict;
    Scratch scratch(ctx, s);
    if (algo == DECXB_CONV_IMPLICIT) {
        /* The column matrix is never written: the GEMM's A tiles are TMA boxes of the (split)
         * source tensor, one filter tap and 32 channels per k-block. */
        if (((uintptr_t)src % 16) || (src_stride % 4) || ((uintptr_t)dst % 16) || (dst_stride % 4))
            return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "implicit convolution needs 16-byte aligned tensors");
        if (H * wp * dp > 0x7fffffffffLL || batch > 0x7fffffffLL) return decxb_fail(ctx, DECXB_ERR_TOO_LARGE, "tensor");
        const int64_t cp = decxb_ceil_to(dp, 32), Kc = kW * kH * cp;
        float *k_hi = nullptr, *k_lo = nullptr, *s_hi = nullptr, *s_lo = nullptr;
        if (pf) { k_hi = pf->hi; k_lo = pf->lo; }
        else {
            if ((rc = scratch.get((size_t)g.Np * Kc * 4, (void**)&k_hi))) return rc;
            if (x3 && (rc = scratch.get((size_t)g.Np * Kc * 4, (void**)&k_lo))) return rc;
            if ((rc = decxb_launch_filter_matrix(ctx, filters, kW, kH, depth, N, k_hi, k_lo, g.Np, Kc, x3 ? 0 : 1, s, cp))) return rc;
        }
        decxb_conv_gemm_args a = {};
        const int64_t img = H * wp * dp;
        if (x3) {
            if ((rc = scratch.get((size_t)batch * img * 4, (void**)&s_hi))) return rc;
            if ((rc = scratch.get((size_t)batch * img * 4, (void**)&s_lo))) return rc;
            if (src_stride == img) {
                if ((rc = decxb_launch_split_rows(ctx, src, batch * H * wp, dp, dp, s_hi, s_lo, dp, batch * H * wp, s))) return rc;
            } else {
                for (int64_t b0 = 0; b0 < batch; ++b0)
                    if ((rc = decxb_launch_split_rows(ctx, src + b0 * src_stride, H * wp, dp, dp, s_hi + b0 * img, s_lo + b0 * img,
                                                      dp, H * wp, s))) return rc;
            }
            a.src_hi = s_hi; a.src_lo = s_lo; a.src_img_stride = img;
        } else { a.src_hi = src; a.src_lo = nullptr; a.src_img_stride = src_stride; }
        a.dp = dp; a.wp = wp; a.H = H; a.batch = batch;
        a.k_hi = k_hi; a.k_lo = k_lo; a.k_rows = g.Np; a.k_cols = Kc; a.ldk = Kc;
        a.kW = kW; a.kH = kH;
        a.off_x = flag == DECXB_CONV_ZERO_COMPENSATE ? -(int)(kW / 2) : 0;
        a.off_y = flag == DECXB_CONV_ZERO_COMPENSATE ? -(int)(kH / 2) : 0;
        a.out_h = g.out_h; a.eq_w = g.eq_w; a.Np = g.Np;
        a.dst = dst; a.dst_img_stride = dst_stride;
        a.bias = bias; a.act = act;
        a.chunked = strict ? 1 : 0;
        rc = decxb_launch_conv_implicit(ctx, a, s);
        scratch.release();
        return rc;
    }

    /* filter matrix [Np][Kp] (hi/lo), rows >= N zero so padding channels come out 0 */
    float *k_hi = nullptr, *k_lo = nullptr;
    if (pf) { k_hi = pf->hi; k_lo = pf->lo; }
    else {
        if ((rc = scratch.get((size_t)g.Np * g.Kp * 4, (void**)&k_hi))) return rc;
        if (x3 && (rc = scratch.get((size_t)g.Np * g.Kp * 4, (void**)&k_lo))) return rc;
        if ((rc = decxb_launch_filter_matrix(ctx, filters, kW, kH, depth, N, k_hi, k_lo, g.Np, g.Kp, x3 ? 0 : 1, s))) return rc;
    }

    /* images are processed in groups so that the column matrix of a group stays a few hundred MB */
    const int64_t i2c_bytes_img = g.M * g.Kp * 4;
    int64_t group = (512LL << 20) / i2c_bytes_img;
    if (group < 1) group = 1;
    if (group > batch) group = batch;
    /* a group of images forms ONE tall GEMM when the destination images are densely packed */
    const bool dense_dst = dst_stride == g.M * g.Np;
    /* 3xTF32: the pack is pure indexing, so packing the hi and lo parts of the SOURCE gives the
     * hi and lo parts of the column matrix; the fp32 column matrix itself is not needed here
     * (decxb_im2col_pack_f32 is the entry that delivers it) and is neither written nor re-read. */
    float *i2c = nullptr, *a_hi = nullptr, *a_lo = nullptr, *s_hi = nullptr, *s_lo = nullptr;
    const int64_t img = H * wp * dp;
    if (x3) {
        if ((rc = scratch.get((size_t)group * i2c_bytes_img, (void**)&a_hi))) return rc;
        if ((rc = scratch.get((size_t)group * i2c_bytes_img, (void**)&a_lo))) return rc;
        if ((rc = scratch.get((size_t)group * img * 4, (void**)&s_hi))) return rc;
        if ((rc = scratch.get((size_t)group * img * 4, (void**)&s_lo))) return rc;
    } else {
        if ((rc = scratch.get((size_t)group * i2c_bytes_img, (void**)&i2c))) return rc;
    }
    for (int64_t b0 = 0; b0 < batch; b0 += group) {
        const int64_t nb = batch - b0 < group ? batch - b0 : group;
        if (x3) {
            for (int64_t j = 0; j < (src_stride == img ? 1 : nb); ++j) {
                const int64_t rows = (src_stride == img ? nb : 1) * H * wp;
                if ((rc = decxb_launch_split_rows(ctx, src + (b0 + j) * src_stride, rows, dp, dp, s_hi + j * img, s_lo + j * img,
                                                  dp, rows, s))) return rc;
            }
            if ((rc = decxb_launch_pack(ctx, s_hi, W, H, depth, kW, kH, flag, a_hi, nb, img, g.M * g.Kp, s))) return rc;
            if ((rc = decxb_launch_pack(ctx, s_lo, W, H, depth, kW, kH, flag, a_lo, nb, img, g.M * g.Kp, s))) return rc;
        } else {
            if ((rc = decxb_launch_pack(ctx, src + b0 * src_stride, W, H, depth, kW, kH, flag, i2c, nb, src_stride, g.M * g.Kp, s))) return rc;
        }
        const int64_t n_gemm = dense_dst ? 1 : nb;
        const int64_t rows_per = dense_dst ? nb * g.M : g.M;
        for (int64_t j = 0; j < n_gemm; ++j) {
            decxb_gemm_args a = {};
            a.M = rows_per; a.N = g.Np; a.K = g.Kp;
            a.a_hi = (x3 ? a_hi : i2c) + j * g.M * g.Kp; a.a_lo = x3 ? a_lo + j * g.M * g.Kp : nullptr; a.lda = g.Kp;
            a.b_hi = k_hi; a.b_lo = k_lo; a.ldb = g.Kp; a.b_rows = g.Np;
            a.C = nullptr; a.ldc = 0;
            a.D = dst + (b0 + j) * dst_stride; a.ldd = g.Np;
            a.tile = DECXB_TILE_AUTO;
            a.bias = bias; a.act = act;
            a.chunked = strict ? 1 : 0;
            if ((rc = decxb_launch_gemm_tn(ctx, a, s))) return rc;
        }
    }
    scratch.release();
    return DECXB_OK;
}

}  // namespace

extern "C" int decxb_conv_prepare_filters(decxb_ctx* ctx, int mode, int algo, const float* filters, int64_t kW, int64_t kH,
                                          int64_t depth, int64_t N, void* stream, decxb_prepared_filters** out)
{
    if (!out) return DECXB_ERR_BAD_PARAM;
    *out = nullptr;
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (mode != DECXB_GEMM_3XTF32 && mode != DECXB_GEMM_1XTF32 && mode != DECXB_GEMM_3XTF32_STRICT)
        return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "gemm mode");
    if (algo != DECXB_CONV_EXPLICIT && algo != DECXB_CONV_IMPLICIT) return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "conv algo");
    decxb_conv_geom g;
    if (!filters || (rc = decxb_conv_geometry(2 * kW, 2 * kH, depth, kW, kH, N, DECXB_CONV_ZERO_COMPENSATE, &g)))
        return decxb_fail(ctx, rc ? rc : DECXB_ERR_BAD_PARAM, "filter bank");
    cudaStream_t s = pick_stream(ctx, stream);
    const bool x3 = mode != DECXB_GEMM_1XTF32;
    const int64_t dp = decxb_ceil_to(depth, 4);
    const int64_t cp = algo == DECXB_CONV_IMPLICIT ? decxb_ceil_to(dp, 32) : dp;
    const int64_t ld = kW * kH * cp;
    float *hi = nullptr, *lo = nullptr;
    if ((rc = decxb_malloc_on_stream(ctx, (size_t)g.Np * ld * 4, (void**)&hi, s))) return rc;
    if (x3 && (rc = decxb_malloc_on_stream(ctx, (size_t)g.Np * ld * 4, (void**)&lo, s))) { decxb_free_on_stream(ctx, hi, s); return rc; }
    rc = decxb_launch_filter_matrix(ctx, filters, kW, kH, depth, N, hi, lo, g.Np, ld, x3 ? 0 : 1, s, algo == DECXB_CONV_IMPLICIT ? cp : 0);
    if (rc) { decxb_free_on_stream(ctx, hi, s); if (lo) decxb_free_on_stream(ctx, lo, s); return rc; }
    *out = new decxb_prepared_filters{ctx, mode, algo, kW, kH, depth, N, ld, hi, lo};
    return DECXB_OK;
}

extern "C" int decxb_conv_release_filters(decxb_ctx* ctx, decxb_prepared_filters* pf, void* stream)
{
    if (!pf) return DECXB_OK;
    if (!ctx || pf->ctx != ctx) return DECXB_ERR_BAD_PARAM;
    cudaStream_t s = pick_stream(ctx, stream);
    decxb_free_on_stream(ctx, pf->hi, s);
    if (pf->lo) decxb_free_on_stream(ctx, pf->lo, s);
    delete pf;
    return DECXB_OK;
}

extern "C" int decxb_conv2_im2col_f32_prepared(decxb_ctx* ctx, int flag, const float* src, int64_t W, int64_t H,
                                               const decxb_prepared_filters* pf, const float* bias, int activation,
                                               float* dst, int64_t batch, int64_t src_stride, int64_t dst_stride, void* stream)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (!pf || pf->ctx != ctx) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "prepared filters of another context");
    return conv_device(ctx, pf->mode, pf->algo, flag, src, W, H, pf->depth, nullptr, pf->kW, pf->kH, pf->N, dst, batch, src_stride,
                       dst_stride, pick_stream(ctx, stream), bias, activation, pf);
}

extern "C" int decxb_conv2_im2col_f32(decxb_ctx* ctx, int mode, int algo, int flag,
                                      const float* src, int64_t W, int64_t H, int64_t depth,
                                      const float* filters, int64_t kW, int64_t kH, int64_t N,
                                      float* dst, int64_t batch, int64_t src_stride, int64_t dst_stride, void* stream)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    return conv_device(ctx, mode, algo, flag, src, W, H, depth, filters, kW, kH, N, dst, batch, src_stride, dst_stride,
                       pick_stream(ctx, stream));
}

extern "C" int decxb_conv2_im2col_f32_act(decxb_ctx* ctx, int mode, int algo, int flag,
                                          const float* src, int64_t W, int64_t H, int64_t depth,
                                          const float* filters, int64_t kW, int64_t kH, int64_t N,
                                          const float* bias, int activation,
                                          float* dst, int64_t batch, int64_t src_stride, int64_t dst_stride, void* stream)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    return conv_device(ctx, mode, algo, flag, src, W, H, depth, filters, kW, kH, N, dst, batch, src_stride, dst_stride,
                       pick_stream(ctx, stream), bias, activation);
}

extern "C" int decxb_conv2_im2col_f32_host(decxb_ctx* ctx, int mode, int algo, int flag,
                                           const float* h_src, int64_t W, int64_t H, int64_t depth,
                                           const float* h_filters, int64_t kW, int64_t kH, int64_t N,
                                           float* h_dst, int64_t batch, int64_t src_stride, int64_t dst_stride)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (!h_src || !h_filters || !h_dst) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "null tensor");
    decxb_conv_geom g;
    rc = decxb_conv_geometry(W, H, depth, kW, kH, N, flag, &g);
    if (rc) return decxb_fail(ctx, rc, "convolution geometry");
    if (batch <= 0) return DECXB_OK;
    const int64_t dp = decxb_ceil_to(depth, 4), wp = decxb_ceil_to(W, 4), kwp = decxb_ceil_to(kW, 4);
    const int64_t src_img = H * wp * dp, dst_img = g.M * g.Np;
    if (src_stride == 0) src_stride = src_img;
    if (dst_stride == 0) dst_stride = dst_img;
    /* uploads, compute and downloads on three streams, pipelined over groups of images; the
     * filter bank goes up in one copy (the reference issues one 2-D copy per filter,
     * conv2_mk_im2col.h:226-231) */
    cudaStream_t s = ctx->stream, up = ctx->copy_stream[0], down = ctx->copy_stream[1];
    Scratch scratch(ctx, s);
    ChunkEvents evs;
    float *d_src, *d_flt, *d_dst;
    if ((rc = scratch.get((size_t)batch * src_img * 4, (void**)&d_src))) return rc;
    if ((rc = scratch.get((size_t)N * kH * kwp * dp * 4, (void**)&d_flt))) return rc;
    if ((rc = scratch.get((size_t)batch * dst_img * 4, (void**)&d_dst))) return rc;
    if ((rc = fence_copy_streams(ctx, evs))) return rc;
    auto fail = [&](int code) { drain_all_streams(ctx); return code; };
    PIPE_TRY(cudaMemcpyAsync(d_flt, h_filters, (size_t)N * kH * kwp * dp * 4, cudaMemcpyHostToDevice, up));
    /* the filter matrix is built once for all image groups, as soon as the bank has landed */
    cudaEvent_t e_flt = evs.make();
    if (!e_flt) return fail(decxb_fail(ctx, DECXB_ERR_CUDA, "cudaEventCreate"));
    PIPE_TRY(cudaEventRecord(e_flt, up));
    PIPE_TRY(cudaStreamWaitEvent(s, e_flt, 0));
    decxb_prepared_filters* pf = nullptr;
    if ((rc = decxb_conv_prepare_filters(ctx, mode, algo, d_flt, kW, kH, depth, N, s, &pf))) return fail(rc);
    struct PfGuard { decxb_ctx* c; decxb_prepared_filters* p; cudaStream_t st; ~PfGuard() { decxb_conv_release_filters(c, p, st); } } pf_guard{ctx, pf, s};
    /* many small groups: the first upload and the last download are not overlapped with anything,
     * so they should be short; 1/32 of the batch, but at least 8 MiB per copy */
    int64_t group = decxb_ceil_div(batch, 32);
    const int64_t min_group = decxb_ceil_div((int64_t)8 << 20, src_img * 4);      /* at least 8 MiB per upload */
    if (group < min_group) group = min_group;
    if (group > batch) group = batch;
    for (int64_t b0 = 0; b0 < batch; b0 += group) {
        const int64_t nb = batch - b0 < group ? batch - b0 : group;
        cudaEvent_t e_up = evs.make(), e_done = evs.make();
        if (!e_up || !e_done) return fail(decxb_fail(ctx, DECXB_ERR_CUDA, "cudaEventCreate"));
        PIPE_TRY(cudaMemcpy2DAsync(d_src + b0 * src_img, src_img * 4, h_src + b0 * src_stride, src_stride * 4,
                                             src_img * 4, nb, cudaMemcpyHostToDevice, up));
        PIPE_TRY(cudaEventRecord(e_up, up));
        PIPE_TRY(cudaStreamWaitEvent(s, e_up, 0));
        rc = conv_device(ctx, mode, algo, flag, d_src + b0 * src_img, W, H, depth, nullptr, kW, kH, N, d_dst + b0 * dst_img,
                         nb, src_img, dst_img, s, nullptr, DECXB_ACT_NONE, pf);
        if (rc) return fail(rc);
        PIPE_TRY(cudaEventRecord(e_done, s));
        PIPE_TRY(cudaStreamWaitEvent(down, e_done, 0));
        PIPE_TRY(cudaMemcpy2DAsync(h_dst + b0 * dst_stride, dst_stride * 4, d_dst + b0 * dst_img, dst_img * 4,
                                             dst_img * 4, nb, cudaMemcpyDeviceToHost, down));
    }
    if ((rc = sync_all_streams(ctx))) return rc;
    scratch.release();
    return decxb_check_dev_status(ctx);
}

/* ---- sharding over ranks ----------------------------------------------------------------------- */
extern "C" int decxb_shard_range(int64_t total, int world, int rank, int64_t* first, int64_t* last)
{
    if (total < 0 || world <= 0 || rank < 0 || rank >= world) return DECXB_ERR_BAD_PARAM;
    const int64_t base = total / world, extra = total % world;
    const int64_t f = rank * base + (rank < extra ? rank : extra);
    if (first) *first = f;
    if (last) *last = f + base + (rank < extra ? 1 : 0);
    return DECXB_OK;
}

extern "C" int decxb_gemm_f32_rowshard(decxb_ctx* ctx, int mode, int tile, int world, int rank,
                                       int64_t M, int64_t N, int64_t K,
                                       const float* A_rows, int64_t lda, const float* B, int64_t ldb,
                                       const float* C_rows, int64_t ldc, float* D_rows, int64_t ldd,
                                       void* stream, int64_t* first, int64_t* last)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    int64_t f = 0, l = 0;
    if (decxb_shard_range(M, world, rank, &f, &l)) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "bad world/rank");
    if (first) *first = f;
    if (last) *last = l;
    if (l == f) return DECXB_OK;                 /* more ranks than rows: nothing to do here */
    return gemm_device(ctx, mode, tile, l - f, N, K, A_rows, lda, B, ldb, false, C_rows, ldc, D_rows, ldd, pick_stream(ctx, stream));
}

extern "C" int decxb_conv2_im2col_f32_batchshard(decxb_ctx* ctx, int mode, int algo, int flag, int world, int rank,
                                                 const float* src, int64_t W, int64_t H, int64_t depth,
                                                 const float* filters, int64_t kW, int64_t kH, int64_t N,
                                                 float* dst, int64_t batch, int64_t src_stride, int64_t dst_stride,
                                                 void* stream, int64_t* first, int64_t* last)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    int64_t f = 0, l = 0;
    if (decxb_shard_range(batch, world, rank, &f, &l)) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "bad world/rank");
    if (first) *first = f;
    if (last) *last = l;
    if (l == f) return DECXB_OK;
    return conv_device(ctx, mode, algo, flag, src, W, H, depth, filters, kW, kH, N, dst, l - f, src_stride, dst_stride,
                       pick_stream(ctx, stream));
}
