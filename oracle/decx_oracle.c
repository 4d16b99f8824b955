/*
 * decx_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C CPU restatement of the arithmetic of DECX's fp32 GEMM and im2col
 * convolution.  It exists only to check the CUDA library: the test-suite, the
 * smoke check and the CPU-baseline leg of the benchmark may call it; the
 * product library never links, loads or calls anything in this file.
 *
 * Parity status: PINNED.  The GEMM chain below is checked bit-for-bit against
 * the reference's own CPU GEMM (decx::sgemm_caller, compiled from the
 * reference tree into oracle/_ref) and against the analytic known-answer case
 * of the reference's test program test/test/CUDA_GEMM/CUDA_GEMM.cpp:24-42.
 * The im2col pack and the convolution have no test in the reference; they are
 * pinned against the reference's own CUDA kernel sources executed on host
 * threads (oracle/ref_kernels_host.cpp) and against the golden vectors that
 * run produced (tests/golden/).
 *
 * Each function names the reference file:line whose behaviour it restates
 * (paths are relative to the reference project root).
 */
#ifndef _GNU_SOURCE
#define _GNU_SOURCE
#endif
#include <math.h>
#include <pthread.h>
#include <sched.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define DECXO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------
 * Row-parallel helper (plain pthreads): body(ctx, first, last) is called on
 * disjoint row ranges.  Every output element is still computed by one
 * thread in the order the restated algorithm prescribes.
 * ---------------------------------------------------------------------- */
typedef void (*decxo_range_fn)(void* ctx, int64_t first, int64_t last);
typedef struct { decxo_range_fn fn; void* ctx; int64_t first, last; } decxo_job;

static void* decxo_job_main(void* p)
{
    decxo_job* j = (decxo_job*)p;
    j->fn(j->ctx, j->first, j->last);
    return NULL;
}

static int g_threads = 0;

DECXO_API int decxo_num_threads(void)
{
    if (g_threads > 0) return g_threads;
    cpu_set_t set;
    int n = 1;
    if (sched_getaffinity(0, sizeof(set), &set) == 0) n = CPU_COUNT(&set);
    if (n < 1) n = 1;
    if (n > 64) n = 64;
    return n;
}

DECXO_API void decxo_set_num_threads(int n) { g_threads = n; }

static void parallel_rows(decxo_range_fn fn, void* ctx, int64_t n)
{
    int nt = decxo_num_threads();
    if (n < 2 * nt) nt = n > 1 ? (int)(n / 2) : 1;
    if (nt <= 1) { fn(ctx, 0, n); return; }
    pthread_t th[64]; decxo_job jobs[64];
    const int64_t chunk = (n + nt - 1) / nt;
    int started = 0;
    for (int t = 0; t < nt; ++t) {
        jobs[t].fn = fn; jobs[t].ctx = ctx;
        jobs[t].first = t * chunk; jobs[t].last = (t + 1) * chunk < n ? (t + 1) * chunk : n;
        if (jobs[t].first >= jobs[t].last) break;
        if (pthread_create(&th[t], NULL, decxo_job_main, &jobs[t]) != 0) { fn(ctx, jobs[t].first, jobs[t].last); th[t] = 0; }
        started = t + 1;
    }
    for (int t = 0; t < started; ++t) if (th[t]) pthread_join(th[t], NULL);
}

/* ------------------------------------------------------------------------
 * Seeded synthetic data: counter-based, so host, device and every rank can
 * produce element i of stream `seed` independently.  v in [-1, 1).
 * (No counterpart in the reference, whose tests fill matrices with index
 * formulas; the CUDA library carries a device twin of this generator and the
 * tests check that both produce identical bits.)
 * ---------------------------------------------------------------------- */
static inline uint32_t fmix32(uint32_t h)
{
    h ^= h >> 16; h *= 0x85EBCA6Bu;
    h ^= h >> 13; h *= 0xC2B2AE35u;
    h ^= h >> 16;
    return h;
}

static inline float uniform_pm1(uint32_t seed, uint64_t idx)
{
    uint32_t hi = fmix32((uint32_t)(idx >> 32) + seed * 0x85EBCA77u + 0x165667B1u);
    uint32_t u  = fmix32(((uint32_t)idx * 0x9E3779B1u) ^ hi);
    return (float)(u >> 8) * (1.0f / 8388608.0f) - 1.0f;
}

DECXO_API void decxo_fill_uniform(float* dst, uint64_t n, uint32_t seed, uint64_t first_index)
{
    for (uint64_t i = 0; i < n; ++i) dst[i] = uniform_pm1(seed, first_index + i);
}

/* Fill a pitched 2-D array: element (r, c) takes counter r*cols + c; the
 * pitch tail is set to zero (DECX containers zero their padding,
 * srcs/classes/Tensor.h:312). */
DECXO_API void decxo_fill_uniform_2d(float* dst, uint64_t rows, uint64_t cols, uint64_t pitch,
                                     uint32_t seed, uint64_t first_index)
{
    for (uint64_t r = 0; r < rows; ++r) {
        float* row = dst + r * pitch;
        for (uint64_t c = 0; c < cols; ++c) row[c] = uniform_pm1(seed, first_index + r * cols + c);
        for (uint64_t c = cols; c < pitch; ++c) row[c] = 0.0f;
    }
}

/* ------------------------------------------------------------------------
 * GEMM.  D = A*B (+C).  The reference's CUDA kernels compute every output as
 * ONE fp32 fused-multiply-add chain with k strictly ascending:
 *     c = 0 (or C[i][j]);  for k = 0..K-1:  c = fmaf(A[i][k], B[k][j], c)
 * srcs/GEMM/CUDA/large_squares/GEMM.cuh:53-94 (k loop), :83-92 (the 16 inner
 * steps), accumulator preload for A*B+C at :223; FMA macro at
 * srcs/GEMM/CUDA/GEMM_kernel_def.cuh:33-55.  The reference's CPU GEMM
 * (srcs/GEMM/CPU/sgemm_calc_kernel.h:24-29, _mm256_fmadd_ps with a[k]
 * broadcast) produces the same bits.
 * The j loop is innermost so the compiler can vectorise across columns; every
 * (i, j) still sees its own chain in ascending k.
 * ---------------------------------------------------------------------- */
typedef struct {
    int64_t M, N, K; const float *A, *B, *C; float* D; double* D64; int64_t lda, ldb, ldc, ldd;
} gemm_ctx;

static void gemm_fmaf_rows(void* p, int64_t i0, int64_t i1)
{
    const gemm_ctx* g = (const gemm_ctx*)p;
    for (int64_t i = i0; i < i1; ++i) {
        float* restrict d = g->D + i * g->ldd;
        if (g->C) memcpy(d, g->C + i * g->ldc, (size_t)g->N * sizeof(float));
        else      memset(d, 0, (size_t)g->N * sizeof(float));
        const float* a = g->A + i * g->lda;
        for (int64_t k = 0; k < g->K; ++k) {
            const float av = a[k];
            const float* restrict b = g->B + k * g->ldb;
            for (int64_t j = 0; j < g->N; ++j) d[j] = fmaf(av, b[j], d[j]);
        }
    }
}

DECXO_API void decxo_gemm_fmaf(int64_t M, int64_t N, int64_t K,
                               const float* A, int64_t lda,
                               const float* B, int64_t ldb,
                               const float* C, int64_t ldc,
                               float* D, int64_t ldd)
{
    gemm_ctx g = { M, N, K, A, B, C, D, NULL, lda, ldb, ldc, ldd };
    parallel_rows(gemm_fmaf_rows, &g, M);
}

/* Same product with B given K-contiguous ([N][K], "ker_buf" orientation of
 * srcs/convolution/CUDA/im2col/eq_GEMM.cuh:109-209: dst[m][n] = sum_k
 * I2C[m][k] * ker_buf[n][k], one ascending-k fmaf chain, :65-74, :172-193). */
static void gemm_fmaf_nt_rows(void* p, int64_t i0, int64_t i1)
{
    const gemm_ctx* g = (const gemm_ctx*)p;
    for (int64_t i = i0; i < i1; ++i) {
        const float* a = g->A + i * g->lda;
        for (int64_t j = 0; j < g->N; ++j) {
            const float* b = g->B + j * g->ldb;
            float c = 0.0f;
            for (int64_t k = 0; k < g->K; ++k) c = fmaf(a[k], b[k], c);
            g->D[i * g->ldd + j] = c;
        }
    }
}

DECXO_API void decxo_gemm_fmaf_nt(int64_t M, int64_t N, int64_t K,
                                  const float* A, int64_t lda,
                                  const float* Bt, int64_t ldbt,
                                  float* D, int64_t ldd)
{
    gemm_ctx g = { M, N, K, A, Bt, NULL, D, NULL, lda, ldbt, 0, ldd };
    parallel_rows(gemm_fmaf_nt_rows, &g, M);
}

/* fp64 product, reported beside the fp32 chain (not a reference behaviour). */
static void gemm_f64_rows(void* p, int64_t i0, int64_t i1)
{
    const gemm_ctx* g = (const gemm_ctx*)p;
    for (int64_t i = i0; i < i1; ++i) {
        double* restrict d = g->D64 + i * g->ldd;
        for (int64_t j = 0; j < g->N; ++j) d[j] = g->C ? (double)g->C[i * g->ldc + j] : 0.0;
        for (int64_t k = 0; k < g->K; ++k) {
            const double av = (double)g->A[i * g->lda + k];
            const float* restrict b = g->B + k * g->ldb;
            for (int64_t j = 0; j < g->N; ++j) d[j] += av * (double)b[j];
        }
    }
}

DECXO_API void decxo_gemm_f64(int64_t M, int64_t N, int64_t K,
                              const float* A, int64_t lda,
                              const float* B, int64_t ldb,
                              const float* C, int64_t ldc,
                              double* D, int64_t ldd)
{
    gemm_ctx g = { M, N, K, A, B, C, NULL, D, lda, ldb, ldc, ldd };
    parallel_rows(gemm_f64_rows, &g, M);
}

/* ------------------------------------------------------------------------
 * Tensor geometry.  DECX tensors are HWC with the channel innermost and both
 * the channel and the width padded to a multiple of 4:
 *   dpitch = ceil(depth/4)*4, wpitch = ceil(width/4)*4,
 *   element (row, col, ch) at ptr[(row*wpitch + col)*dpitch + ch]
 * srcs/classes/Tensor.h:162-184 (attributes), :389-394 (index).
 * ---------------------------------------------------------------------- */
static inline int64_t ceil4(int64_t v) { return (v + 3) / 4 * 4; }

typedef struct {
    int64_t out_w, out_h;   /* logical output size                          */
    int64_t eq_w;           /* ceil4(out_w): pixels per output row in I2C    */
    int64_t M;              /* eq_w * out_h rows of the column matrix        */
    int64_t Kp;             /* kW*kH*dpitch columns of the column matrix     */
    int64_t off_y, off_x;   /* source offset of tap (0,0) for output (0,0)   */
} decxo_conv_geom;

/* srcs/convolution/CUDA/im2col/conv2_mk_im2col.h:62-66,77-78,85-86 (valid
 * mode, flag 0) and :172-176,188-189,195-196 (zero-border mode, flag 1). */
DECXO_API int decxo_conv_geometry(int64_t W, int64_t H, int64_t depth, int64_t kW, int64_t kH, int flag,
                                  decxo_conv_geom* g)
{
    if (W <= 0 || H <= 0 || depth <= 0 || kW <= 0 || kH <= 0) return 1;
    if (kW / 2 > 8 || kH / 2 > 8) return 2;           /* fixed apron of 8, :170 */
    const int64_t dp = ceil4(depth);
    if (flag == 1) {            /* de_conv_zero_compensate */
        g->out_w = W; g->out_h = H;
        g->off_y = -(kH / 2); g->off_x = -(kW / 2);
    } else if (flag == 0) {     /* de_conv_no_compensate */
        g->out_w = W - (kW / 2) * 2; g->out_h = H - (kH / 2) * 2;
        g->off_y = 0; g->off_x = 0;
        if (g->out_w <= 0 || g->out_h <= 0) return 3;
    } else return 4;
    g->eq_w = ceil4(g->out_w);
    g->M = g->eq_w * g->out_h;
    g->Kp = kW * kH * dp;
    return 0;
}

/* ------------------------------------------------------------------------
 * im2col pack.  Restates cu_sIm2Col_r8_within
 * (srcs/convolution/CUDA/im2col/im2col.cuh:86-178) together with the
 * staging that feeds it (conv2_mk_im2col.h:234-238: the host tensor is
 * copied, padding pixels included, into a larger buffer at pixel offset
 * (8,8) for the zero-border mode, or (8-kH/2, 8-kW/2) for the valid mode;
 * the rest of that buffer, the apron, is taken to be zero).
 *
 * Thread (row y, column group) of the kernel writes, for each tap (ky, kx)
 * and channel slice, the value it finds at
 *    frag[ty + kernel_shift.x + ky][4*tx + kernel_shift.y + kx + j]
 * (im2col.cuh:146-172), which is buffer pixel (y + 8 - kH/2 + ky,
 * x + 8 - kW/2 + kx).  Mapped back to source coordinates this is
 *    I2C[(y*eq_w + x)*Kp + (ky*kW + kx)*dpitch + c] = S[y + ky + off_y][x + kx + off_x][c]
 * with S = source value when 0<=row<H and 0<=col<wpitch (padding pixels of
 * the tensor are part of the copy and are zero in a DECX tensor), else 0.
 * Columns are ordered (ky, kx, c) with c innermost: glo_dex_dst =
 * row*pitch_dst + ker_iter*depth + i (im2col.cuh:153).
 * ---------------------------------------------------------------------- */
DECXO_API int decxo_im2col_pack(const float* src, int64_t W, int64_t H, int64_t depth,
                                int64_t kW, int64_t kH, int flag, float* i2c)
{
    decxo_conv_geom g;
    int rc = decxo_conv_geometry(W, H, depth, kW, kH, flag, &g);
    if (rc) return rc;
    const int64_t dp = ceil4(depth), wp = ceil4(W);
    for (int64_t y = 0; y < g.out_h; ++y) {
        for (int64_t x = 0; x < g.eq_w; ++x) {
            float* row = i2c + (y * g.eq_w + x) * g.Kp;
            for (int64_t ky = 0; ky < kH; ++ky) {
                for (int64_t kx = 0; kx < kW; ++kx) {
                    const int64_t r = y + ky + g.off_y, q = x + kx + g.off_x;
                    float* seg = row + (ky * kW + kx) * dp;
                    if (r >= 0 && r < H && q >= 0 && q < wp)
                        memcpy(seg, src + (r * wp + q) * dp, (size_t)dp * sizeof(float));
                    else
                        memset(seg, 0, (size_t)dp * sizeof(float));
                }
            }
        }
    }
    return 0;
}

/* Filter bank -> [n_pad][Kp] matrix, filter n in row n, column
 * (ky*kW + kx)*dpitch + c.  conv2_mk_im2col.h:226-231: one 2-D copy per
 * filter of kH rows of kW*dpitch floats out of a TensorArray whose filters
 * lie `gap = dpitch*wpitch*kH` floats apart (srcs/classes/TensorArray.h:174-198).
 * Rows n >= N are zero.  `ld` is the row pitch of the result. */
DECXO_API void decxo_kernel_matrix(const float* filters, int64_t kW, int64_t kH, int64_t depth, int64_t N,
                                   int64_t n_rows, int64_t ld, float* ker)
{
    const int64_t dp = ceil4(depth), kwp = ceil4(kW);
    const int64_t gap = dp * kwp * kH;
    memset(ker, 0, (size_t)(n_rows * ld) * sizeof(float));
    for (int64_t n = 0; n < N; ++n)
        for (int64_t ky = 0; ky < kH; ++ky)
            memcpy(ker + n * ld + ky * kW * dp, filters + n * gap + ky * kwp * dp,
                   (size_t)(kW * dp) * sizeof(float));
}

/* ------------------------------------------------------------------------
 * im2col convolution = pack, then the "equivalent GEMM".
 * de::cuda::Conv2_MK_im2col, conv2_mk_im2col.h:278-306; zero-border driver
 * :167-274, valid driver :57-162.  The result buffer is [M][ceil4(N)] and is
 * copied flat into the destination tensor (:266), whose padded HWC layout it
 * equals: wpitch_dst = eq_w, dpitch_dst = ceil4(N).  Padding pixels
 * x in [out_w, eq_w) therefore hold the convolution evaluated at those
 * positions, and padding channels n in [N, ceil4(N)) hold 0 (zero filter
 * rows).  Cross-correlation (no kernel flip), stride 1.
 * `dst` must hold out_h * eq_w * ceil4(N) floats.
 * ---------------------------------------------------------------------- */
DECXO_API int decxo_conv2_im2col(const float* src, int64_t W, int64_t H, int64_t depth,
                                 const float* filters, int64_t kW, int64_t kH, int64_t N,
                                 int flag, float* dst)
{
    decxo_conv_geom g;
    int rc = decxo_conv_geometry(W, H, depth, kW, kH, flag, &g);
    if (rc) return rc;
    const int64_t Np = ceil4(N);
    float* i2c = (float*)malloc((size_t)(g.M * g.Kp) * sizeof(float));
    float* ker = (float*)malloc((size_t)(Np * g.Kp) * sizeof(float));
    if (!i2c || !ker) { free(i2c); free(ker); return 5; }
    decxo_im2col_pack(src, W, H, depth, kW, kH, flag, i2c);
    decxo_kernel_matrix(filters, kW, kH, depth, N, Np, g.Kp, ker);
    decxo_gemm_fmaf_nt(g.M, Np, g.Kp, i2c, g.Kp, ker, g.Kp, dst, Np);
    free(i2c); free(ker);
    return 0;
}

/* Activations applied after the GEMM / convolution, restating the reference's stand-alone
 * operators: ReLU keeps x when its sign bit is clear and gives 0 otherwise
 * (srcs/nn/operators/ReLU.h:48-75), sigmoid = 1 / (1 + exp(-x)) (sigmoid.h:45-46),
 * tanh = (exp(2x) - 1) / (exp(2x) + 1) (tanh.h:41-42).  The reference uses the GPU's fast
 * __expf; expf here, so the comparison carries __expf's documented error (2 ulp + a term
 * growing with |x|).  act: 1 ReLU, 2 sigmoid, 3 tanh; bias (per column, may be NULL) is added
 * first. */
DECXO_API void decxo_bias_activation(float* x, int64_t rows, int64_t cols, int64_t ld, const float* bias, int act)
{
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) {
            float v = x[r * ld + c] + (bias ? bias[c] : 0.0f);
            if (act == 1) v = v < 0.0f ? 0.0f : v;
            else if (act == 2) v = 1.0f / (1.0f + expf(-v));
            else if (act == 3) { const float e = expf(2.0f * v); v = (e - 1.0f) / (e + 1.0f); }
            x[r * ld + c] = v;
        }
}

/* Normalised error of the parity rule: max|X - R| / (K * max|a| * max|b|). */
DECXO_API double decxo_max_abs_diff(const float* x, const float* r, uint64_t n)
{
    double m = 0.0;
    for (uint64_t i = 0; i < n; ++i) {
        double d = fabs((double)x[i] - (double)r[i]);
        if (d > m || d != d) m = d;
    }
    return m;
}

