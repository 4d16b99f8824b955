/*
 * Memory-bound helper kernels of the decxb library (sm_100a):
 *   - seeded synthetic data,
 *   - the TF32 hi/lo operand split (with and without transposition) that feeds the
 *     3xTF32 tensor-core GEMM,
 *   - the filter bank -> [N][Kp] matrix gather of the convolution
 *     (what the reference does with one cudaMemcpy2DAsync per filter,
 *      srcs/convolution/CUDA/im2col/conv2_mk_im2col.h:226-231).
 * All of them stream their operands once with 128-bit accesses where alignment allows.
 */
#include "common.h"

#include <cuda_bf16.h>

/* ------------------------------------------------------------------------------------ */
__device__ __forceinline__ uint32_t fmix32(uint32_t h)
{
    h ^= h >> 16; h *= 0x85EBCA6Bu;
    h ^= h >> 13; h *= 0xC2B2AE35u;
    h ^= h >> 16;
    return h;
}

__device__ __forceinline__ float uniform_pm1(uint32_t seed, uint64_t idx)
{
    uint32_t hi = fmix32((uint32_t)(idx >> 32) + seed * 0x85EBCA77u + 0x165667B1u);
    uint32_t u = fmix32(((uint32_t)idx * 0x9E3779B1u) ^ hi);
    return __fsub_rn(__fmul_rn((float)(u >> 8), 1.0f / 8388608.0f), 1.0f);
}

/* Programmatic dependent launch: lets the next kernel in the stream (the GEMM, launched with the
 * matching attribute) be scheduled while this grid drains; that kernel still waits for this
 * grid's completion (griddepcontrol.wait) before it touches memory.  A no-op otherwise. */
__device__ __forceinline__ void allow_dependent_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__global__ void __launch_bounds__(256)
decxb_fill_uniform_kernel(float* __restrict__ dst, uint64_t rows, uint64_t cols, uint64_t pitch,
                          uint32_t seed, uint64_t first_index, const decxb_bounds bnd)
{
    const uint64_t total = rows * pitch;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / pitch, c = i - r * pitch;
        if (DECXB_OK_OUT0(bnd, dst + i, 4)) dst[i] = c < cols ? uniform_pm1(seed, first_index + r * cols + c) : 0.0f;
    }
}

extern "C" int decxb_fill_uniform_f32(decxb_ctx* ctx, float* dptr, uint64_t rows, uint64_t cols, uint64_t pitch,
                                      uint32_t seed, uint64_t first_index, void* stream)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (!dptr || pitch < cols) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "fill_uniform");
    if (rows == 0 || pitch == 0) return DECXB_OK;
    cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
    const uint64_t total = rows * pitch;
    int blocks = (int)((total + 255) / 256 < (uint64_t)ctx->sm_count * 16 ? (total + 255) / 256 : (uint64_t)ctx->sm_count * 16);
    {
        decxb_launch_scope scope(ctx, s, DECXB_K_FILL);
        const decxb_bounds bnd = {ctx->d_status, {}, decxb_make_extent(dptr, (size_t)total * 4), {}, DECXB_BK_FILL};
        decxb_fill_uniform_kernel<<<blocks, 256, 0, s>>>(dptr, rows, cols, pitch, seed, first_index, bnd);
    }
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    return DECXB_OK;
}

/* ------------------------------------------------------------------------------------
 * TF32 split.  hi = round-to-nearest TF32 of a (low 13 mantissa bits zero), lo = TF32 of
 * the exact remainder a - hi.  Both are exactly representable in TF32, so whatever the
 * tensor core does with the low bits of its inputs cannot matter.
 * ---------------------------------------------------------------------------------- */
__device__ __forceinline__ float tf32_rna(float x)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

__device__ __forceinline__ void split1(float a, float& hi, float& lo)
{
    hi = tf32_rna(a);
    lo = tf32_rna(__fsub_rn(a, hi));
}

/* in[rows][ld_in] -> hi/lo[rows_out][ld_out]; columns >= cols and rows >= rows are written
 * as zero.  One thread per 4 output columns. */
struct SplitRowsArgs {
    const float* in; int64_t rows, cols, ld_in;
    float *hi, *lo; int64_t ld_out, rows_out;
    int in_vec_ok; int64_t nbatch, in_batch_stride; int raw;
    decxb_bounds bnd;
};

/* The work of block `bid` of `nblocks` blocks of 256 threads. */
__device__ __forceinline__ void split_rows_body(const SplitRowsArgs& a, int64_t bid, int64_t nblocks)
{
    /* nbatch matrices: matrix b reads rows [0, rows) at in + b*in_batch_stride and writes rows
     * [b*rows_out, (b+1)*rows_out) of the stacked output (rows beyond `rows` are zero) */
    const int64_t q_per_row = a.ld_out >> 2;
    const int64_t total = a.nbatch * a.rows_out * q_per_row;
    for (int64_t i = bid * blockDim.x + threadIdx.x; i < total; i += nblocks * blockDim.x) {
        const int64_t r_all = i / q_per_row, c = (i - r_all * q_per_row) << 2;
        const int64_t b = a.nbatch > 1 ? r_all / a.rows_out : 0, r = r_all - b * a.rows_out;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < a.rows) {
            const float* p = a.in + b * a.in_batch_stride + r * a.ld_in + c;
            if (a.in_vec_ok && c + 3 < a.cols) {
                if (DECXB_OK_IN(a.bnd, p, 16)) {
                    const float4 t = __ldg(reinterpret_cast<const float4*>(p));
                    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) if (c + j < a.cols && DECXB_OK_IN(a.bnd, p + j, 4)) v[j] = __ldg(p + j);
            }
        }
        float4 h, l;
        if (a.raw) { h = make_float4(v[0], v[1], v[2], v[3]); l = h; }
        else { split1(v[0], h.x, l.x); split1(v[1], h.y, l.y); split1(v[2], h.z, l.z); split1(v[3], h.w, l.w); }
        if (DECXB_OK_OUT0(a.bnd, a.hi + r_all * a.ld_out + c, 16)) *reinterpret_cast<float4*>(a.hi + r_all * a.ld_out + c) = h;
        if (a.lo && !a.raw && DECXB_OK_OUT1(a.bnd, a.lo + r_all * a.ld_out + c, 16)) *reinterpret_cast<float4*>(a.lo + r_all * a.ld_out + c) = l;
    }
}

__global__ void __launch_bounds__(256)
decxb_split_rows_kernel(const SplitRowsArgs a)
{
    allow_dependent_launch();
    split_rows_body(a, blockIdx.x, gridDim.x);
}

static decxb_bounds split_rows_bounds(decxb_ctx* ctx, const float* in, int64_t rows, int64_t cols, int64_t ld_in, float* hi, float* lo,
                                      int64_t ld_out, int64_t rows_out, int64_t nbatch, int64_t in_batch_stride)
{
    const size_t in_elems = rows > 0 ? (size_t)((nbatch - 1) * in_batch_stride + (rows - 1) * ld_in + cols) : 0;
    const size_t out_elems = (size_t)(nbatch * rows_out * ld_out);
    return decxb_bounds{ctx->d_status, decxb_make_extent(in, in_elems * 4), decxb_make_extent(hi, out_elems * 4),
                        decxb_make_extent(lo, out_elems * 4), DECXB_BK_SPLIT_ROWS};
}

int decxb_launch_split_rows(decxb_ctx* ctx, const float* in, int64_t rows, int64_t cols, int64_t ld_in,
                            float* hi, float* lo, int64_t ld_out, int64_t rows_out, cudaStream_t s,
                            int64_t nbatch, int64_t in_batch_stride, int raw)
{
    if (ld_out % 4 || ld_out < cols || rows_out < rows) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "split_rows pitch");
    if (nbatch < 1) nbatch = 1;
    const int64_t total = nbatch * rows_out * (ld_out / 4);
    if (total == 0) return DECXB_OK;
    const int vec_ok = ((uintptr_t)in % 16 == 0) && (ld_in % 4 == 0) && (in_batch_stride % 4 == 0);
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)ctx->sm_count * 32) blocks = (int64_t)ctx->sm_count * 32;
    {
        decxb_launch_scope scope(ctx, s, DECXB_K_SPLIT);
        const SplitRowsArgs a = {in, rows, cols, ld_in, hi, lo, ld_out, rows_out, vec_ok, nbatch, in_batch_stride, raw,
                                 split_rows_bounds(ctx, in, rows, cols, ld_in, hi, lo, ld_out, rows_out, nbatch, in_batch_stride)};
        decxb_split_rows_kernel<<<(int)blocks, 256, 0, s>>>(a);
    }
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    return DECXB_OK;
}

/* in[K][ld_in] (K rows, N columns) -> hi/lo[N][ld_out] with K contiguous.  64x64 tiles
 * through shared memory; `raw` stores hi = a unrounded (plain-TF32 mode) and skips lo. */
/* Vectorised form for 16-byte aligned input with a pitch that is a multiple of 4: 128-bit
 * loads along n into the tile, 128-bit stores along k out of it.  A thread of the store phase
 * owns 4 consecutive k of one n, so a 16-thread group writes one 256-byte run of an output
 * row.  (The tile pitch of 65 words keeps the column reads at most 2-way bank conflicted.) */
struct SplitTransposeArgs {
    const float* in; int64_t K, N, ld_in;
    float *hi, *lo; int64_t ld_out; int raw;
    int64_t tiles_n, nbatch, in_batch_stride, out_batch_rows;
    decxb_bounds bnd;
};

__device__ __forceinline__ void split_transpose_vec_body(const SplitTransposeArgs& a, float (*tile)[65], int64_t bid, int64_t nblocks)
{
    const int tid = threadIdx.x;
    const int64_t tiles_k = (a.ld_out + 63) / 64;
    const int64_t n_tiles = tiles_k * a.tiles_n;
    for (int64_t tt = bid; tt < n_tiles * a.nbatch; tt += nblocks) {
        const int64_t bb = tt / n_tiles, t = tt - bb * n_tiles;
        const float* in = a.in + bb * a.in_batch_stride;
        float* hi = a.hi + bb * a.out_batch_rows * a.ld_out;
        float* lo = a.lo ? a.lo + bb * a.out_batch_rows * a.ld_out : nullptr;
        const int64_t k0 = (t / a.tiles_n) * 64, n0 = (t % a.tiles_n) * 64;
        /* load: 64 k-rows x 16 float4 along n */
#pragma unroll
        for (int i = tid; i < 1024; i += 256) {
            const int kr = i >> 4, n4 = (i & 15) << 2;
            const int64_t k = k0 + kr, n = n0 + n4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k < a.K) {
                const float* p = in + k * a.ld_in + n;
                if (n + 3 < a.N) { if (DECXB_OK_IN(a.bnd, p, 16)) v = __ldg(reinterpret_cast<const float4*>(p)); }
                else {
                    if (n < a.N && DECXB_OK_IN(a.bnd, p, 4)) v.x = __ldg(p);
                    if (n + 1 < a.N && DECXB_OK_IN(a.bnd, p + 1, 4)) v.y = __ldg(p + 1);
                    if (n + 2 < a.N && DECXB_OK_IN(a.bnd, p + 2, 4)) v.z = __ldg(p + 2);
                }
            }
            tile[kr][n4] = v.x; tile[kr][n4 + 1] = v.y; tile[kr][n4 + 2] = v.z; tile[kr][n4 + 3] = v.w;
        }
        __syncthreads();
        /* store: 64 n-rows x 16 float4 along k */
#pragma unroll
        for (int i = tid; i < 1024; i += 256) {
            const int nr = i >> 4, k4 = (i & 15) << 2;
            const int64_t n = n0 + nr, k = k0 + k4;
            if (n < a.N && k < a.ld_out) {
                const float a0 = tile[k4][nr], a1 = tile[k4 + 1][nr], a2 = tile[k4 + 2][nr], a3 = tile[k4 + 3][nr];
                float4 h, l;
                if (a.raw) { h = make_float4(a0, a1, a2, a3); }
                else { split1(a0, h.x, l.x); split1(a1, h.y, l.y); split1(a2, h.z, l.z); split1(a3, h.w, l.w); }
                if (DECXB_OK_OUT0(a.bnd, hi + n * a.ld_out + k, 16)) *reinterpret_cast<float4*>(hi + n * a.ld_out + k) = h;
                if (!a.raw && DECXB_OK_OUT1(a.bnd, lo + n * a.ld_out + k, 16)) *reinterpret_cast<float4*>(lo + n * a.ld_out + k) = l;
            }
        }
        __syncthreads();
    }
}

/* The same for inputs that do not allow 128-bit accesses: one word per thread and step. */
__global__ void __launch_bounds__(256)
decxb_split_transpose_kernel(const SplitTransposeArgs a)
{
    __shared__ float tile[64][65];
    allow_dependent_launch();
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;   /* 64 x 4 */
    const int64_t tiles_k = (a.ld_out + 63) / 64;
    const int64_t n_tiles = tiles_k * a.tiles_n;
    for (int64_t tt = blockIdx.x; tt < n_tiles * a.nbatch; tt += gridDim.x) {
        const int64_t bb = tt / n_tiles, t = tt - bb * n_tiles;
        const float* in = a.in + bb * a.in_batch_stride;
        float* hi = a.hi + bb * a.out_batch_rows * a.ld_out;
        float* lo = a.lo ? a.lo + bb * a.out_batch_rows * a.ld_out : nullptr;
        const int64_t k0 = (t / a.tiles_n) * 64, n0 = (t % a.tiles_n) * 64;
#pragma unroll 4
        for (int j = ty; j < 64; j += 4) {
            const int64_t k = k0 + j, n = n0 + tx;
            tile[j][tx] = (k < a.K && n < a.N && DECXB_OK_IN(a.bnd, in + k * a.ld_in + n, 4)) ? __ldg(in + k * a.ld_in + n) : 0.0f;
        }
        __syncthreads();
#pragma unroll 4
        for (int j = ty; j < 64; j += 4) {
            const int64_t n = n0 + j, k = k0 + tx;
            if (n < a.N && k < a.ld_out) {
                const float v = tile[tx][j];
                if (a.raw) {
                    if (DECXB_OK_OUT0(a.bnd, hi + n * a.ld_out + k, 4)) hi[n * a.ld_out + k] = v;
                } else {
                    float h, l; split1(v, h, l);
                    if (DECXB_OK_OUT0(a.bnd, hi + n * a.ld_out + k, 4)) hi[n * a.ld_out + k] = h;
                    if (DECXB_OK_OUT1(a.bnd, lo + n * a.ld_out + k, 4)) lo[n * a.ld_out + k] = l;
                }
            }
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256)
decxb_split_transpose_vec_kernel(const SplitTransposeArgs a)
{
    __shared__ float tile[64][65];
    allow_dependent_launch();
    split_transpose_vec_body(a, tile, blockIdx.x, gridDim.x);
}

/* Both operands of a product in ONE grid: the first `blocks_rows` blocks split A row-wise, the rest
 * split and transpose B.  A small product is otherwise three launches, two of which only write the
 * hi/lo copies and each of which fills a fraction of the GPU. */
__global__ void __launch_bounds__(256)
decxb_split_ab_kernel(const SplitRowsArgs ra, const SplitTransposeArgs ta, int blocks_rows)
{
    __shared__ float tile[64][65];
    allow_dependent_launch();
    if ((int)blockIdx.x < blocks_rows) split_rows_body(ra, blockIdx.x, blocks_rows);
    else split_transpose_vec_body(ta, tile, (int64_t)blockIdx.x - blocks_rows, (int64_t)gridDim.x - blocks_rows);
}

static decxb_bounds split_transpose_bounds(decxb_ctx* ctx, const float* in, int64_t K, int64_t N, int64_t ld_in, float* hi, float* lo,
                                           int64_t ld_out, int64_t nbatch, int64_t in_batch_stride, int64_t out_batch_rows)
{
    const size_t in_elems = (size_t)((nbatch - 1) * in_batch_stride + (K - 1) * ld_in + N);
    const size_t out_elems = (size_t)(((nbatch - 1) * out_batch_rows + N) * ld_out);
    return decxb_bounds{ctx->d_status, decxb_make_extent(in, in_elems * 4), decxb_make_extent(hi, out_elems * 4),
                        decxb_make_extent(lo, out_elems * 4), DECXB_BK_SPLIT_TRANSPOSE};
}

bool decxb_split_ab_possible(const float* B, int64_t ldb, const float* b_hi, const float* b_lo)
{
    return ((uintptr_t)B % 16 == 0) && (ldb % 4 == 0) && ((uintptr_t)b_hi % 16 == 0) && ((uintptr_t)b_lo % 16 == 0);
}

int decxb_launch_split_ab(decxb_ctx* ctx, const float* A, int64_t M, int64_t K, int64_t lda, float* a_hi, float* a_lo,
                          const float* B, int64_t N, int64_t ldb, float* b_hi, float* b_lo, int64_t ld_out, cudaStream_t s)
{
    if (ld_out % 4 || ld_out < K) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "split pitch");
    const int64_t total_rows = M * (ld_out / 4);
    const int64_t tiles_n = (N + 63) / 64, tiles_k = (ld_out + 63) / 64;
    int64_t blocks_rows = (total_rows + 255) / 256, blocks_t = tiles_n * tiles_k;
    const int64_t cap = (int64_t)ctx->sm_count * 16;
    if (blocks_rows > cap) blocks_rows = cap;
    if (blocks_t > cap) blocks_t = cap;
    const int vec_ok = ((uintptr_t)A % 16 == 0) && (lda % 4 == 0);
    const SplitRowsArgs ra = {A, M, K, lda, a_hi, a_lo, ld_out, M, vec_ok, 1, 0, 0,
                              split_rows_bounds(ctx, A, M, K, lda, a_hi, a_lo, ld_out, M, 1, 0)};
    const SplitTransposeArgs ta = {B, K, N, ldb, b_hi, b_lo, ld_out, 0, tiles_n, 1, 0, 0,
                                   split_transpose_bounds(ctx, B, K, N, ldb, b_hi, b_lo, ld_out, 1, 0, 0)};
    {
        decxb_launch_scope scope(ctx, s, DECXB_K_SPLIT);
        decxb_split_ab_kernel<<<(int)(blocks_rows + blocks_t), 256, 0, s>>>(ra, ta, (int)blocks_rows);
    }
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    return DECXB_OK;
}

int decxb_launch_split_transpose(decxb_ctx* ctx, const float* in, int64_t K, int64_t N, int64_t ld_in,
                                 float* hi, float* lo, int64_t ld_out, int raw, cudaStream_t s,
                                 int64_t nbatch, int64_t in_batch_stride, int64_t out_batch_rows)
{
    if (ld_out % 4 || ld_out < K) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "split_transpose pitch");
    if (nbatch < 1) nbatch = 1;
    const int64_t tiles_n = (N + 63) / 64, tiles_k = (ld_out + 63) / 64;
    int64_t blocks = tiles_n * tiles_k * nbatch;
    if (blocks == 0) return DECXB_OK;
    if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
    const SplitTransposeArgs a = {in, K, N, ld_in, hi, lo, ld_out, raw, tiles_n, nbatch, in_batch_stride, out_batch_rows,
                                  split_transpose_bounds(ctx, in, K, N, ld_in, hi, lo, ld_out, nbatch, in_batch_stride, out_batch_rows)};
    if (((uintptr_t)in % 16 == 0) && (ld_in % 4 == 0) && (in_batch_stride % 4 == 0) && ((uintptr_t)hi % 16 == 0) &&
        (raw || (uintptr_t)lo % 16 == 0)) {
        decxb_launch_scope scope(ctx, s, DECXB_K_SPLIT);
        decxb_split_transpose_vec_kernel<<<(int)blocks, 256, 0, s>>>(a);
        DECXB_CUDA_TRY(ctx, cudaGetLastError());
        return DECXB_OK;
    }
    {
        decxb_launch_scope scope(ctx, s, DECXB_K_SPLIT);
        decxb_split_transpose_kernel<<<(int)blocks, 256, 0, s>>>(a);
    }
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    return DECXB_OK;
}

/* Filter bank -> matrix.  Row n, column (ky*kW + kx)*cp + c  <-  filters[n][ky][kx][c]
 * (TensorArray layout [N][kH][ceil4(kW)][dp]); cp = dp for the explicit path, cp = ceil32(dp)
 * for the implicit path (one 32-channel-padded block row per tap).  Rows n >= N, channels
 * c >= dp and columns >= kW*kH*cp are zero. */
__global__ void __launch_bounds__(256)
decxb_filter_matrix_kernel(const float* __restrict__ filters, int kW, int kH, int dp, int cp, int64_t N,
                           float* __restrict__ hi, float* __restrict__ lo, int64_t rows_out, int64_t ld_out, int raw,
                           const decxb_bounds bnd)
{
    allow_dependent_launch();
    const int64_t Kp = (int64_t)kW * kH * cp;
    const int64_t kwp = (kW + 3) / 4 * 4;
    const int64_t gap = (int64_t)dp * kwp * kH;
    const int64_t total = rows_out * ld_out;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / ld_out, k = i - n * ld_out;
        float a = 0.0f;
        if (n < N && k < Kp) {
            const int64_t tap = k / cp, c = k - tap * cp;
            const int64_t ky = tap / kW, kx = tap - ky * kW;
            if (c < dp && DECXB_OK_IN(bnd, filters + n * gap + (ky * kwp + kx) * dp + c, 4)) a = __ldg(filters + n * gap + (ky * kwp + kx) * dp + c);
        }
        if (raw) { if (DECXB_OK_OUT0(bnd, hi + i, 4)) hi[i] = a; }
        else {
            float h, l; split1(a, h, l);
            if (DECXB_OK_OUT0(bnd, hi + i, 4)) hi[i] = h;
            if (DECXB_OK_OUT1(bnd, lo + i, 4)) lo[i] = l;
        }
    }
}

int decxb_launch_filter_matrix(decxb_ctx* ctx, const float* filters, int64_t kW, int64_t kH, int64_t depth,
                               int64_t N, float* hi, float* lo, int64_t rows_out, int64_t ld_out, int raw,
                               cudaStream_t s, int64_t chan_pitch)
{
    const int64_t dp = decxb_ceil_to(depth, 4);
    const int64_t cp = chan_pitch > 0 ? chan_pitch : dp;
    const int64_t total = rows_out * ld_out;
    if (total == 0) return DECXB_OK;
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
    {
        decxb_launch_scope scope(ctx, s, DECXB_K_SPLIT);
        const size_t bank = (size_t)N * (size_t)(dp * decxb_ceil_to(kW, 4) * kH) * 4;
        const decxb_bounds bnd = {ctx->d_status, decxb_make_extent(filters, bank), decxb_make_extent(hi, (size_t)total * 4),
                                  decxb_make_extent(lo, (size_t)total * 4), DECXB_BK_FILTER_MATRIX};
        decxb_filter_matrix_kernel<<<(int)blocks, 256, 0, s>>>(filters, (int)kW, (int)kH, (int)dp, (int)cp, N, hi, lo, rows_out, ld_out, raw, bnd);
    }
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    return DECXB_OK;
}

/* fp16 transpose for the fp16 GEMM's B operand: in[K][ld_in] -> out[N][ld_out], 64x64 tiles of
 * 16-bit words through shared memory; output columns k >= K (up to ld_out) are zero. */
__global__ void __launch_bounds__(256)
decxb_transpose_f16_kernel(const unsigned short* __restrict__ in, int64_t K, int64_t N, int64_t ld_in,
                           unsigned short* __restrict__ out, int64_t ld_out, int64_t tiles_n, const decxb_bounds bnd)
{
    __shared__ unsigned short tile[64][66];
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    const int64_t tiles_k = (ld_out + 63) / 64;
    const int64_t n_tiles = tiles_k * tiles_n;
    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const int64_t k0 = (t / tiles_n) * 64, n0 = (t % tiles_n) * 64;
#pragma unroll 4
        for (int j = ty; j < 64; j += 4) {
            const int64_t k = k0 + j, n = n0 + tx;
            tile[j][tx] = (k < K && n < N && DECXB_OK_IN(bnd, in + k * ld_in + n, 2)) ? in[k * ld_in + n] : (unsigned short)0;
        }
        __syncthreads();
#pragma unroll 4
        for (int j = ty; j < 64; j += 4) {
            const int64_t n = n0 + j, k = k0 + tx;
            if (n < N && k < ld_out && DECXB_OK_OUT0(bnd, out + n * ld_out + k, 2)) out[n * ld_out + k] = tile[tx][j];
        }
        __syncthreads();
    }
}

int decxb_launch_transpose_f16(decxb_ctx* ctx, const void* in, int64_t K, int64_t N, int64_t ld_in,
                               void* out, int64_t ld_out, cudaStream_t s)
{
    if (ld_out < K) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "transpose_f16 pitch");
    const int64_t tiles_n = (N + 63) / 64, tiles_k = (ld_out + 63) / 64;
    int64_t blocks = tiles_n * tiles_k;
    if (blocks == 0) return DECXB_OK;
    if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
    {
        decxb_launch_scope scope(ctx, s, DECXB_K_SPLIT);
        const decxb_bounds bnd = {ctx->d_status, decxb_make_extent(in, (size_t)((K - 1) * ld_in + N) * 2),
                                  decxb_make_extent(out, (size_t)(N * ld_out) * 2), {}, DECXB_BK_TRANSPOSE_F16};
        decxb_transpose_f16_kernel<<<(int)blocks, 256, 0, s>>>(static_cast<const unsigned short*>(in), K, N, ld_in,
                                                               static_cast<unsigned short*>(out), ld_out, tiles_n, bnd);
    }
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    return DECXB_OK;
}

/* ------------------------------------------------------------------------------------
 * Operands of the TF32 + 2 x bf16 mode: hi = tf32(a) as above, and two bf16 arrays for the cross
 * products, lo16 = bf16(a - hi) and a16 = bf16(a) (round to nearest even).  One thread per 8
 * consecutive k, so that the bf16 stores are 16 bytes.  Row pitches: hi `ld_hi` floats (a multiple of
 * 4), bf16 arrays `ld16` values (a multiple of 8); pad columns are written as zero.
 * ---------------------------------------------------------------------------------- */
__device__ __forceinline__ uint32_t pack_bf16x2(float x, float y)
{
    const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ void split8_store(const float* v, float* hi_row, unsigned short* lo16_row, unsigned short* a16_row,
                                             int64_t k, int64_t ld_hi)
{
    float h[8], l[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { h[j] = tf32_rna(v[j]); l[j] = __fsub_rn(v[j], h[j]); }
    *reinterpret_cast<float4*>(hi_row + k) = make_float4(h[0], h[1], h[2], h[3]);
    if (k + 4 < ld_hi) *reinterpret_cast<float4*>(hi_row + k + 4) = make_float4(h[4], h[5], h[6], h[7]);
    *reinterpret_cast<uint4*>(lo16_row + k) = make_uint4(pack_bf16x2(l[0], l[1]), pack_bf16x2(l[2], l[3]), pack_bf16x2(l[4], l[5]), pack_bf16x2(l[6], l[7]));
    *reinterpret_cast<uint4*>(a16_row + k) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
}

__global__ void __launch_bounds__(256)
decxb_split_rows_bf16_kernel(const float* __restrict__ in, int64_t rows, int64_t cols, int64_t ld_in,
                             float* __restrict__ hi, unsigned short* __restrict__ lo16, unsigned short* __restrict__ a16,
                             int64_t ld_hi, int64_t ld16, int in_vec_ok)
{
    allow_dependent_launch();
    const int64_t o_per_row = ld16 >> 3;
    const int64_t total = rows * o_per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / o_per_row, k = (i - r * o_per_row) << 3;
        float v[8];
        if (in_vec_ok && k + 7 < cols) {
            const float4 t0 = __ldg(reinterpret_cast<const float4*>(in + r * ld_in + k));
            const float4 t1 = __ldg(reinterpret_cast<const float4*>(in + r * ld_in + k + 4));
            v[0] = t0.x; v[1] = t0.y; v[2] = t0.z; v[3] = t0.w; v[4] = t1.x; v[5] = t1.y; v[6] = t1.z; v[7] = t1.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (k + j < cols) ? __ldg(in + r * ld_in + k + j) : 0.0f;
        }
        split8_store(v, hi + r * ld_hi, lo16 + r * ld16, a16 + r * ld16, k, ld_hi);
    }
}

/* in[K][ld_in] (K rows, N columns) -> the same three arrays of the transposed operand, [N][...] with K contiguous. */
__global__ void __launch_bounds__(256)
decxb_split_transpose_bf16_kernel(const float* __restrict__ in, int64_t K, int64_t N, int64_t ld_in,
                                  float* __restrict__ hi, unsigned short* __restrict__ lo16, unsigned short* __restrict__ b16,
                                  int64_t ld_hi, int64_t ld16, int64_t tiles_n)
{
    __shared__ float tile[64][65];
    allow_dependent_launch();
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    const int64_t tiles_k = (ld16 + 63) / 64;
    for (int64_t t = blockIdx.x; t < tiles_k * tiles_n; t += gridDim.x) {
        const int64_t k0 = (t / tiles_n) * 64, n0 = (t % tiles_n) * 64;
#pragma unroll 4
        for (int j = ty; j < 64; j += 4) {
            const int64_t k = k0 + j, n = n0 + tx;
            tile[j][tx] = (k < K && n < N) ? __ldg(in + k * ld_in + n) : 0.0f;
        }
        __syncthreads();
        /* 64 n-rows x 8 runs of 8 consecutive k */
        for (int i = threadIdx.x; i < 512; i += 256) {
            const int nr = i >> 3, k8 = (i & 7) << 3;
            const int64_t n = n0 + nr, k = k0 + k8;
            if (n < N && k < ld16) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = tile[k8 + j][nr];
                split8_store(v, hi + n * ld_hi, lo16 + n * ld16, b16 + n * ld16, k, ld_hi);
            }
        }
        __syncthreads();
    }
}

int decxb_launch_split_rows_bf16(decxb_ctx* ctx, const float* in, int64_t rows, int64_t cols, int64_t ld_in,
                                 float* hi, void* lo16, void* a16, int64_t ld_hi, int64_t ld16, cudaStream_t s)
{
    if (ld16 % 8 || ld16 < cols || ld_hi % 4 || ld_hi < cols || ld_hi > ld16) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "bf16 split pitch");
    const int64_t total = rows * (ld16 / 8);
    if (total == 0) return DECXB_OK;
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)ctx->sm_count * 32) blocks = (int64_t)ctx->sm_count * 32;
    {
        decxb_launch_scope scope(ctx, s, DECXB_K_SPLIT);
        const int vec_ok = ((uintptr_t)in % 16 == 0) && (ld_in % 4 == 0);
        decxb_split_rows_bf16_kernel<<<(int)blocks, 256, 0, s>>>(in, rows, cols, ld_in, hi, static_cast<unsigned short*>(lo16),
                                                                 static_cast<unsigned short*>(a16), ld_hi, ld16, vec_ok);
    }
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    return DECXB_OK;
}

int decxb_launch_split_transpose_bf16(decxb_ctx* ctx, const float* in, int64_t K, int64_t N, int64_t ld_in,
                                      float* hi, void* lo16, void* b16, int64_t ld_hi, int64_t ld16, cudaStream_t s)
{
    if (ld16 % 8 || ld16 < K || ld_hi % 4 || ld_hi < K || ld_hi > ld16) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "bf16 split pitch");
    const int64_t tiles_n = (N + 63) / 64, tiles_k = (ld16 + 63) / 64;
    int64_t blocks = tiles_n * tiles_k;
    if (blocks == 0) return DECXB_OK;
    if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
    {
        decxb_launch_scope scope(ctx, s, DECXB_K_SPLIT);
        decxb_split_transpose_bf16_kernel<<<(int)blocks, 256, 0, s>>>(in, K, N, ld_in, hi, static_cast<unsigned short*>(lo16),
                                                                      static_cast<unsigned short*>(b16), ld_hi, ld16, tiles_n);
    }
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    return DECXB_OK;
}

/* Self-test of the debug bounds build: splits a small matrix while the launcher is told that the
 * input array is one row shorter than it is.  The memory IS there (nothing can fault); the check
 * must trip, skip the accesses to that row and leave DECXB_ERR_BOUNDS for the host. */
extern "C" int decxb_selftest_bounds(decxb_ctx* ctx)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (!decxb_bounds_build()) return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "this library was built without DECXB_BOUNDS");
    const int64_t rows = 64, cols = 128;
    float *in = nullptr, *hi = nullptr, *lo = nullptr;
    if ((rc = decxb_malloc(ctx, rows * cols * 4, (void**)&in)) || (rc = decxb_malloc(ctx, rows * cols * 4, (void**)&hi)) ||
        (rc = decxb_malloc(ctx, rows * cols * 4, (void**)&lo))) return rc;
    cudaStream_t s = ctx->stream;
    DECXB_CUDA_TRY(ctx, cudaMemsetAsync(in, 0, rows * cols * 4, s));
    {
        SplitRowsArgs a = {in, rows, cols, cols, hi, lo, cols, rows, 1, 1, 0, 0,
                           split_rows_bounds(ctx, in, rows - 1, cols, cols, hi, lo, cols, rows, 1, 0)};   /* declared one row short */
        decxb_launch_scope scope(ctx, s, DECXB_K_SPLIT);
        decxb_split_rows_kernel<<<32, 256, 0, s>>>(a);
    }
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    DECXB_CUDA_TRY(ctx, cudaStreamSynchronize(s));
    rc = decxb_check_dev_status(ctx);
    decxb_free(ctx, in); decxb_free(ctx, hi); decxb_free(ctx, lo);
    return rc;
}
