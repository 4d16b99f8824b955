/*
 * decxb.h -- C ABI of the B200 (sm_100a) implementation of DECX's dense-contraction
 * hot path: the fp32 GEMM and the im2col convolution.
 *
 * Plain pointers and sizes only; every function returns a decxb_status.  This is the
 * boundary a DECX build binds instead of launching its own kernels and using its own
 * device pool on this path.  Each entry names the reference interface it replaces
 * (paths relative to the reference project root).
 *
 * Conventions
 *  - Matrices are row-major fp32 with a leading dimension in ELEMENTS (DECX "pitch",
 *    srcs/classes/Matrix.h:253-267).  DECX names sizes (width, height); here
 *    M = height of A, K = width of A = height of B, N = width of B.
 *  - Tensors are DECX's padded HWC layout (srcs/classes/Tensor.h:162-184, :389-394):
 *    dpitch = ceil4(depth), wpitch = ceil4(width), element (row, col, ch) at
 *    ptr[(row*wpitch + col)*dpitch + ch]; filter banks are TensorArrays
 *    (srcs/classes/TensorArray.h:174-198): filters lie dpitch*wpitch*height floats apart.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the context's own stream).
 *    Device-resident entry points are asynchronous on that stream; host-resident
 *    entry points block until the result is in host memory, as the reference does
 *    (srcs/GEMM/CUDA/large_squares/GEMM.h:122, conv2_mk_im2col.h:268).
 *  - There is no CPU fallback: without a usable sm_100 device every compute entry
 *    fails with DECXB_ERR_NO_DEVICE / DECXB_ERR_ARCH.
 */
#ifndef DECXB_H_
#define DECXB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DECXB_API __attribute__((visibility("default")))

typedef enum decxb_status {
    DECXB_OK               = 0,
    DECXB_ERR_NOT_INIT     = 1,   /* maps to DECX_FAIL_not_init        (srcs/handles/decx_handles.h:10) */
    DECXB_ERR_DIM_MISMATCH = 3,   /* maps to DECX_FAIL_DimsNotMatching (:14)                            */
    DECXB_ERR_BAD_KERNEL   = 5,   /* maps to DECX_FAIL_ConvBadKernel   (:17)                            */
    DECXB_ERR_BAD_FLAG     = 11,  /* maps to DECX_FAIL_ErrorFlag       (:27)                            */
    DECXB_ERR_BAD_PARAM    = 13,  /* maps to DECX_FAIL_ErrorParams     (:31)                            */
    DECXB_ERR_ALLOC        = 16,  /* maps to DECX_FAIL_ALLOCATION      (:37)                            */
    DECXB_ERR_CUDA         = 100, /* a CUDA runtime/driver call failed; see decxb_last_error            */
    DECXB_ERR_NO_DEVICE    = 101,
    DECXB_ERR_ARCH         = 102, /* device is not compute capability 10.x                              */
    DECXB_ERR_TIMEOUT      = 103, /* a bounded device-side wait expired; the context stays usable       */
    DECXB_ERR_TOO_LARGE    = 104, /* request exceeds a documented fixed limit                           */
    DECXB_ERR_COMM         = 105, /* the communication library failed or could not be loaded            */
    DECXB_ERR_BOUNDS       = 106  /* debug bounds build only: an access outside its array was caught    */
} decxb_status;

/* Precision of the tensor-core GEMM.  3xTF32 (default) splits every fp32 operand into a
 * TF32 "hi" part and a TF32 "lo" remainder and accumulates lo*hi + hi*lo + hi*hi in fp32,
 * which keeps max|C-Cref| / (K max|a| max|b|) below 1e-6 against the reference's fp32 FMA
 * chain (srcs/GEMM/CUDA/large_squares/GEMM.cuh:53-94).  Plain TF32 is opt-in. */
typedef enum decxb_gemm_mode {
    DECXB_GEMM_3XTF32 = 0,
    DECXB_GEMM_1XTF32 = 1,
    /* 3xTF32 with the K dimension accumulated in chunks of 128: every chunk starts a fresh
     * tensor-core accumulator, and the epilogue warps add the finished chunks to a running sum in
     * registers with IEEE fp32 adds (round to nearest) while the tensor core works on the next
     * chunk, all inside the one kernel.  The tensor core's accumulator rounds toward zero, which
     * biases long sums of same-sign terms (the reference test program's all-positive matrices
     * reach 2.9e-6 of K max|a| max|b| at K = 2048); chunking brings such inputs to 3.3e-7.
     * Accepted by every fp32 GEMM and convolution entry point. */
    DECXB_GEMM_3XTF32_STRICT = 2,
    /* Opt-in, beyond the reference's arithmetic and beyond 3xTF32: the hi*hi product in TF32 and the
     * two cross products a_lo*b and a*b_lo in bf16 on the tensor cores (bf16 runs at twice the TF32
     * rate, so a k-block costs 8 MMA slots instead of 12), K accumulated in chunks like the strict
     * mode.  The cross terms carry a relative error of about 2^-20 per product instead of 2^-22;
     * rounding is to nearest, so the errors do not add up in one direction: on the seeded inputs the
     * result stays within the 1e-6 bar with a wide margin (see the tests), adversarial inputs can
     * come to about 2e-6.  Accepted by decxb_gemm_f32 and decxb_gemm_f32_act only. */
    DECXB_GEMM_TF32_2XBF16 = 3
} decxb_gemm_mode;

/* Tile configuration of the GEMM kernel (0 = choose from the shape). */
typedef enum decxb_gemm_tile {
    DECXB_TILE_AUTO        = 0,
    DECXB_TILE_1CTA_128x128 = 1,
    DECXB_TILE_2CTA_256x256 = 2,  /* CTA pair, tcgen05 cta_group::2 */
    DECXB_TILE_1CTA_128x256 = 3,
    DECXB_TILE_1CTA_128x64  = 4
} decxb_gemm_tile;

/* Border handling of the convolution: values of decx::conv_property
 * (srcs/convolution/CUDA/conv_flags.h:16-20). */
typedef enum decxb_conv_flag {
    DECXB_CONV_NO_COMPENSATE   = 0,   /* "valid": output (W-2*(kW/2)) x (H-2*(kH/2)) */
    DECXB_CONV_ZERO_COMPENSATE = 1    /* zero border: output W x H                      */
} decxb_conv_flag;

/* Activation fused into the GEMM / convolution epilogue, with the formulas of the reference's
 * stand-alone operators de::nn::ReLU_f, sigmoid_f, tanh_f (srcs/nn/operators/ReLU.h:28,
 * sigmoid.h:25, tanh.h:21). */
typedef enum decxb_activation {
    DECXB_ACT_NONE = 0, DECXB_ACT_RELU = 1, DECXB_ACT_SIGMOID = 2, DECXB_ACT_TANH = 3
} decxb_activation;

/* Convolution algorithm. */
typedef enum decxb_conv_algo {
    DECXB_CONV_EXPLICIT = 0,  /* pack kernel writes the column matrix, then the GEMM (the reference's two steps) */
    DECXB_CONV_IMPLICIT = 1   /* column tiles are built in shared memory; the column matrix is never written    */
} decxb_conv_algo;

typedef struct decxb_ctx decxb_ctx;

/* ---- context ---------------------------------------------------------------------
 * Replaces de::InitCuda / decx::cuP (srcs/core/configs/config.h:50-78).  One context per
 * device; it owns a stream, the device arena and the status word device-side waits report to. */
DECXB_API int decxb_init(int device, decxb_ctx** out);
DECXB_API int decxb_destroy(decxb_ctx* ctx);
DECXB_API const char* decxb_status_string(int status);
/* Text of the last failure on this context (never NULL; valid until the next call). */
DECXB_API const char* decxb_last_error(decxb_ctx* ctx);
DECXB_API int decxb_device(decxb_ctx* ctx);
DECXB_API void* decxb_stream(decxb_ctx* ctx);
DECXB_API int decxb_synchronize(decxb_ctx* ctx);
/* Device-side waits give up after this many milliseconds (default 2000). */
DECXB_API int decxb_set_wait_limit_ms(decxb_ctx* ctx, int ms);

/* ---- device arena -----------------------------------------------------------------
 * Replaces decx::alloc::_alloc_D / _dealloc_D and MemPool_D
 * (srcs/core/allocators/allocator.h:83-97, srcs/core/memory_management/MemoryPool_D.h:18-194).
 * 256-byte aligned, size_t-clean (the reference's `1 << n` int shift breaks at 2 GiB,
 * MemoryPool_D.h:129), thread-safe; freed blocks are cached for reuse. */
DECXB_API int decxb_malloc(decxb_ctx* ctx, size_t bytes, void** dptr);
/* Does not wait for the device (cudaFree would): the block is handed out again only after the
 * work queued on the CONTEXT's stream at the time of the free has finished.  A block used by
 * work on a caller-supplied stream must be freed only after that stream has been synchronised. */
DECXB_API int decxb_free(decxb_ctx* ctx, void* dptr);
/* Return every cached block to the driver: de::release_all_tmp
 * (srcs/core/memory_management/Memory_pool.h:28-38). */
DECXB_API int decxb_release_cached(decxb_ctx* ctx);
typedef struct decxb_arena_stats {
    size_t bytes_in_use, bytes_cached, peak_bytes_in_use;
    uint64_t n_driver_allocs, n_reuses;
} decxb_arena_stats;
DECXB_API int decxb_arena_get_stats(decxb_ctx* ctx, decxb_arena_stats* out);

/* Pinned host memory for DATA_STORE_TYPE::Page_Locked containers
 * (srcs/core/allocators/aligned_allocators.h:76, srcs/classes/store_types.h:24-28). */
DECXB_API int decxb_host_alloc(size_t bytes, void** hptr);
DECXB_API int decxb_host_free(void* hptr);

/* Plain copies used by the GPU containers' Load_from_host / Load_to_host
 * (srcs/classes/GPU_Matrix.h:334-354, GPU_Tensor.h:355-371). kind: 1 H2D, 2 D2H, 3 D2D. */
DECXB_API int decxb_memcpy2d(decxb_ctx* ctx, void* dst, size_t dpitch_bytes, const void* src, size_t spitch_bytes,
                             size_t width_bytes, size_t rows, int kind);
DECXB_API int decxb_memset(decxb_ctx* ctx, void* dptr, int value, size_t bytes);

/* ---- seeded synthetic data ---------------------------------------------------------
 * Fills rows x cols (row pitch `pitch` elements, pitch tail zeroed) with uniform [-1,1)
 * values; element (r, c) is a pure function of (seed, first_index + r*cols + c).  No
 * counterpart in the reference (its tests fill from index formulas). */
DECXB_API int decxb_fill_uniform_f32(decxb_ctx* ctx, float* dptr, uint64_t rows, uint64_t cols, uint64_t pitch,
                                     uint32_t seed, uint64_t first_index, void* stream);

/* ---- GEMM -------------------------------------------------------------------------
 * D[M][N] = A[M][K] * B[K][N] (+ C[M][N] when C != NULL), all device-resident.
 * Replaces the kernel selection and launches of de::cuda::GEMM on GPU_Matrix
 * (srcs/GEMM/CUDA/large_squares/GEMM.h:398-454 and, with C, :522-582), i.e. kernels
 * cu_GEMM_fp32_spec / _ABC_spec and the six ragged variants (GEMM.cuh:31-100,206-280;
 * GEMM_nonuniform.cuh:32-693).  Any M, N, K >= 1; no alignment demands beyond fp32. */
DECXB_API int decxb_gemm_f32(decxb_ctx* ctx, int mode, int tile,
                             int64_t M, int64_t N, int64_t K,
                             const float* A, int64_t lda,
                             const float* B, int64_t ldb,
                             const float* C, int64_t ldc,
                             float* D, int64_t ldd, void* stream);

/* D = act(A*B (+C) + bias[column]): decxb_gemm_f32 with the fused epilogue described at
 * decxb_conv2_im2col_f32_act (bias: N floats on the device, or NULL). */
DECXB_API int decxb_gemm_f32_act(decxb_ctx* ctx, int mode, int tile,
                                 int64_t M, int64_t N, int64_t K,
                                 const float* A, int64_t lda, const float* B, int64_t ldb,
                                 const float* C, int64_t ldc, const float* bias, int activation,
                                 float* D, int64_t ldd, void* stream);

/* Same product with B given K-contiguous: Bt[N][K] ("TN"), the orientation of the
 * convolution's filter matrix (cu_conv_eq_mm, srcs/convolution/CUDA/im2col/eq_GEMM.cuh:109-209). */
DECXB_API int decxb_gemm_f32_nt(decxb_ctx* ctx, int mode, int tile,
                                int64_t M, int64_t N, int64_t K,
                                const float* A, int64_t lda,
                                const float* Bt, int64_t ldbt,
                                const float* C, int64_t ldc,
                                float* D, int64_t ldd, void* stream);

/* Host-resident operands: stages A, B (and C) to the device, multiplies, copies D back and
 * blocks until done.  Replaces de::cuda::GEMM on Matrix (GEMM.h:56-131, with C :136-221). */
DECXB_API int decxb_gemm_f32_host(decxb_ctx* ctx, int mode, int tile,
                                  int64_t M, int64_t N, int64_t K,
                                  const float* hA, int64_t lda,
                                  const float* hB, int64_t ldb,
                                  const float* hC, int64_t ldc,
                                  float* hD, int64_t ldd);

/* fp16 product D = A*B (+C): operands, addend and result are IEEE half (passed as void*), the
 * accumulation is fp32 on the tensor cores (tcgen05 kind::f16).  Replaces the fp16 overloads of
 * de::cuda::GEMM (srcs/GEMM/CUDA/large_squares/GEMM.h:33-49, kernels cu_GEMM_fp16_spec /
 * _ABC_spec, GEMM.cuh:119, :297), which accumulate in half with __hfma2
 * (srcs/GEMM/CUDA/GEMM_kernel_def.cuh:100-107): results here are at least as close to the
 * exact product as the reference's.  Leading dimensions in halves. */
DECXB_API int decxb_gemm_f16(decxb_ctx* ctx, int64_t M, int64_t N, int64_t K,
                             const void* A, int64_t lda, const void* B, int64_t ldb,
                             const void* C, int64_t ldc, void* D, int64_t ldd, void* stream);
DECXB_API int decxb_gemm_f16_host(decxb_ctx* ctx, int64_t M, int64_t N, int64_t K,
                                  const void* hA, int64_t lda, const void* hB, int64_t ldb,
                                  const void* hC, int64_t ldc, void* hD, int64_t ldd);

/* Batched product over arrays of equally sized matrices, D[i] = A[i]*B[i] (+C[i]); matrix i of
 * an array starts stride* elements after matrix i-1.  Replaces de::cuda::GEMM3 on MatrixArray
 * (srcs/GEMM/CUDA/large_squares/GEMM3.h:45-114 and, with C, :120-200; its copy/compute
 * pipeline is the macro GEMM3_part, GEMM3_macros.h:140-248).  The host-resident form uploads
 * matrix i while matrix i-1 is multiplied and result i-2 is downloaded, and blocks until done. */
DECXB_API int decxb_gemm_f32_batched(decxb_ctx* ctx, int mode, int tile, int64_t batch, int64_t M, int64_t N, int64_t K,
                                     const float* A, int64_t lda, int64_t strideA,
                                     const float* B, int64_t ldb, int64_t strideB,
                                     const float* C, int64_t ldc, int64_t strideC,
                                     float* D, int64_t ldd, int64_t strideD, void* stream);
DECXB_API int decxb_gemm_f32_batched_host(decxb_ctx* ctx, int mode, int tile, int64_t batch, int64_t M, int64_t N, int64_t K,
                                          const float* hA, int64_t lda, int64_t strideA,
                                          const float* hB, int64_t ldb, int64_t strideB,
                                          const float* hC, int64_t ldc, int64_t strideC,
                                          float* hD, int64_t ldd, int64_t strideD);

/* B prepared once for many products.  In the use this path is made for, B holds weights that
 * stay the same from call to call, while every call of decxb_gemm_f32 splits and transposes it
 * again (a tenth of the time of a large product, a third of a small one).  decxb_gemm_prepare_b
 * does that work once, into arena memory owned by the handle; decxb_gemm_f32_prepared then
 * computes D[M][N] = act(A[M][K] * B (+C) (+bias[column])) with results bit-identical to
 * decxb_gemm_f32 / decxb_gemm_f32_act in the handle's mode; decxb_gemm_release_b gives the memory
 * back (in stream order on `stream`).  The handle is bound to its context; B may be overwritten
 * once decxb_gemm_prepare_b's work on `stream` has run.  No counterpart in the reference, which
 * re-stages both operands on every call (srcs/GEMM/CUDA/large_squares/GEMM.h:398-454). */
typedef struct decxb_prepared_b decxb_prepared_b;
DECXB_API int decxb_gemm_prepare_b(decxb_ctx* ctx, int mode, int64_t K, int64_t N, const float* B, int64_t ldb,
                                   void* stream, decxb_prepared_b** out);
DECXB_API int decxb_gemm_f32_prepared(decxb_ctx* ctx, int tile, int64_t M, const float* A, int64_t lda,
                                      const decxb_prepared_b* B, const float* C, int64_t ldc,
                                      const float* bias, int activation, float* D, int64_t ldd, void* stream);
DECXB_API int decxb_gemm_release_b(decxb_ctx* ctx, decxb_prepared_b* B, void* stream);

/* The 3xTF32 product D = A*B (+C) of decxb_gemm_f32 for callers that must not allocate
 * device memory (this entry has no counterpart in the reference).  Such callers exist: a
 * process in which a framework's caching pool has reserved the whole card, so that a
 * cudaMalloc would fail; a latency-critical loop that cannot take cudaMalloc's implicit
 * device-wide synchronisation.  The regular entry point draws its hi/lo operand scratch
 * from the context's arena; this one needs no context and keeps that scratch in a fixed
 * 64 MiB array inside the library image, which every device that uses this entry holds
 * until the process exits.
 *  - Limit: 2*(M+N)*ceil4(K)*4 bytes (each of the four parts rounded up to 256) must fit in
 *    64 MiB, e.g. 2048 x 2048 x 2048; larger problems return DECXB_ERR_TOO_LARGE and `err`
 *    says how much was asked for.
 *  - It calls no cudaMalloc, cudaFree or other allocating routine.  The first call on a
 *    device resolves the array's device address (cudaGetSymbolAddress) with that device
 *    current; make that first call before any stream capture begins.  The calling thread's
 *    current device is the same after the call as before it.
 *  - Loading device code takes device memory too, and CUDA does it on first use: the first call
 *    on a device loads the module that carries the array (with CUDA_MODULE_LOADING=EAGER every
 *    process that initialises CUDA with this library loaded pays the 64 MiB per device at once),
 *    and the first problem that selects a tile shape not used before loads that kernel.  Warm up
 *    before the other allocator takes the card: one call per device for each shape used later.
 *    After that a call leaves the device's free memory unchanged.
 *  - Calls on the same device take one host lock each; calls on different devices run side
 *    by side.  `stream`, when given, must belong to `device` (DECXB_ERR_BAD_PARAM otherwise).
 *  - All calls share the one array and it keeps the previous call's contents; the entry
 *    rewrites the parts it uses and clears its status word itself.  It blocks until D is
 *    complete.  Calls that would overlap on the GPU (from several threads or streams) race on
 *    the array: issue them one after another.
 *  - A, B, C, D are device pointers; `stream` is a cudaStream_t (NULL = default stream);
 *    `err` (optional, err_len bytes) receives a message when the status is not DECXB_OK.
 *  - Arithmetic: the DECXB_GEMM_3XTF32 mode (the tensor core accumulates over all of K). */
DECXB_API int decxb_gemm_f32_noalloc(int device, int64_t M, int64_t N, int64_t K,
                                     const float* A, int64_t lda, const float* B, int64_t ldb,
                                     const float* C, int64_t ldc, float* D, int64_t ldd,
                                     void* stream, char* err, size_t err_len);

/* ---- im2col convolution --------------------------------------------------------------
 * Geometry shared by the entry points below (conv2_mk_im2col.h:60-93, :170-199). */
typedef struct decxb_conv_geom {
    int64_t out_w, out_h;  /* logical output size                                   */
    int64_t eq_w;          /* ceil4(out_w) = wpitch of the destination tensor       */
    int64_t M;             /* eq_w * out_h: rows of the column matrix                */
    int64_t Kp;            /* kW*kH*dpitch: columns of the column matrix             */
    int64_t Np;            /* ceil4(N): dpitch of the destination tensor             */
} decxb_conv_geom;
DECXB_API int decxb_conv_geometry(int64_t W, int64_t H, int64_t depth, int64_t kW, int64_t kH, int64_t N,
                                  int flag, decxb_conv_geom* out);

/* The pack step alone: column matrix I2C[M][Kp] of one tensor, bit-exact to
 * cu_sIm2Col_r8_within (srcs/convolution/CUDA/im2col/im2col.cuh:86-178) fed by the staging of
 * conv2_mk_im2col.h:234-238 with a zero apron:
 *   I2C[(y*eq_w + x)*Kp + (ky*kW + kx)*dpitch + c] = S[y+ky-oy][x+kx-ox][c]
 * (oy, ox) = (kH/2, kW/2) for the zero-border flag, (0, 0) for the valid flag; S is the
 * tensor value for 0<=row<H, 0<=col<wpitch and 0 elsewhere.  `batch` tensors lie
 * src_stride / i2c_stride elements apart. */
DECXB_API int decxb_im2col_pack_f32(decxb_ctx* ctx, const float* src, int64_t W, int64_t H, int64_t depth,
                                    int64_t kW, int64_t kH, int flag,
                                    float* i2c, int64_t batch, int64_t src_stride, int64_t i2c_stride,
                                    void* stream);

/* Which of the three bit-identical pack kernels the context uses: 0 (default) copy-engine pack
 * (TMA load of the source rows, bulk stores of the output runs; falls back when the rows do not
 * fit shared memory), 1 threads copy out of shared-memory staged rows, 2 threads copy straight
 * from global memory.  For measurement and tests. */
DECXB_API int decxb_set_pack_variant(decxb_ctx* ctx, int variant);

/* Whole convolution on device-resident tensors.  Replaces the pack and GEMM launches of
 * de::cuda::Conv2_MK_im2col (conv2_mk_im2col.h:278-306; drivers :57-162 and :167-274;
 * kernels cu_sIm2Col_r8_within and cu_conv_eq_mm).  dst is the destination tensor in its
 * padded layout [out_h][eq_w][Np] per image; padding pixels hold the convolution
 * evaluated there and padding channels hold 0, as in the reference.  Cross-correlation,
 * stride 1, kernel radius <= 8 (conv2_mk_im2col.h:170).  `batch` images lie
 * src_stride / dst_stride elements apart (0 = densely packed). */
DECXB_API int decxb_conv2_im2col_f32(decxb_ctx* ctx, int mode, int algo, int flag,
                                     const float* src, int64_t W, int64_t H, int64_t depth,
                                     const float* filters, int64_t kW, int64_t kH, int64_t N,
                                     float* dst, int64_t batch, int64_t src_stride, int64_t dst_stride,
                                     void* stream);

/* The same convolution with a fused epilogue: dst = act(conv + bias[filter]).  bias (device,
 * ceil4(N) floats, or NULL) and the activation are applied while the accumulator leaves tensor
 * memory, so the tensor is not read and written again by a separate operator (the reference
 * runs de::nn::ReLU_f / sigmoid_f / tanh_f as extra passes over the result). */
DECXB_API int decxb_conv2_im2col_f32_act(decxb_ctx* ctx, int mode, int algo, int flag,
                                         const float* src, int64_t W, int64_t H, int64_t depth,
                                         const float* filters, int64_t kW, int64_t kH, int64_t N,
                                         const float* bias, int activation,
                                         float* dst, int64_t batch, int64_t src_stride, int64_t dst_stride,
                                         void* stream);

/* Filter bank prepared once for many convolutions (weights stay the same from call to call): the
 * gather of the bank into the filter matrix and its hi/lo split are done by
 * decxb_conv_prepare_filters into arena memory owned by the handle; decxb_conv2_im2col_f32_prepared
 * is decxb_conv2_im2col_f32_act on that handle (mode and algorithm are the handle's; results are
 * bit-identical); decxb_conv_release_filters gives the memory back.  The reference re-stages the
 * bank with one copy per filter on every call (conv2_mk_im2col.h:226-231); no counterpart there. */
typedef struct decxb_prepared_filters decxb_prepared_filters;
DECXB_API int decxb_conv_prepare_filters(decxb_ctx* ctx, int mode, int algo, const float* filters, int64_t kW, int64_t kH,
                                         int64_t depth, int64_t N, void* stream, decxb_prepared_filters** out);
DECXB_API int decxb_conv2_im2col_f32_prepared(decxb_ctx* ctx, int flag, const float* src, int64_t W, int64_t H,
                                              const decxb_prepared_filters* filters, const float* bias, int activation,
                                              float* dst, int64_t batch, int64_t src_stride, int64_t dst_stride, void* stream);
DECXB_API int decxb_conv_release_filters(decxb_ctx* ctx, decxb_prepared_filters* filters, void* stream);

/* Host-resident tensors; blocks until dst is in host memory. */
DECXB_API int decxb_conv2_im2col_f32_host(decxb_ctx* ctx, int mode, int algo, int flag,
                                          const float* h_src, int64_t W, int64_t H, int64_t depth,
                                          const float* h_filters, int64_t kW, int64_t kH, int64_t N,
                                          float* h_dst, int64_t batch, int64_t src_stride, int64_t dst_stride);

/* ---- introspection for tests and benchmarks --------------------------------------- */
/* Tile order of the GEMM kernel: tiles are walked in groups of `tile_rows` tile-rows, column by
 * column inside a group, so that the blocks running at the same time share A row-panels and B
 * column-panels in L2 (1..64, default 8).  Results do not depend on it.  For measurement. */
DECXB_API int decxb_set_tile_group(decxb_ctx* ctx, int tile_rows);
/* Wave alignment of the GEMM kernel (on by default): in launches of several waves of a long-K product
 * the block pairs wait for one another at tile starts, so that the pairs sharing an operand panel
 * read it from L2 together instead of each fetching it from HBM (the slowest pair sets the pace
 * either way).  Results do not depend on it.  1 (default): such launches are cooperative, so all
 * blocks are resident together; only the launches that decxb_gemm_f32_rowshard_gather makes beside
 * a running transfer are plain ones with the same waits (a cooperative launch could be held back
 * until the transfer's blocks have gone).  2: the waits in plain launches throughout (a profiler
 * that cannot capture cooperative launches): the blocks are resident together only as long as
 * nothing else holds SMs, and a wait that cannot be met ends in DECXB_ERR_TIMEOUT after the limit.
 * 0: the pairs run free.  For measurement. */
DECXB_API int decxb_set_wave_align(decxb_ctx* ctx, int on);
/* Measurement: while `dbuf` (device memory, sm_count x tiles_per_cluster 64-bit words) is set, the
 * producer of every block (pair) of the GEMM kernel stores the GPU's global timer at the start of
 * each of its tiles at dbuf[block_pair * tiles_per_cluster + i], which shows how far the blocks
 * that share operand panels in L2 drift apart.  NULL or 0 switches it off. */
DECXB_API int decxb_set_tile_trace(decxb_ctx* ctx, unsigned long long* dbuf, int tiles_per_cluster);
/* Per-kernel device timing.  While enabled, every kernel the library launches is bracketed
 * by CUDA events on its own stream; decxb_profile_read synchronises the device, adds the
 * elapsed times to the totals below and returns them (decxb_profile_enable(ctx, 1) also
 * resets the totals).  No counterpart in the reference (its tests time whole calls with
 * clock(), test/test/CUDA_GEMM/CUDA_GEMM.cpp:43-55). */
enum { DECXB_K_GEMM = 0, DECXB_K_SPLIT = 1, DECXB_K_PACK = 2, DECXB_K_FILL = 3, DECXB_K_CLASSES = 4 };
typedef struct decxb_profile {
    double   ms[DECXB_K_CLASSES];        /* summed device time per kernel class */
    uint64_t launches[DECXB_K_CLASSES];
} decxb_profile;
DECXB_API int decxb_profile_enable(decxb_ctx* ctx, int on);
DECXB_API int decxb_profile_read(decxb_ctx* ctx, decxb_profile* out);

/* ---- sharding over ranks (one process per GPU) ---------------------------------------
 * The reference is single-GPU ("supports only single GPU", DECX_cpu/DECX_CPU.cpp:9); these
 * entries have no counterpart there.  The path shards into independent units: GEMM by rows of A
 * and C (B replicated), the convolution by images (filters replicated).  No data crosses
 * ranks to compute; gathering the result blocks, when the caller wants the whole result on every
 * rank, is what the decxb_comm_* entries further down do.
 *
 * decxb_shard_range: units [first, last) of `total` owned by `rank` of `world`; contiguous
 * blocks, the first total % world ranks own one unit more.
 * decxb_gemm_f32_rowshard: this rank's rows of D = A * B (+C).  A_rows / C_rows / D_rows point
 * at the rank's own row block (row `first` of the whole matrix), B is the whole matrix.
 * decxb_conv2_im2col_f32_batchshard: this rank's images; src / dst point at image `first`.
 * Both report the block they computed through first / last (either may be NULL). */
DECXB_API int decxb_shard_range(int64_t total, int world, int rank, int64_t* first, int64_t* last);
DECXB_API int decxb_gemm_f32_rowshard(decxb_ctx* ctx, int mode, int tile, int world, int rank,
                                      int64_t M, int64_t N, int64_t K,
                                      const float* A_rows, int64_t lda, const float* B, int64_t ldb,
                                      const float* C_rows, int64_t ldc, float* D_rows, int64_t ldd,
                                      void* stream, int64_t* first, int64_t* last);
DECXB_API int decxb_conv2_im2col_f32_batchshard(decxb_ctx* ctx, int mode, int algo, int flag, int world, int rank,
                                                const float* src, int64_t W, int64_t H, int64_t depth,
                                                const float* filters, int64_t kW, int64_t kH, int64_t N,
                                                float* dst, int64_t batch, int64_t src_stride, int64_t dst_stride,
                                                void* stream, int64_t* first, int64_t* last);

/* Tensor-core ceiling probe: runs nothing but a stream of tcgen05.mma kind::tf32 256 x 256 x 8
 * instructions (CTA pairs on all SMs, operands resident in shared memory, no TMA, no epilogue)
 * for about target_ms and reports what the tensor pipe delivered.  pattern 0: one MMA per
 * k-step, the TF32 issue peak; 1: the three MMAs of the GEMM kernel's 3xTF32 k-step on four
 * distinct operand tiles, the ceiling its shared-memory operand reads leave; 2: as 1 with a_hi
 * kept in the collector buffer; 3, 4, 5: pattern 2 on the single-CTA tiles 128 x 64, 128 x 128,
 * 128 x 256.  algorithmic_tflops = tensor_tflops / MMAs per k-step, directly
 * comparable with the GEMM's 2 M N K / t.  The denominators of the benchmark's roofline come
 * from here.  No counterpart in the reference (it publishes no peak figure). */
typedef struct decxb_tensor_probe {
    double ms;                   /* duration of the measured launch                       */
    double tensor_tflops;        /* flops the tensor pipe executed / ms                   */
    double algorithmic_tflops;   /* the same divided by the MMAs per k-step (1 or 3)      */
    int64_t iterations;          /* k-blocks (4 k-steps) issued per CTA pair              */
    int sms;                     /* SMs that took part                                    */
} decxb_tensor_probe;
DECXB_API int decxb_probe_tensor_peak(decxb_ctx* ctx, int pattern, double target_ms, decxb_tensor_probe* out);

/* Host-side fault injection for tests: the CUDA call number `nth_call` (0 = the next one) that a
 * host-resident pipeline (decxb_gemm_f32_host, _f16_host, _batched_host,
 * decxb_conv2_im2col_f32_host) makes from now on is not issued and reports a failure instead;
 * the pipeline must drain its streams, return DECXB_ERR_CUDA and leave the context usable.
 * nth_call < 0 switches it off.  Nothing on the device faults.  No counterpart in the reference
 * (its error path prints and exits, srcs/core/error.h:33-42). */
DECXB_API int decxb_inject_pipeline_error(decxb_ctx* ctx, int nth_call);

/* ---- gathering the blocks of a sharded result (NCCL over NVLink) ---------------------------
 * No counterpart in the reference (single GPU).  The shards above need no communication; these
 * entries serve callers that want the WHOLE result on every rank.  NCCL is loaded at run time
 * (libnccl.so.2, or the file the environment variable DECXB_NCCL_LIB names); a process that
 * never calls them never loads it.
 *
 * decxb_comm_unique_id: 128 bytes that rank 0 creates and hands to every rank by its own means
 *   (a file, a socket, MPI, torch.distributed).
 * decxb_comm_init: joins `world` ranks, one per GPU; blocks until all have joined or timeout_ms
 *   (<= 0: 30 s) has passed, then DECXB_ERR_TIMEOUT.  The same limit bounds every later wait on
 *   this communicator; after a timeout or an NCCL error the communicator has been aborted and
 *   only decxb_comm_destroy may be called on it.
 * decxb_comm_allgather_blocks: `base` holds total_units units of unit_bytes each, laid out alike
 *   on every rank; the rank's own units (decxb_shard_range) are valid, the others arrive.  Ordered
 *   after the work queued on `stream`, and `stream` continues after the transfer (no host wait).
 * decxb_gemm_f32_rowshard_gather: this rank's rows of D = A * B computed in `groups` row-panel
 *   groups (1..64) straight into D_full[M][N] (dense, leading dimension N), each group sent to
 *   the peers while the next is multiplied; on return everything is queued, and `stream`
 *   continues only after all rows of D_full have arrived.  groups = 1 computes, then gathers.
 *   The last group, whose transfer nothing overlaps, is a third of an even share and travels
 *   through a communicator with many thread blocks per NCCL kernel (32, environment variable
 *   DECXB_COMM_WIDE_CTAS; decxb_comm_allgather_blocks uses the same one); the groups that travel
 *   beside a GEMM use a second communicator limited to a few (two per rank, 4 to 16; DECXB_COMM_MAX_CTAS), and the GEMM
 *   leaves that many SMs free (decxb_comm_set_reserved_sms changes the number of SMs).  A_rows
 *   points at the rank's first row; B is the whole matrix.
 * decxb_comm_synchronize: waits (bounded) until the transfers queued so far have finished. */
#define DECXB_COMM_ID_BYTES 128
typedef struct decxb_comm decxb_comm;
DECXB_API int decxb_comm_unique_id(void* id128);
DECXB_API int decxb_comm_init(decxb_ctx* ctx, int world, int rank, const void* id128, int timeout_ms, decxb_comm** out);
DECXB_API int decxb_comm_destroy(decxb_comm* comm);
DECXB_API const char* decxb_comm_last_error(decxb_comm* comm);
DECXB_API int decxb_comm_set_reserved_sms(decxb_comm* comm, int sms);
DECXB_API int decxb_comm_synchronize(decxb_comm* comm);
DECXB_API int decxb_comm_allgather_blocks(decxb_comm* comm, void* base, size_t unit_bytes, int64_t total_units, void* stream);
DECXB_API int decxb_gemm_f32_rowshard_gather(decxb_ctx* ctx, decxb_comm* comm, int mode, int tile,
                                             int64_t M, int64_t N, int64_t K,
                                             const float* A_rows, int64_t lda, const float* B, int64_t ldb,
                                             float* D_full, int groups, void* stream);
/* Host-resident operands on several GPUs: this rank's rows of D = A * B, with hA_rows / hD_rows pointing at the
 * rank's first row in host memory and hB at the whole B (every rank can read it; pinned memory makes the copies fast).
 * A rank uploads only its own 1/world of B's rows and the ranks all-gather B on the device over NVLink, because the
 * host's copy bandwidth is shared by all ranks of a box and NVLink is not; the rank's rows of A go up in row blocks
 * that overlap the arithmetic and the way back of the result.  Blocks until hD_rows is complete (bounded by the
 * communicator's time limit).  The single-GPU counterpart in the reference is de::cuda::GEMM on Matrix
 * (srcs/GEMM/CUDA/large_squares/GEMM.h:56-131); the sharding has none. */
DECXB_API int decxb_gemm_f32_rowshard_host(decxb_ctx* ctx, decxb_comm* comm, int mode, int tile,
                                           int64_t M, int64_t N, int64_t K,
                                           const float* hA_rows, int64_t lda, const float* hB, int64_t ldb,
                                           float* hD_rows, int64_t ldd);
/* How decxb_gemm_f32_host (world = 1) and decxb_gemm_f32_rowshard_host (M = the rank's rows) cut a product: pure
 * host arithmetic, no CUDA call.  Writes up to `capacity` triples (kind, first, count) in the order of use and
 * returns how many there are (-1 for bad arguments): kind 0 = a column block of B (columns first .. first+count),
 * kind 1 = a piece of the first row-block of A, kind 2 = a later row-block.  The column blocks cover [0, N) once,
 * pieces and row-blocks together cover [0, M) once.  For tests and for callers that want to see the granularity of
 * the copies; no counterpart in the reference, whose host path copies whole matrices (GEMM.h:106-123). */
DECXB_API int decxb_gemm_host_plan(int64_t M, int64_t N, int64_t K, int world, int64_t* kind_first_count, int capacity);
/* Failure-detection self-test on the host: the joining half of decxb_comm_init (load the library at
 * nccl_path, non-blocking init, bounded poll, abort on expiry) with no CUDA call, so that a rank
 * which never arrives can be played by a stand-in library on a machine without a GPU. */
DECXB_API int decxb_comm_selftest_handshake(const char* nccl_path, int world, int rank, const void* id128, int timeout_ms,
                                            char* err, size_t err_len);

/* Debug bounds build.  `make -C backup_1_b200/csrc bounds` builds libdecxb_bounds.so, the same library
 * compiled with -DDECXB_BOUNDS: every global load and store made by the threads of the
 * memory-bound kernels (operand split, transposes, filter matrix, pack, fill) is checked against
 * the extent of its array; the first violation is recorded in the status word and the access
 * skipped (nothing faults), and the next status check (decxb_synchronize, the blocking entries)
 * returns DECXB_ERR_BOUNDS.  decxb_bounds_build tells which library is loaded;
 * decxb_selftest_bounds provokes one caught violation (valid memory, an extent declared one row
 * short).  The reference has no such facility (its kernels are unchecked); it stands in for a
 * memory checker where none can be run. */
DECXB_API int decxb_bounds_build(void);
DECXB_API int decxb_selftest_bounds(decxb_ctx* ctx);

/* Number of kernels this library has launched on the context since it was created. */
DECXB_API uint64_t decxb_kernel_launch_count(decxb_ctx* ctx);
/* Failure-detection self-test: launches one tiny kernel whose only thread waits, with the
 * library's bounded wait, on a barrier that nothing signals.  Returns DECXB_ERR_TIMEOUT after
 * `limit_ms` (1..1000) when the mechanism works; the context stays usable.  No counterpart in
 * the reference (its kernels have no device-side waits). */
DECXB_API int decxb_selftest_bounded_wait(decxb_ctx* ctx, int limit_ms);
DECXB_API const char* decxb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DECXB_H_ */
