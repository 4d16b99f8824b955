/* Shared declarations of the decxb CUDA library (internal; the public ABI is include/decxb.h). */
#ifndef DECXB_COMMON_H_
#define DECXB_COMMON_H_

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "decxb.h"

/* Status word the kernels report to (device memory, one per context; copied to the pinned
 * host twin when the host checks it). */
struct decxb_dev_status {
    int code;        /* 0 = fine; else a DECXB_DEVERR_* code              */
    int where;       /* role/barrier id that gave up                       */
    int block;       /* blockIdx.x of the reporter                         */
    int detail;      /* stage / tile index                                 */
};

/* Per-device tables (kernel attributes set once per device) are sized by this; decxb_init
 * refuses device indices beyond it. */
#define DECXB_MAX_DEVICES 64
#define DECXB_WAVE_SLOTS 32

enum {
    DECXB_DEVERR_NONE = 0,
    DECXB_DEVERR_WAIT_EXPIRED = 1,
    DECXB_DEVERR_BOUNDS = 2,          /* debug bounds build: an access outside its array was caught and skipped */
};

/* Debug bounds build (compile the library with -DDECXB_BOUNDS; `make bounds` builds it beside the
 * normal one): every global load and store that the threads of the memory-bound kernels make
 * (operand split, transposes, filter matrix, pack, fill) is checked against the extent of the array
 * it belongs to.  The first violation is recorded in the context's status word (kernel id, block,
 * element offset) and the access is skipped, so nothing faults; the host reports
 * DECXB_ERR_BOUNDS at its next status check.  In the normal build the checks compile to nothing.
 * (compute-sanitizer would do this job and is not available where this library is developed.) */
struct decxb_extent { const char* lo; const char* hi; };      /* [lo, hi) */
struct decxb_bounds {
    decxb_dev_status* status;
    decxb_extent in, out0, out1;
    int kernel;                       /* DECXB_BK_* */
};
enum { DECXB_BK_FILL = 1, DECXB_BK_SPLIT_ROWS, DECXB_BK_SPLIT_TRANSPOSE, DECXB_BK_FILTER_MATRIX, DECXB_BK_TRANSPOSE_F16, DECXB_BK_PACK };

static inline decxb_extent decxb_make_extent(const void* base, size_t bytes)
{
    return decxb_extent{static_cast<const char*>(base), static_cast<const char*>(base) + (base ? bytes : 0)};
}

#if defined(__CUDACC__)
#ifdef DECXB_BOUNDS
__device__ __forceinline__ bool decxb_access_ok(const decxb_bounds& b, const decxb_extent& e, const void* p, size_t bytes)
{
    const char* c = static_cast<const char*>(p);
    if (c >= e.lo && c + bytes <= e.hi) return true;
    if (atomicCAS(&b.status->code, 0, DECXB_DEVERR_BOUNDS) == 0) {
        b.status->where = b.kernel; b.status->block = (int)blockIdx.x;
        b.status->detail = (int)((c - e.lo) >> 2);
        __threadfence_system();
    }
    return false;
}
#define DECXB_OK_IN(b, p, n)   decxb_access_ok((b), (b).in, (p), (n))
#define DECXB_OK_OUT0(b, p, n) decxb_access_ok((b), (b).out0, (p), (n))
#define DECXB_OK_OUT1(b, p, n) decxb_access_ok((b), (b).out1, (p), (n))
#else
#define DECXB_OK_IN(b, p, n)   true
#define DECXB_OK_OUT0(b, p, n) true
#define DECXB_OK_OUT1(b, p, n) true
#endif
#endif

/* A cached block remembers the stream that used it last and an event recorded there when it
 * was released, so the same stream can take it again at once (stream order protects it) and
 * another stream waits on the event first. */
struct decxb_cached_block { void* ptr; cudaStream_t stream; cudaEvent_t ev; };

struct decxb_arena {
    std::mutex mtx;
    std::unordered_map<void*, size_t> live;           /* ptr -> block bytes */
    std::multimap<size_t, decxb_cached_block> cached; /* block bytes -> block */
    std::vector<cudaEvent_t> ev_pool;
    size_t bytes_in_use = 0, bytes_cached = 0, peak = 0;
    uint64_t n_driver_allocs = 0, n_reuses = 0;
};

/* Encoded 2-D tensor maps of recent GEMM operands (see make_map in gemm_tcgen05.cu). */
struct decxb_map_key {
    const void* base; int64_t rows, K, ld; int box_rows;
    bool operator==(const decxb_map_key& o) const { return base == o.base && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows; }
};
struct decxb_map_entry { bool used = false; decxb_map_key key = {}; CUtensorMap map; uint64_t stamp = 0; };

struct decxb_ctx {
    int device = -1;
    int sm_count = 0;
    cudaStream_t stream = nullptr;      /* the context's own compute stream        */
    cudaStream_t copy_stream[2] = {nullptr, nullptr};
    decxb_arena arena;
    decxb_dev_status* h_status = nullptr;   /* pinned host twin                     */
    decxb_dev_status* d_status = nullptr;   /* device word the kernels write        */
    long long wait_limit_ns = 2000000000LL;
    int pack_variant = 0;               /* 0 = copy-engine (TMA) pack, 1 = shared-memory staged, 2 = direct */
    std::atomic<uint64_t> launches{0};
    std::mutex map_mtx;
    decxb_map_entry map_cache[16];
    uint64_t map_clock = 0;
    /* wave alignment of the GEMM kernel: one monotonic counter per launching stream (so that launches on
     * different streams, whose order on the GPU is not the host's, never share one), and what it will read
     * when the launches queued so far have run */
    unsigned long long* wave_counters = nullptr;      /* device, DECXB_WAVE_SLOTS words, zero at start */
    std::mutex wave_mtx;
    struct WaveSlot { cudaStream_t stream; unsigned long long base; bool used; } wave_slots[DECXB_WAVE_SLOTS] = {};
    int wave_align = 1;                               /* decxb_set_wave_align */
    unsigned long long* trace = nullptr;   /* decxb_set_tile_trace: device buffer [clusters][trace_tiles] of tile start times */
    int trace_tiles = 0;
    int tile_group = 8;                 /* tile-rows per group of the GEMM kernel's tile order (decxb_set_tile_group) */
    int reserved_sms = 0;               /* SMs the next GEMM launches leave free (a transfer kernel runs beside them) */
    int inject_countdown = -1;          /* >= 0: that many pipeline CUDA calls from now, one reports a failure (tests) */
    std::string last_error;
    /* per-kernel event timing (decxb_profile_*) */
    bool profiling = false;
    std::mutex prof_mtx;
    struct ProfSpan { int cls; cudaEvent_t a, b; };
    std::vector<ProfSpan> prof_open;
    std::vector<cudaEvent_t> prof_pool;
    decxb_profile prof_total = {};
};

/* RAII bracket around one kernel launch: counts it and, when profiling, records events. */
struct decxb_launch_scope {
    decxb_ctx* ctx; cudaStream_t s; int cls; cudaEvent_t b = nullptr;
    decxb_launch_scope(decxb_ctx* c, cudaStream_t st, int k);
    ~decxb_launch_scope();
};

#define DECXB_CUDA_TRY(ctx, expr)                                                              \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess) {                                                               \
            decxb_set_error((ctx), std::string(#expr) + ": " + cudaGetErrorString(_e));       \
            return DECXB_ERR_CUDA;                                                             \
        }                                                                                      \
    } while (0)

int decxb_fail(decxb_ctx* ctx, int status, const std::string& msg);
void decxb_set_error(decxb_ctx* ctx, const std::string& msg);
/* Binds the context's device to the calling thread. */
int decxb_bind(decxb_ctx* ctx);
/* Stream-ordered scratch: the block may be handed out again while work queued on `s` before
 * the release is still running; a taker on another stream waits for it on the device. */
int decxb_malloc_on_stream(decxb_ctx* ctx, size_t bytes, void** dptr, cudaStream_t s);
int decxb_free_on_stream(decxb_ctx* ctx, void* dptr, cudaStream_t s);
/* Wave alignment bookkeeping: the counter of stream `s` and its value before a launch that will add `arrivals`
 * to it (false: no slot free, launch without alignment); _unslot takes the arrivals of a launch that was not made
 * back; _reset zeroes everything after a launch gave up (device idle). */
bool decxb_wave_slot(decxb_ctx* ctx, cudaStream_t s, unsigned long long arrivals, unsigned long long** counter, unsigned long long* base);
void decxb_wave_unslot(decxb_ctx* ctx, cudaStream_t s, unsigned long long arrivals);
void decxb_wave_reset(decxb_ctx* ctx);
/* Reads (and clears) the device status word after a synchronisation. */
int decxb_check_dev_status(decxb_ctx* ctx);

static inline int64_t decxb_ceil_to(int64_t v, int64_t m) { return (v + m - 1) / m * m; }
static inline int64_t decxb_ceil_div(int64_t v, int64_t m) { return (v + m - 1) / m; }
/* Row pitch (floats) of the library's own hi/lo operand arrays for a row of K values: a multiple of 4
 * (16 bytes, the copy engine's rule).  (Padding power-of-two pitches by a line was measured at
 * 16384^3 and changed neither the DRAM traffic nor the time.) */
static inline int64_t decxb_split_pitch(int64_t K) { return decxb_ceil_to(K, 4); }

/* ---- internal kernels' launchers (each returns a decxb_status) ------------------------ */

/* hi = tf32(a), lo = tf32(a - hi); out pitch `ld_out` (pad columns zeroed).  lo may be NULL. */
int decxb_launch_split_rows(decxb_ctx* ctx, const float* in, int64_t rows, int64_t cols, int64_t ld_in,
                            float* hi, float* lo, int64_t ld_out, int64_t rows_out, cudaStream_t s,
                            int64_t nbatch = 1, int64_t in_batch_stride = 0, int raw = 0);
/* Transposing variant: in[K][ld_in] (K rows, N cols) -> hi/lo[N][ld_out]; `raw` keeps hi = a unrounded. */
int decxb_launch_split_transpose(decxb_ctx* ctx, const float* in, int64_t K, int64_t N, int64_t ld_in,
                                 float* hi, float* lo, int64_t ld_out, int raw, cudaStream_t s,
                                 int64_t nbatch = 1, int64_t in_batch_stride = 0, int64_t out_batch_rows = 0);

/* A -> hi/lo [M][ld_out] and B[K][N] -> hi/lo [N][ld_out] in one launch (3xTF32 operands of one product);
 * possible when B and its outputs allow 128-bit accesses. */
bool decxb_split_ab_possible(const float* B, int64_t ldb, const float* b_hi, const float* b_lo);
int decxb_launch_split_ab(decxb_ctx* ctx, const float* A, int64_t M, int64_t K, int64_t lda, float* a_hi, float* a_lo,
                          const float* B, int64_t N, int64_t ldb, float* b_hi, float* b_lo, int64_t ld_out, cudaStream_t s);

/* Operands of the TF32 + 2 x bf16 mode: hi = tf32(a) [rows][ld_hi], lo16 = bf16(a - hi) and a16 = bf16(a) [rows][ld16]. */
int decxb_launch_split_rows_bf16(decxb_ctx* ctx, const float* in, int64_t rows, int64_t cols, int64_t ld_in,
                                 float* hi, void* lo16, void* a16, int64_t ld_hi, int64_t ld16, cudaStream_t s);
int decxb_launch_split_transpose_bf16(decxb_ctx* ctx, const float* in, int64_t K, int64_t N, int64_t ld_in,
                                      float* hi, void* lo16, void* b16, int64_t ld_hi, int64_t ld16, cudaStream_t s);

/* The tensor-core GEMM on K-contiguous operands.  a_hi/a_lo: [M][lda], b_hi/b_lo: [N][ldb]
 * (lo pointers NULL for plain TF32).  C optional addend, D output. */
struct decxb_gemm_args {
    int64_t M, N, K;
    const float *a_hi, *a_lo; int64_t lda;
    const float *b_hi, *b_lo; int64_t ldb;
    int64_t b_rows;            /* rows of the B operand arrays that exist (>= N is not required: rows beyond are read as 0) */
    const float* C; int64_t ldc;
    float* D; int64_t ldd;
    int tile;
    const float* bias; int act;      /* fused epilogue (NULL / DECXB_ACT_NONE = off) */
    int chunked;                     /* 1 = accumulate K in chunks of 128 added in IEEE fp32 (3xTF32 only) */
    /* TF32 + 2 x bf16 mode (a_16 != NULL): bf16(a), bf16(a_lo), bf16(b), bf16(b_lo), [rows][ld16] with K contiguous */
    const void *a_16, *a_lo16, *b_16, *b_lo16; int64_t ld16;
    /* batched: nbatch > 1 stacked matrices; A holds m_pad rows per matrix, B n_pad rows per matrix
     * (both multiples of the tile chosen by `tile`, which must then be explicit) */
    int64_t nbatch, m_pad, n_pad, d_batch_stride, c_batch_stride;
};
/* Tile shape (rows, cols) of a decxb_gemm_tile value; the AUTO choice for a batched problem. */
void decxb_tile_shape(int tile, int* tm, int* tn);
int decxb_pick_tile(decxb_ctx* ctx, int64_t M, int64_t N, int64_t nbatch);
int decxb_launch_gemm_tn(decxb_ctx* ctx, const decxb_gemm_args& a, cudaStream_t s);

/* fp16 GEMM on K-contiguous operands: A [M][lda], Bt [N][ldbt] (halves), optional fp16 addend,
 * fp16 result, fp32 accumulation. */
struct decxb_gemm_f16_args {
    int64_t M, N, K;
    const void* A; int64_t lda;
    const void* Bt; int64_t ldbt;
    const void* C; int64_t ldc;
    void* D; int64_t ldd;
    int act;
};
int decxb_launch_gemm_f16_tn(decxb_ctx* ctx, const decxb_gemm_f16_args& a, cudaStream_t s);
/* in[K][ld_in] halves (K rows, N columns) -> out[N][ld_out] halves, columns >= K zeroed. */
int decxb_launch_transpose_f16(decxb_ctx* ctx, const void* in, int64_t K, int64_t N, int64_t ld_in,
                               void* out, int64_t ld_out, cudaStream_t s);

/* Implicit-GEMM convolution: the A tiles are boxes of the (split) source tensor, the filter
 * matrix is [k_rows][ldk] with one 32-channel-padded block row per tap: column
 * (tap * cblocks + cb) * 32 + c'. */
struct decxb_conv_gemm_args {
    const float *src_hi, *src_lo;     /* [batch][H][wp][dp]; lo NULL for plain TF32 */
    int64_t dp, wp, H, batch, src_img_stride;
    const float *k_hi, *k_lo; int64_t k_rows, k_cols, ldk;
    int64_t kW, kH; int off_x, off_y;
    int64_t out_h, eq_w, Np;
    float* dst; int64_t dst_img_stride;
    const float* bias; int act;
    int chunked;                      /* as decxb_gemm_args::chunked */
};
int decxb_launch_conv_implicit(decxb_ctx* ctx, const decxb_conv_gemm_args& a, cudaStream_t s);

/* Rows of D = A * B (+C) (+bias, activation) with B prepared by decxb_gemm_prepare_b. */
/* B of a host-resident product arriving in shares (several ranks): this rank uploads rows [k_first, k_last) of each
 * column block; `gather` (ordered after `s`'s earlier work, and `s` waits for it) completes the block from the peers:
 * `units` rows of unit_bytes each, partitioned over the ranks by decxb_shard_range. */
struct decxb_b_share {
    int world;
    int64_t k_first, k_last;
    int (*gather)(void* user, float* base, size_t unit_bytes, int64_t units, cudaStream_t s);
    void* user;
};
int decxb_gemm_host_pipeline(decxb_ctx* ctx, int mode, int tile, int64_t M, int64_t N, int64_t K,
                             const float* hA, int64_t lda, const float* hB, int64_t ldb,
                             const float* hC, int64_t ldc, float* hD, int64_t ldd, const decxb_b_share* share);

int decxb_gemm_rows_prepared_b(decxb_ctx* ctx, int mode, int tile, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                               const decxb_prepared_b* pb, const float* C, int64_t ldc, float* D, int64_t ldd, cudaStream_t s,
                               const float* bias = nullptr, int act = DECXB_ACT_NONE);

/* cuTensorMapEncodeTiled, resolved through cudaGetDriverEntryPoint (NULL if unavailable). */
void* decxb_tensor_map_encoder();

int decxb_launch_pack(decxb_ctx* ctx, const float* src, int64_t W, int64_t H, int64_t depth,
                      int64_t kW, int64_t kH, int flag, float* i2c, int64_t batch,
                      int64_t src_stride, int64_t i2c_stride, cudaStream_t s);

/* Filter bank (TensorArray layout) -> hi/lo [rows_out][ld_out] matrices, filter n in row n. */
int decxb_launch_filter_matrix(decxb_ctx* ctx, const float* filters, int64_t kW, int64_t kH, int64_t depth,
                               int64_t N, float* hi, float* lo, int64_t rows_out, int64_t ld_out, int raw,
                               cudaStream_t s, int64_t chan_pitch = 0);

#endif
