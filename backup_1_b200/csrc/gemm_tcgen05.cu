/*
 * fp32 GEMM on Blackwell tensor cores (sm_100a): D[M][N] = A[M][K] * Bt[N][K]^T (+ C).
 *
 * Replaces the reference's CUDA-core FFMA kernels cu_GEMM_fp32_spec / _ABC_spec and their
 * ragged variants (srcs/GEMM/CUDA/large_squares/GEMM.cuh:31-100, :206-280;
 * GEMM_nonuniform.cuh:32-693) and the convolution's cu_conv_eq_mm
 * (srcs/convolution/CUDA/im2col/eq_GEMM.cuh:109-209).
 *
 * Shape of the kernel
 *  - Both operands arrive K-contiguous ("TN"), already split into TF32 hi/lo parts for the
 *    3xTF32 mode (prep_kernels.cu).  Every k-block of 32 floats is one 128-byte row, loaded
 *    by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a ring of shared-memory stages.
 *  - tcgen05.mma kind::tf32, accumulators in tensor memory (TMEM), fp32.  3xTF32 issues
 *    a_lo*b_hi, a_hi*b_lo, a_hi*b_hi into the same accumulator for every k-step of 8.
 *  - Warp-specialised, persistent: warp 0 = TMA producer, warp 1 = MMA issuer (and TMEM
 *    owner), warps 2..9 = epilogue, four TMEM lane quarters x two column halves (warps 2..5 in
 *    the fp16 kernel) (tcgen05.ld -> registers -> a swizzled 32 x 32 box in shared
 *    memory -> one TMA store per box; 128-bit stores from the threads for layouts the copy
 *    engine cannot describe).  The accumulator is double-buffered in TMEM so the epilogue of
 *    tile i overlaps the main loop of tile i+1.
 *  - CTAS = 2 pairs two CTAs (one thread-block cluster) on a 256 x (2*BN) tile with
 *    cta_group::2: each CTA loads its own 128 rows of A and its own half of B, the leader
 *    CTA issues the MMAs for both, completion is signalled to both CTAs with one commit.
 *    Loads are plain (non-multicast) TMA into the issuing CTA's own shared memory.
 *  - Every wait on an mbarrier is bounded (wall-clock limit from the context); on expiry the
 *    waiter records where it gave up in the context's status word, all roles drain, tensor
 *    memory is released and the kernel returns.
 */
#include "common.h"
#include "tc_ptx.cuh"

#include <cudaTypedefs.h>
#include <cuda_fp16.h>

namespace {

constexpr int BM_CTA = 128;        /* rows of A (and of the accumulator) per CTA          */
constexpr int BK = 32;             /* floats per k-block = one 128-byte swizzle row        */
constexpr int UMMA_K = 8;          /* k per tcgen05.mma kind::tf32                          */
constexpr int NUM_THREADS_F16 = 192;   /* fp16 kernel: producer, MMA issuer, 4 epilogue warps     */
constexpr int NUM_THREADS = 320;   /* fp32 whole-K kernels: producer, MMA issuer, 8 epilogue warps (4 lane quarters x 2 column halves) */
constexpr int NUM_THREADS_CHUNKED = 384;   /* chunked accumulation: warp group 0 = producer, MMA issuer
                                              and two idle warps; warp groups 1, 2 = 8 epilogue warps */
constexpr int KCHUNK = 4;          /* k-blocks per chunk of the chunked accumulation: 128 values of K
                                      (256 for the first two chunks of a tile, see chunk_blocks).
                                      Largest error seen on the all-positive 2048^3 case, relative to
                                      K max|a| max|b|, with uniform chunks of 64 -> 1.9e-7,
                                      128 -> 3.3e-7, 256 -> 6.5e-7, 512 -> 1.2e-6, whole K -> 2.9e-6 */
constexpr int SMEM_LIMIT = 232448; /* 227 KiB opt-in maximum per CTA                        */
#ifndef DECXB_A_COLLECTOR
#define DECXB_A_COLLECTOR 1
#endif
constexpr bool A_COLLECTOR = DECXB_A_COLLECTOR != 0;   /* collector-buffer reuse of a_hi in the 3xTF32 k-step */

using namespace tcptx;


struct GemmParams {
    int64_t M, N, K;
    const float* C; int64_t ldc;
    float* D; int64_t ldd;
    int tiles_m, tiles_n, num_kb;
    long long wait_limit_ns;
    decxb_dev_status* status;
    /* implicit-GEMM convolution only: an M tile of one CTA is a BX x BY patch of output
     * pixels of one image; a k-block is 32 channels of one filter tap */
    int bx, by;                 /* patch of output pixels that one TMA box covers, bx * by = 128 / nbox  */
    int nbox;                   /* patches (boxes) per CTA tile: 1, 2 or 4; patch s of the launch is patch
                                   s % (tiles_x * tiles_y) of image s / (tiles_x * tiles_y), x fastest, and
                                   CTA c of tile t owns patches ((t * CTAS + c) * nbox + j), j < nbox   */
    int tiles_x, tiles_y;       /* patches per image row / per image column                      */
    int batch;                  /* images                                                        */
    int out_h, eq_w;            /* output rows, pixels per output row (= wpitch of destination)  */
    int kw, off_x, off_y;       /* filter width, source offset of tap (0,0)                      */
    int cblocks;                /* 32-channel blocks per tap                                     */
    int64_t dst_img_stride;     /* floats between destination images                             */
    /* batched GEMM: the operand arrays stack `nbatch` matrices, each padded to whole tiles
     * (tiles_m_per tiles of rows in A, b_batch_rows rows in B); results lie d_batch_stride apart */
    int tiles_m_per;            /* 0 = not batched                                                */
    int64_t b_batch_rows, d_batch_stride, c_batch_stride;
    /* fused epilogue: D = act(acc (+C) (+bias[col])) */
    const float* bias;          /* per output column (filter), or NULL                            */
    int act;                    /* DECXB_ACT_*                                                    */
    int tma_store;              /* 1 = results leave through shared memory and TMA stores (map_d)   */
    int tile_group;             /* tile-rows per group of the tile order                            */
    /* wave alignment (see align_wave): counter shared by all blocks of the launch, value it had before the launch */
    unsigned long long* wave_counter;
    unsigned long long wave_base;
    unsigned long long* trace;  /* measurement: global-timer value at the start of every tile of every cluster, or NULL */
    int trace_tiles;            /* entries per cluster in `trace`                                   */
};

/* Activations with the reference's formulas (srcs/nn/operators/ReLU.h:48-75 keeps x when its
 * sign bit is clear; sigmoid.h:45-46: 1 / (1 + __expf(-x)); tanh.h:41-42:
 * (__expf(2x) - 1) / (__expf(2x) + 1)). */
__device__ __forceinline__ float apply_act(float x, int act)
{
    switch (act) {
    case DECXB_ACT_RELU: return x < 0.0f ? 0.0f : x;
    case DECXB_ACT_SIGMOID: return __frcp_rn(__fadd_rn(1.0f, __expf(__fmul_rn(x, -1.0f))));
    case DECXB_ACT_TANH: { const float e = __expf(__fmul_rn(x, 2.0f)); return __fdiv_rn(__fsub_rn(e, 1.0f), __fadd_rn(e, 1.0f)); }
    default: return x;
    }
}

/* Bounded wait.  Returns false when it gave up (or another role already had). */
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, const GemmParams& p, int where, int detail)
{
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 1023u) == 0) {
            if (*reinterpret_cast<volatile int*>(&p.status->code) != 0) return false;
            if ((long long)(globaltimer_ns() - t0) > p.wait_limit_ns) {
                if (atomicCAS(&p.status->code, 0, DECXB_DEVERR_WAIT_EXPIRED) == 0) {
                    p.status->where = where; p.status->block = (int)blockIdx.x; p.status->detail = detail;
                    __threadfence_system();
                }
                return false;
            }
        }
    }
    return true;
}

/* Wave alignment.  All block pairs walk the tile list in lock step (pair c takes tiles c, c + P, c + 2P, ...),
 * and the pairs of one wave share operand panels: the L2 serves a panel's k-block to every pair that asks for
 * it while it is still resident.  Left alone the pairs drift apart (some SMs are a percent or two slower;
 * measured: 400 us of spread after 50 tiles of 540 us at 16384^3), the same k-block is then fetched from HBM
 * once per pair instead of once per wave, and the DRAM traffic grows to 20 times the operands.  So before the
 * first load of its tile i >= 1 the leading producer announces itself on a counter in global memory and waits,
 * with the usual time limit, until every pair that has a tile i has done the same.  The slowest pair sets the
 * pace either way (the launch ends when it ends); the others now wait at tile starts instead of at the end.
 * The launch is made cooperative, so all blocks are resident together and the wait can always be satisfied. */
__device__ __noinline__ bool align_wave_wait(unsigned long long* counter, unsigned long long target, long long limit_ns,
                                            decxb_dev_status* status, int detail)
{
    /* (not inlined: the producer that calls it lives on 56 registers in the chunked kernels) */
    atomicAdd(counter, 1ULL);
    volatile unsigned long long* c = counter;
    if (*c >= target) return true;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (*c < target) {
        __nanosleep(100);
        if ((++spins & 63u) == 0) {
            if (*reinterpret_cast<volatile int*>(&status->code) != 0) return false;
            if ((long long)(globaltimer_ns() - t0) > limit_ns) {
                if (atomicCAS(&status->code, 0, DECXB_DEVERR_WAIT_EXPIRED) == 0) {
                    status->where = 500; status->block = (int)blockIdx.x; status->detail = detail;
                    __threadfence_system();
                }
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ bool align_wave(const GemmParams& p, int local_tile, int num_clusters, int num_tiles, int t)
{
    const int with_tile = min(num_clusters, num_tiles - local_tile * num_clusters);
    const unsigned long long target = p.wave_base + (unsigned long long)(local_tile - 1) * (unsigned long long)num_clusters +
                                      (unsigned long long)with_tile;
    return align_wave_wait(p.wave_counter, target, p.wait_limit_ns, p.status, t);
}

/* Writes 32 consecutive result columns of one row, first column `col_first`:
 * (+C) (+bias[col]) activation, with 128-bit stores when `vec` says the rows allow them. */
__device__ __forceinline__ void store32_f32(const float* v, int64_t col_first, const GemmParams& p,
                                            float* __restrict__ drow, const float* __restrict__ crow, bool vec)
{
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const int64_t col = col_first + j;
        if (col + 3 < p.N && vec) {
            float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            if (crow) {
                const float4 ci = __ldg(reinterpret_cast<const float4*>(crow + col));
                o.x += ci.x; o.y += ci.y; o.z += ci.z; o.w += ci.w;
            }
            if (p.bias) {
                o.x += __ldg(p.bias + col); o.y += __ldg(p.bias + col + 1);
                o.z += __ldg(p.bias + col + 2); o.w += __ldg(p.bias + col + 3);
            }
            if (p.act) {
                o.x = apply_act(o.x, p.act); o.y = apply_act(o.y, p.act);
                o.z = apply_act(o.z, p.act); o.w = apply_act(o.w, p.act);
            }
            *reinterpret_cast<float4*>(drow + col) = o;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (col + e < p.N) {
                    float x = v[j + e] + (crow ? __ldg(crow + col + e) : 0.0f);
                    if (p.bias) x += __ldg(p.bias + col + e);
                    drow[col + e] = p.act ? apply_act(x, p.act) : x;
                }
        }
    }
}

/* The same 32 columns for the 32 rows of a warp at once, through the warp's 4 KiB staging box
 * and one TMA store: lane r writes its row into the box (16-byte pieces XOR-swizzled by the row,
 * the 128-byte swizzle the tensor map describes, so the four-way minimum of bank conflicts),
 * lane 0 hands the box to the copy engine, which writes 32 full 128-byte row segments and
 * clips what lies beyond M or N.  Against per-thread stores (32 rows per instruction, 16 bytes
 * each) this takes the result traffic off the load/store path that the tensor core's operand
 * reads keep busy. */
template <bool CONV, int BOXES>
__device__ __forceinline__ void store32_tma(const float* v, int64_t col_first, int64_t row_first, bool row_ok,
                                            const GemmParams& p, const float* __restrict__ crow, bool c_vec,
                                            uint32_t stg0, uint32_t& box_turn, const CUtensorMap* map, int lane,
                                            int box_x = 0, int box_y = 0, int box_img = 0)
{
    /* with two boxes the store issued before the last one must have been read: its box is reused now */
    if (lane == 0) tma_store_wait_read<BOXES - 1>();
    __syncwarp();
    const uint32_t stg = stg0 + (BOXES == 2 ? (box_turn & 1u) * 4096u : 0u);
    ++box_turn;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const int64_t col = col_first + j;
        float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (crow && row_ok) {
            if (c_vec && col + 3 < p.N) {
                const float4 ci = __ldg(reinterpret_cast<const float4*>(crow + col));
                o.x += ci.x; o.y += ci.y; o.z += ci.z; o.w += ci.w;
            } else {
                if (col < p.N) o.x += __ldg(crow + col);
                if (col + 1 < p.N) o.y += __ldg(crow + col + 1);
                if (col + 2 < p.N) o.z += __ldg(crow + col + 2);
                if (col + 3 < p.N) o.w += __ldg(crow + col + 3);
            }
        }
        if (p.bias) {
            if (col < p.N) o.x += __ldg(p.bias + col);
            if (col + 1 < p.N) o.y += __ldg(p.bias + col + 1);
            if (col + 2 < p.N) o.z += __ldg(p.bias + col + 2);
            if (col + 3 < p.N) o.w += __ldg(p.bias + col + 3);
        }
        if (p.act) {
            o.x = apply_act(o.x, p.act); o.y = apply_act(o.y, p.act);
            o.z = apply_act(o.z, p.act); o.w = apply_act(o.w, p.act);
        }
        const uint32_t dst = stg + (uint32_t)lane * 128u + ((uint32_t)((j >> 2) ^ (lane & 7)) << 4);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" :: "r"(dst), "f"(o.x), "f"(o.y), "f"(o.z), "f"(o.w) : "memory");
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        /* convolution: the warp's 32 tile rows are the pixels (box_x.., box_y..) of one image, x fastest */
        if (CONV) tma_store_4d(map, stg, (int)col_first, box_x, box_y, box_img);
        else      tma_store_2d(map, stg, (int)col_first, (int)row_first);
        tma_store_commit();
    }
}

/* k-blocks of the chunk that starts at k-block kb0 (chunked accumulation).  The first two chunks
 * of a tile are twice as long as the rest: while the epilogue warps still write the previous
 * tile's result they cannot take chunks, and the tensor core can only work two chunks (the two
 * TMEM buffers) into the next tile before it has to wait for them. */
template <int KCH>
__device__ __forceinline__ int chunk_blocks(int kb0)
{
    return kb0 < 4 * KCH ? 2 * KCH : KCH;
}

/* Tile order: groups of 8 tile-rows, column by column inside a group, so that the CTAs
 * running at the same time share A row-panels and B column-panels in L2. */
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int GROUP, int& tm, int& tn)
{
    const int per_group = GROUP * tiles_n;
    const int g = t / per_group;
    const int first_m = g * GROUP;
    const int gsz = min(tiles_m - first_m, GROUP);
    const int r = t - g * per_group;
    tm = first_m + r % gsz;
    tn = r / gsz;
}

/* --------------------------------------------------------------------------------------
 * CTAS   : 1 or 2 CTAs per tile (cta_group)
 * BN     : rows of the B operand (columns of D) loaded per CTA; UMMA N = BN * CTAS
 * NSPLIT : 3 = 3xTF32 (hi and lo parts of both operands), 1 = plain TF32,
 *          2 = the hi * hi product in TF32 and the two cross products a_lo * b and a * b_lo in bf16 (kind::f16 with
 *          bf16 operands, twice the TF32 rate): the stage holds the TF32 hi tile and, in the space of the lo tile,
 *          two bf16 tiles of 64-byte rows (64-byte swizzle); 4 + 4 MMAs per k-block instead of 12,
 *          16 = fp16 operands and fp16 result with fp32 accumulation (kind::f16); a k-block is
 *          then 64 halves, still one 128-byte row, and a k-step 16 halves, still 32 bytes
 * KCH    : 0 = the tensor core accumulates over all of K.  > 0 = chunked accumulation: the
 *          tensor core accumulates KCH k-blocks (KCH * 32 values of K) at a time into one of the
 *          two TMEM buffers, and eight epilogue warps add each finished chunk to a running sum
 *          held in registers with IEEE round-to-nearest fp32 adds, while the tensor core works
 *          on the next chunk in the other buffer.  (The tensor core's own accumulator rounds
 *          toward zero, which biases long sums of same-sign products; short chunks bound it.)
 * ------------------------------------------------------------------------------------ */
template <int CTAS, int BN, int NSPLIT, int KCH = 0>
struct Cfg {
    static constexpr int PARTS = (NSPLIT == 3 || NSPLIT == 2) ? 2 : 1;
    static constexpr int EPI_WARPS = NSPLIT == 16 ? 4 : 8;
    static constexpr int THREADS = KCH ? NUM_THREADS_CHUNKED : NSPLIT == 16 ? NUM_THREADS_F16 : NUM_THREADS;
    /* one 32 x 32 fp32 box (4 KiB, 128-byte swizzled) per epilogue warp for the TMA result stores */
    static constexpr int STAGING1 = NSPLIT == 16 ? 0 : EPI_WARPS * 4096;
    static constexpr int UMMA_M = BM_CTA * CTAS;
    static constexpr int UMMA_N = BN * CTAS;
    static constexpr int A_BYTES = BM_CTA * BK * 4;            /* 16 KiB */
    static constexpr int B_BYTES = BN * BK * 4;
    static constexpr int STAGE_BYTES = PARTS * (A_BYTES + B_BYTES);
    static constexpr int STAGES_RAW = (SMEM_LIMIT - 2048 - STAGING1) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    /* a second box per warp (two result stores in flight) where it fits beside the stages */
    static constexpr int BOXES = (NSPLIT != 16 && SMEM_LIMIT - 2048 - STAGES * STAGE_BYTES >= 2 * STAGING1) ? 2 : 1;
    static constexpr int STAGING = STAGING1 * BOXES;
    static constexpr int TMEM_COLS_RAW = 2 * UMMA_N;
    static constexpr int TMEM_COLS = TMEM_COLS_RAW <= 32 ? 32 : TMEM_COLS_RAW <= 64 ? 64 : TMEM_COLS_RAW <= 128 ? 128
                                   : TMEM_COLS_RAW <= 256 ? 256 : 512;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING + 1024 /* alignment slack */ + 256 /* barriers */;
    static_assert(STAGES >= 2, "need at least two stages");
    static_assert(UMMA_N % 16 == 0 && UMMA_N >= 16 && UMMA_N <= 256, "UMMA N");
    static_assert(TMEM_COLS_RAW <= 512, "two accumulators must fit in TMEM");
};

template <int CTAS, int BN, int NSPLIT, bool CONV, int KCH>
__global__ void __launch_bounds__((Cfg<CTAS, BN, NSPLIT, KCH>::THREADS), 1)
decxb_gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                       const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                       const __grid_constant__ CUtensorMap map_d, const GemmParams p,
                       const __grid_constant__ CUtensorMap map_a_x, const __grid_constant__ CUtensorMap map_b_x)
{
    /* NSPLIT == 2: map_a_lo = bf16(a_lo), map_a_x = bf16(a), map_b_lo = bf16(b_lo), map_b_x = bf16(b); unused otherwise */
    using C = Cfg<CTAS, BN, NSPLIT, KCH>;
    extern __shared__ uint8_t smem_raw[];
    /* 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits 4-9. */
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t staging = smem_base + C::STAGES * C::STAGE_BYTES;      /* 1024-byte aligned */
    const uint32_t bars = staging + C::STAGING;
    auto full_bar   = [&](int s) { return bars + 8u * s; };
    auto empty_bar  = [&](int s) { return bars + 8u * (C::STAGES + s); };
    auto tfull_bar  = [&](int b) { return bars + 8u * (2 * C::STAGES + b); };
    auto tempty_bar = [&](int b) { return bars + 8u * (2 * C::STAGES + 2 + b); };
    const uint32_t tmem_slot = bars + 8u * (2 * C::STAGES + 4);
    auto stage_a = [&](int s, int part) { return smem_base + s * C::STAGE_BYTES + part * C::A_BYTES; };
    auto stage_b = [&](int s, int part) { return smem_base + s * C::STAGE_BYTES + C::PARTS * C::A_BYTES + part * C::B_BYTES; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = CTAS == 2 ? cluster_ctarank() : 0u;
    const bool is_leader = cta_rank == 0;
    const int cluster_id = (int)blockIdx.x / CTAS;
    const int num_clusters = (int)gridDim.x / CTAS;
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a_hi); prefetch_tensormap(&map_b_hi);
        if (NSPLIT == 3 || NSPLIT == 2) { prefetch_tensormap(&map_a_lo); prefetch_tensormap(&map_b_lo); }
        if (NSPLIT == 2) { prefetch_tensormap(&map_a_x); prefetch_tensormap(&map_b_x); }
        if (p.tma_store) prefetch_tensormap(&map_d);
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), C::EPI_WARPS * CTAS); }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc<CTAS>(tmem_slot, C::TMEM_COLS);
        tmem_relinquish<CTAS>();
    }
    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
    /* Programmatic dependent launch: everything above (barriers, tensor memory, descriptor prefetch)
     * may run while the kernel before this one in the stream (the operand split) is still
     * draining; nothing below touches global memory before that kernel has completed. */
    asm volatile("griddepcontrol.wait;" ::: "memory");

    /* Chunked accumulation with 128 running sums per thread: the epilogue warp groups take
     * registers that warp group 0 gives up (168 per thread at launch for 384 threads;
     * 128 * 56 + 256 * 224 = 64512 = 384 * 168).  The host refuses to launch the variant if the
     * kernel was not compiled to 168 registers, so the request can always be met. */
    constexpr bool REALLOC = KCH > 0 && C::UMMA_N / 2 > 64;

    if (KCH ? warp < 4 : warp < 2) {
    if constexpr (REALLOC) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0) {
        /* ------------------------------------------------------------ TMA producer ---- */
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            uint32_t armed = 0, armed_parity = 0;     /* per stage: loads issued at least once / parity of the latest */
            bool alive = true;
            int local_tile = 0;
            for (int t = cluster_id; t < num_tiles && alive; t += num_clusters, ++local_tile) {
                int tm, tn; tile_coords(t, p.tiles_m, p.tiles_n, p.tile_group, tm, tn);
                if (p.wave_counter && is_leader && local_tile > 0 && !align_wave(p, local_tile, num_clusters, num_tiles, t)) { alive = false; break; }
                if (p.trace && is_leader && local_tile < p.trace_tiles)
                    p.trace[(size_t)cluster_id * p.trace_tiles + local_tile] = globaltimer_ns();
                const int row_a = tm * C::UMMA_M + (int)cta_rank * BM_CTA;
                int row_b = tn * C::UMMA_N + (int)cta_rank * BN;
                if (!CONV && p.tiles_m_per) row_b += (tm / p.tiles_m_per) * (int)p.b_batch_rows;   /* matrix of the batch */
                /* convolution: this CTA's patches of output pixels (up to four boxes of 128 / nbox pixels each,
                 * consecutive in the launch's patch order, possibly of different images) */
                int s_img[4] = {0, 0, 0, 0}, s_px[4] = {0, 0, 0, 0}, s_py[4] = {0, 0, 0, 0};
                if (CONV) {
                    const int per_img = p.tiles_x * p.tiles_y;
                    const long long s0 = ((long long)tm * CTAS + (long long)cta_rank) * p.nbox;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const long long sj = s0 + j;
                        const int im = (int)(sj / per_img), r = (int)(sj - (long long)im * per_img);
                        s_img[j] = im; s_py[j] = (r / p.tiles_x) * p.by; s_px[j] = (r % p.tiles_x) * p.bx;
                    }
                }
                const uint32_t sub_bytes = CONV ? (uint32_t)(BM_CTA / p.nbox) * 128u : 0u;   /* rows of one box x 128 bytes */
                int tap = 0, cb = 0;       /* convolution: filter tap and channel block of this k-block */
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if (!wait_bounded(empty_bar(stage), phase ^ 1u, p, 100 + stage, t)) { alive = false; break; }
                    const int kx = kb * (NSPLIT == 16 ? 64 : BK);       /* elements per 128-byte k-block */
                    const int ky_t = CONV ? tap / p.kw : 0;
                    const int cc = cb * BK, dx = (tap - ky_t * p.kw) + p.off_x, dy = ky_t + p.off_y;
                    if (CTAS == 1) {
                        const uint32_t fb = full_bar(stage);
                        mbar_arrive_expect_tx(fb, C::STAGE_BYTES);
                        if (CONV) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (j < p.nbox) {
                                    tma_load_4d(stage_a(stage, 0) + j * sub_bytes, &map_a_hi, fb, cc, s_px[j] + dx, s_py[j] + dy, s_img[j]);
                                    if (NSPLIT == 3)
                                        tma_load_4d(stage_a(stage, 1) + j * sub_bytes, &map_a_lo, fb, cc, s_px[j] + dx, s_py[j] + dy, s_img[j]);
                                }
                        } else {
                            tma_load_2d(stage_a(stage, 0), &map_a_hi, fb, kx, row_a);
                            if (NSPLIT == 3) tma_load_2d(stage_a(stage, 1), &map_a_lo, fb, kx, row_a);
                            if (NSPLIT == 2) {
                                tma_load_2d(stage_a(stage, 1), &map_a_lo, fb, kx, row_a);
                                tma_load_2d(stage_a(stage, 1) + C::A_BYTES / 2, &map_a_x, fb, kx, row_a);
                            }
                        }
                        tma_load_2d(stage_b(stage, 0), &map_b_hi, fb, kx, row_b);
                        if (NSPLIT == 3) tma_load_2d(stage_b(stage, 1), &map_b_lo, fb, kx, row_b);
                        if (NSPLIT == 2) {
                            tma_load_2d(stage_b(stage, 1), &map_b_x, fb, kx, row_b);
                            tma_load_2d(stage_b(stage, 1) + C::B_BYTES / 2, &map_b_lo, fb, kx, row_b);
                        }
                    } else {
                        /* Both CTAs' bytes are counted on the leader's barrier. */
                        if (is_leader) mbar_arrive_expect_tx(full_bar(stage), 2 * C::STAGE_BYTES);
                        const uint32_t fb = mapa(full_bar(stage), 0);
                        if (CONV) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (j < p.nbox) {
                                    tma_load_4d_pair(stage_a(stage, 0) + j * sub_bytes, &map_a_hi, fb, cc, s_px[j] + dx, s_py[j] + dy, s_img[j]);
                                    if (NSPLIT == 3)
                                        tma_load_4d_pair(stage_a(stage, 1) + j * sub_bytes, &map_a_lo, fb, cc, s_px[j] + dx, s_py[j] + dy, s_img[j]);
                                }
                        } else {
                            tma_load_2d_pair(stage_a(stage, 0), &map_a_hi, fb, kx, row_a);
                            if (NSPLIT == 3) tma_load_2d_pair(stage_a(stage, 1), &map_a_lo, fb, kx, row_a);
                            if (NSPLIT == 2) {
                                tma_load_2d_pair(stage_a(stage, 1), &map_a_lo, fb, kx, row_a);
                                tma_load_2d_pair(stage_a(stage, 1) + C::A_BYTES / 2, &map_a_x, fb, kx, row_a);
                            }
                        }
                        tma_load_2d_pair(stage_b(stage, 0), &map_b_hi, fb, kx, row_b);
                        if (NSPLIT == 3) tma_load_2d_pair(stage_b(stage, 1), &map_b_lo, fb, kx, row_b);
                        if (NSPLIT == 2) {
                            tma_load_2d_pair(stage_b(stage, 1), &map_b_x, fb, kx, row_b);
                            tma_load_2d_pair(stage_b(stage, 1) + C::B_BYTES / 2, &map_b_lo, fb, kx, row_b);
                        }
                    }
                    armed |= 1u << stage;
                    armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    if (CONV && ++cb == p.cblocks) { cb = 0; ++tap; }
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            /* A wait gave up somewhere: the MMA issuer no longer consumes the stages, but copies this
             * lane issued may still be on their way into shared memory.  Wait for them (again with a
             * limit) before the block lets go of it.  The barriers are the leader CTA's and count
             * both CTAs' bytes, so the leader's wait covers its peer, which leaves only after the
             * cluster barrier of the teardown. */
            if (is_leader && *reinterpret_cast<volatile int*>(&p.status->code) != 0) {
                for (int s2 = 0; s2 < C::STAGES; ++s2) {
                    if (!((armed >> s2) & 1u)) continue;
                    for (int tries = 0; tries < 2048 && !mbar_try_wait(full_bar(s2), (armed_parity >> s2) & 1u); ++tries)
                        __nanosleep(64);
                }
            }
        }
    } else if (warp == 1) {
        /* ------------------------------------------------------------ MMA issuer ------ */
        if (is_leader && lane == 0) {
            constexpr uint32_t idesc = NSPLIT == 16 ? make_idesc_f16(C::UMMA_M, C::UMMA_N) : make_idesc(C::UMMA_M, C::UMMA_N);
            int stage = 0; uint32_t phase = 0;
            int unit = 0;              /* accumulation units so far: tiles, or (tile, chunk) pairs */
            bool alive = true;
            for (int t = cluster_id; t < num_tiles && alive; t += num_clusters) {
                for (int kb0 = 0, per_unit; kb0 < p.num_kb && alive; kb0 += per_unit, ++unit) {
                    per_unit = KCH ? chunk_blocks<KCH ? KCH : 1>(kb0) : p.num_kb;
                    const int acc = unit & 1;
                    const uint32_t acc_phase = (uint32_t)(unit >> 1) & 1u;
                    if (!wait_bounded(tempty_bar(acc), acc_phase ^ 1u, p, 200 + acc, t)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (uint32_t)(acc * C::UMMA_N);
                    const int kb1 = min(kb0 + per_unit, p.num_kb);
                    for (int kb = kb0; kb < kb1; ++kb) {
                        if (!wait_bounded(full_bar(stage), phase, p, 300 + stage, t)) { alive = false; break; }
                        tc_fence_after();
                        const uint64_t da_hi = make_smem_desc(stage_a(stage, 0));
                        const uint64_t db_hi = make_smem_desc(stage_b(stage, 0));
                        const uint64_t da_lo = make_smem_desc(stage_a(stage, C::PARTS - 1));
                        const uint64_t db_lo = make_smem_desc(stage_b(stage, C::PARTS - 1));
                        if constexpr (NSPLIT == 2) {
                            /* per 16 values of K: a_lo * b and a * b_lo in bf16 (one MMA each, 32 bytes of a 64-byte row),
                             * then hi * hi in TF32 (two MMAs of 8); the small terms first */
                            constexpr uint32_t idesc_bf = make_idesc_bf16(C::UMMA_M, C::UMMA_N);
                            const uint64_t da_lb = make_smem_desc_sw64(stage_a(stage, 1));
                            const uint64_t da_ab = make_smem_desc_sw64(stage_a(stage, 1) + C::A_BYTES / 2);
                            const uint64_t db_bb = make_smem_desc_sw64(stage_b(stage, 1));
                            const uint64_t db_lb = make_smem_desc_sw64(stage_b(stage, 1) + C::B_BYTES / 2);
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const uint32_t first = ((kb - kb0) | h) != 0 ? 1u : 0u;
                                umma_f16<CTAS>(tmem_d, da_lb + (uint64_t)(2 * h), db_bb + (uint64_t)(2 * h), idesc_bf, first);
                                umma_f16<CTAS>(tmem_d, da_ab + (uint64_t)(2 * h), db_lb + (uint64_t)(2 * h), idesc_bf, 1u);
                                umma_tf32<CTAS>(tmem_d, da_hi + (uint64_t)(4 * h), db_hi + (uint64_t)(4 * h), idesc, 1u);
                                umma_tf32<CTAS>(tmem_d, da_hi + (uint64_t)(4 * h + 2), db_hi + (uint64_t)(4 * h + 2), idesc, 1u);
                            }
                        } else {
#pragma unroll
                        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                            /* advance 8 floats = 32 bytes inside the 128-byte swizzled row */
                            const uint64_t koff = (uint64_t)((kk * UMMA_K * 4) >> 4);
                            const uint32_t first = ((kb - kb0) | kk) != 0 ? 1u : 0u;
                            if (NSPLIT == 3) {
                                /* a_hi feeds two consecutive MMAs: the first keeps it in the tensor core's
                                 * collector buffer, the second takes it from there (A_COLLECTOR) */
                                umma_tf32<CTAS>(tmem_d, da_lo + koff, db_hi + koff, idesc, first);
                                umma_tf32<CTAS, A_COLLECTOR ? 1 : 0>(tmem_d, da_hi + koff, db_lo + koff, idesc, 1u);
                                umma_tf32<CTAS, A_COLLECTOR ? 2 : 0>(tmem_d, da_hi + koff, db_hi + koff, idesc, 1u);
                            } else if (NSPLIT == 16) {
                                umma_f16<CTAS>(tmem_d, da_hi + koff, db_hi + koff, idesc, first);
                            } else {
                                umma_tf32<CTAS>(tmem_d, da_hi + koff, db_hi + koff, idesc, first);
                            }
                        }
                        }
                        umma_commit<CTAS>(empty_bar(stage));     /* stage reusable once these MMAs have read it */
                        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                    }
                    if (alive) umma_commit<CTAS>(tfull_bar(acc)); /* accumulator (chunk) complete */
                }
            }
        }
    }
    } else {
        /* ------------------------------------------------------------ epilogue -------- */
        if constexpr (REALLOC) asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        const int q = warp & 3;                   /* TMEM lane quarter this warp may read */
        const bool d_vec = ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) && (p.ldd % 4 == 0) && (p.d_batch_stride % 4 == 0) &&
                           (p.dst_img_stride % 4 == 0);
        const bool c_vec = p.C && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && (p.ldc % 4 == 0) && (p.c_batch_stride % 4 == 0);
        int unit = 0;                             /* same count as the MMA issuer's */
        bool alive = true;
        const int eh = KCH ? (warp - 4) >> 2 : C::EPI_WARPS == 8 ? (warp - 2) >> 2 : 0;   /* column half of this warp */
        const uint32_t stg = staging + (uint32_t)(KCH ? warp - 4 : warp - 2) * (4096u * C::BOXES);   /* this warp's TMA store box(es) */
        uint32_t box_turn = 0;
        for (int t = cluster_id; t < num_tiles && alive; t += num_clusters) {
            int tm, tn; tile_coords(t, p.tiles_m, p.tiles_n, p.tile_group, tm, tn);
            const int bidx = (!CONV && p.tiles_m_per) ? tm / p.tiles_m_per : 0;
            int64_t row = (int64_t)(tm - bidx * p.tiles_m_per) * C::UMMA_M + (int64_t)cta_rank * BM_CTA + q * 32 + lane;
            bool row_ok = row < p.M;
            const int64_t col0 = (int64_t)tn * C::UMMA_N;
            const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
            float* __restrict__ drow = p.D + bidx * p.d_batch_stride + row * p.ldd;
            int box_x = 0, box_y = 0, box_img = 0;    /* convolution: first pixel of the warp's 32 tile rows */
            if (CONV) {
                /* tile row i lies in the CTA's patch i / (bx * by), at pixel (li % bx, li / bx) of it, li = i % (bx * by);
                 * a warp's 32 rows always lie in one patch (a patch has at least 32 pixels) */
                const int per_img = p.tiles_x * p.tiles_y, rpb = BM_CTA / p.nbox;
                const int i0 = q * 32, j = i0 / rpb, li0 = i0 - j * rpb;
                const long long sj = ((long long)tm * CTAS + (long long)cta_rank) * p.nbox + j;
                const int img = (int)(sj / per_img), r = (int)(sj - (long long)img * per_img);
                const int py0 = (r / p.tiles_x) * p.by, px0 = (r % p.tiles_x) * p.bx;
                const int li = li0 + lane;
                const int y = py0 + li / p.bx;
                const int x = px0 + li % p.bx;
                row_ok = (x < p.eq_w) && (y < p.out_h) && (img < p.batch);
                drow = p.D + (int64_t)img * p.dst_img_stride + ((int64_t)y * p.eq_w + x) * p.ldd;
                box_x = px0 + li0 % p.bx; box_y = py0 + li0 / p.bx; box_img = img;
            }
            const float* __restrict__ crow = (p.C && !CONV) ? p.C + bidx * p.c_batch_stride + row * p.ldc : nullptr;
            const bool vec = d_vec && (!crow || c_vec);
            const int64_t row_first = row - lane;     /* first of the warp's 32 rows (TMA store path: plain GEMM only) */
            if constexpr (KCH > 0) {
                /* chunked accumulation: this warp owns NCW columns of its 32 rows */
                constexpr int NCW = C::UMMA_N / 2;
                static_assert(NCW % 32 == 0, "column half must be whole 32-column groups");
                constexpr int DRAIN = NCW < 64 ? NCW : 64;   /* columns fetched per round */
                float sum[NCW];
#pragma unroll
                for (int c = 0; c < NCW; ++c) sum[c] = 0.0f;
                for (int kb0 = 0; kb0 < p.num_kb; kb0 += chunk_blocks<KCH>(kb0), ++unit) {
                    const int acc = unit & 1;
                    const uint32_t acc_phase = (uint32_t)(unit >> 1) & 1u;
                    if (!wait_bounded(tfull_bar(acc), acc_phase, p, 400 + acc, t)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t taddr = tlane + (uint32_t)(acc * C::UMMA_N + eh * NCW);
#pragma unroll
                    for (int c = 0; c < NCW; c += DRAIN) {
                        /* the loads of one round are in flight together; one wait per round */
                        float v[DRAIN];
#pragma unroll
                        for (int g = 0; g < DRAIN; g += 32) tmem_ld_32x32(taddr + (uint32_t)(c + g), v + g);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < DRAIN; ++j) sum[c + j] = __fadd_rn(sum[c + j], v[j]);
                    }
                    /* chunk taken: hand the buffer back to the MMA issuer (in the leader CTA) */
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (CTAS == 1) mbar_arrive_cluster(tempty_bar(acc));
                        else           mbar_arrive_cluster(mapa(tempty_bar(acc), 0));
                    }
                }
                if (!alive) break;
                if (p.tma_store) {
#pragma unroll
                    for (int c = 0; c < NCW; c += 32)
                        if (col0 + eh * NCW + c < p.N)
                            store32_tma<CONV, C::BOXES>(sum + c, col0 + eh * NCW + c, row_first, row_ok, p, crow, c_vec, stg, box_turn,
                                                        &map_d, lane, box_x, box_y, box_img);
                } else if (row_ok) {
#pragma unroll
                    for (int c = 0; c < NCW; c += 32) {
                        if (col0 + eh * NCW + c < p.N) store32_f32(sum + c, col0 + eh * NCW + c, p, drow, crow, vec);
                        asm volatile("" ::: "memory");   /* keep the next group's loads behind these stores */
                    }
                }
            } else {
            const int acc = unit & 1;
            const uint32_t acc_phase = (uint32_t)(unit >> 1) & 1u;
            ++unit;
            if (!wait_bounded(tfull_bar(acc), acc_phase, p, 400 + acc, t)) { alive = false; break; }
            tc_fence_after();
            const uint32_t taddr = tlane + (uint32_t)(acc * C::UMMA_N);
            constexpr int COLS_PER_WARP = C::UMMA_N / (C::EPI_WARPS / 4);
            static_assert(COLS_PER_WARP % 32 == 0, "whole 32-column groups per epilogue warp");
#pragma unroll 1
            for (int c = eh * COLS_PER_WARP; c < (eh + 1) * COLS_PER_WARP; c += 32) {
                if (col0 + c >= p.N) break;           /* warp-uniform */
                float v[32];
                tmem_ld_32x32(taddr + (uint32_t)c, v);
                tmem_ld_wait();
                if (NSPLIT == 16) {
                    /* fp16 result (and addend): 8 halves = 16 bytes per store */
                    if (row_ok) {
                        __half* __restrict__ hrow = reinterpret_cast<__half*>(p.D) + row * p.ldd;
                        const __half* __restrict__ hc = p.C ? reinterpret_cast<const __half*>(p.C) + row * p.ldc : nullptr;
                        const bool hd_vec = ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) && (p.ldd % 8 == 0);
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            const int64_t col = col0 + c + j;
                            float x[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                x[e] = v[j + e] + ((hc && col + e < p.N) ? __half2float(hc[col + e]) : 0.0f);
                                if (p.act) x[e] = apply_act(x[e], p.act);
                            }
                            if (col + 7 < p.N && hd_vec) {
                                uint4 o;
                                __half2 h0 = __floats2half2_rn(x[0], x[1]), h1 = __floats2half2_rn(x[2], x[3]);
                                __half2 h2 = __floats2half2_rn(x[4], x[5]), h3 = __floats2half2_rn(x[6], x[7]);
                                o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
                                o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
                                *reinterpret_cast<uint4*>(hrow + col) = o;
                            } else {
#pragma unroll
                                for (int e = 0; e < 8; ++e) if (col + e < p.N) hrow[col + e] = __float2half_rn(x[e]);
                            }
                        }
                    }
                } else if (p.tma_store) {
                    store32_tma<CONV, C::BOXES>(v, col0 + c, row_first, row_ok, p, crow, c_vec, stg, box_turn, &map_d, lane,
                                                box_x, box_y, box_img);
                } else if (row_ok) {
                    store32_f32(v, col0 + c, p, drow, crow, vec);
                }
            }
            /* accumulator drained: hand it back to the MMA issuer (in the leader CTA) */
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CTAS == 1) mbar_arrive_cluster(tempty_bar(acc));
                else           mbar_arrive_cluster(mapa(tempty_bar(acc), 0));
            }
            }   /* whole-K accumulation */
        }
        if (p.tma_store && lane == 0) tma_store_wait_all();   /* the boxes stay valid until the copy engine is done */
    }

    /* ---------------------------------------------------------------- teardown -------- */
    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<CTAS>(tmem_base, C::TMEM_COLS);
    }
}

/* Self-test of the bounded wait: one thread waits on an mbarrier that nothing will ever arrive
 * on.  The wait must give up after the limit, record itself in the status word and let the
 * kernel return normally. */
__global__ void decxb_wait_probe_kernel(const GemmParams p)
{
    __shared__ __align__(8) uint64_t bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) { mbar_init(b, 1); fence_barrier_init(); }
    __syncthreads();
    if (threadIdx.x == 0) (void)wait_bounded(b, 0u, p, 900, 0);
    __syncthreads();
}

/* ------------------------------------------------------------------ host side -------- */
PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn()
{
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
    });
    return fn;
}

/* rows x K fp32 array with K contiguous and a row pitch of `ld` floats; box = 32 floats x box_rows. */
/* rows x K fp16 array with K contiguous and a row pitch of `ld` halves; box = 64 halves x box_rows. */
int make_map_f16(decxb_ctx* ctx, CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows)
{
    auto fn = get_encode_fn();
    if (!fn) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld % 8))
        return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "TMA fp16 operand must be 16-byte aligned with a pitch that is a multiple of 8 halves");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled (fp16) failed: " + std::to_string((int)r));
    return DECXB_OK;
}

int make_map(decxb_ctx* ctx, CUtensorMap* map, const float* base, int64_t rows, int64_t K, int64_t ld, int box_rows)
{
    auto fn = get_encode_fn();
    if (!fn) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld % 4))
        return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "TMA operand must be 16-byte aligned with a pitch that is a multiple of 4 floats");
    /* A repeated call (same arrays, same shape: a benchmark step, a layer applied again) finds its five
     * descriptors in a small per-context table instead of encoding them again. */
    const decxb_map_key key = {base, rows, K, ld, box_rows};
    {
        std::lock_guard<std::mutex> lock(ctx->map_mtx);
        for (auto& e : ctx->map_cache)
            if (e.used && e.key == key) { *map = e.map; e.stamp = ++ctx->map_clock; return DECXB_OK; }
    }
    struct Store {
        decxb_ctx* c; const decxb_map_key& k; CUtensorMap* m; bool ok = false;
        ~Store()
        {
            if (!ok) return;
            std::lock_guard<std::mutex> lock(c->map_mtx);
            decxb_map_entry* victim = &c->map_cache[0];
            for (auto& e : c->map_cache) { if (!e.used) { victim = &e; break; } if (e.stamp < victim->stamp) victim = &e; }
            victim->used = true; victim->key = k; victim->map = *m; victim->stamp = ++c->map_clock;
        }
    } store{ctx, key, map};
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
    store.ok = true;
    return DECXB_OK;
}

/* Source tensor [nb][H][wp][dp] as a 4-D map (channel, x, y, image); box = 32 x bx x by x 1. */
int make_map_conv(decxb_ctx* ctx, CUtensorMap* map, const float* base, int64_t dp, int64_t wp, int64_t H, int64_t nb,
                  int64_t img_stride, int bx, int by)
{
    auto fn = get_encode_fn();
    if (!fn) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (dp % 4) || (img_stride % 4))
        return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "TMA tensor operand must be 16-byte aligned");
    cuuint64_t dims[4] = {(cuuint64_t)dp, (cuuint64_t)wp, (cuuint64_t)H, (cuuint64_t)nb};
    cuuint64_t strides[3] = {(cuuint64_t)dp * 4, (cuuint64_t)wp * dp * 4, (cuuint64_t)img_stride * 4};
    cuuint32_t box[4] = {(cuuint32_t)BK, (cuuint32_t)bx, (cuuint32_t)by, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed: " + std::to_string((int)r));
    return DECXB_OK;
}

/* Destination tensor [nb][out_h][eq_w][Np] as a 4-D map (channel, x, y, image) for the result
 * stores; box = 32 channels x (bx_s x by_s = 32 pixels) x 1 image, 128-byte swizzle. */
int make_map_conv_dst(decxb_ctx* ctx, CUtensorMap* map, const float* base, int64_t Np, int64_t eq_w, int64_t out_h, int64_t nb,
                      int64_t img_stride, int bx)
{
    auto fn = get_encode_fn();
    if (!fn) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
    const int bxs = bx < 32 ? bx : 32;
    cuuint64_t dims[4] = {(cuuint64_t)Np, (cuuint64_t)eq_w, (cuuint64_t)out_h, (cuuint64_t)nb};
    cuuint64_t strides[3] = {(cuuint64_t)Np * 4, (cuuint64_t)eq_w * Np * 4, (cuuint64_t)img_stride * 4};
    cuuint32_t box[4] = {32, (cuuint32_t)bxs, (cuuint32_t)(32 / bxs), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled (4-D result) failed: " + std::to_string((int)r));
    return DECXB_OK;
}

/* The chunked kernels whose epilogue warps hold 128 running sums move registers between warp
 * groups (setmaxnreg) and count on exactly 168 registers per thread at launch.  Whether the
 * toolkit compiled them that way is asked once per device; when it did not, the callers take
 * the 128 x 128 tile, whose chunked kernel needs no register hand-over and gives the same bits. */
template <int CTAS, int BN, bool CONV, int NSPLIT = 3>
bool chunked_regs_ok(decxb_ctx* ctx)
{
    using C = Cfg<CTAS, BN, NSPLIT, KCHUNK>;
    if (C::UMMA_N / 2 <= 64) return true;
    static std::atomic<int> regs[DECXB_MAX_DEVICES];
    int r = regs[ctx->device].load();
    if (r == 0) {
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, decxb_gemm_tf32_kernel<CTAS, BN, NSPLIT, CONV, KCHUNK>) != cudaSuccess) { cudaGetLastError(); return false; }
        r = fa.numRegs;
        regs[ctx->device].store(r);
    }
    if (r != 168)
        decxb_set_error(ctx, "note: chunked " + std::to_string(C::UMMA_M) + "x" + std::to_string(C::UMMA_N) + " kernel compiled to " +
                             std::to_string(r) + " registers (168 expected); the 128x128 tile is used instead");
    return r == 168;
}

template <int CTAS, int BN, int NSPLIT, bool CONV, int KCH = 0>
int launch_kernel(decxb_ctx* ctx, const CUtensorMap& ma_hi, const CUtensorMap& ma_lo, const CUtensorMap& mb_hi,
                  const CUtensorMap& mb_lo, const CUtensorMap& md, const GemmParams& p, cudaStream_t s,
                  const CUtensorMap* ma_x_or_null = nullptr, const CUtensorMap* mb_x_or_null = nullptr)
{
    const CUtensorMap& ma_x = ma_x_or_null ? *ma_x_or_null : ma_hi;
    const CUtensorMap& mb_x = mb_x_or_null ? *mb_x_or_null : mb_hi;
    using C = Cfg<CTAS, BN, NSPLIT, KCH>;
    auto kernel = decxb_gemm_tf32_kernel<CTAS, BN, NSPLIT, CONV, KCH>;
    static std::once_flag once[DECXB_MAX_DEVICES];
    static cudaError_t attr_err[DECXB_MAX_DEVICES];
    const int dev = ctx->device;           /* decxb_init refuses indices >= DECXB_MAX_DEVICES */
    std::call_once(once[dev], [&] {
        attr_err[dev] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    });
    if (attr_err[dev] != cudaSuccess)
        return decxb_fail(ctx, DECXB_ERR_CUDA, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(attr_err[dev]));
    /* never launch a register-moving kernel whose register count does not add up: its epilogue would wait forever */
    if constexpr (KCH > 0 && (NSPLIT == 3 || NSPLIT == 2)) {
        if (!chunked_regs_ok<CTAS, BN, CONV, NSPLIT>(ctx))
            return decxb_fail(ctx, DECXB_ERR_CUDA, "chunked GEMM kernel was not compiled to 168 registers");
    }
    const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
    int64_t clusters = (ctx->sm_count - ctx->reserved_sms) / CTAS;
    if (clusters > tiles) clusters = tiles;
    if (clusters < 1) clusters = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(clusters * CTAS), 1, 1);
    cfg.blockDim = dim3(C::THREADS, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 2;
    GemmParams pp = p;
    pp.tile_group = ctx->tile_group > 0 ? ctx->tile_group : 8;
    pp.trace = ctx->trace; pp.trace_tiles = ctx->trace_tiles;
    /* Several waves of a long-K product: keep the block pairs of a wave aligned (align_wave).  Such a launch is
     * cooperative (all blocks resident together); if the device refuses that, the launch is repeated without. */
    const bool want_align = !CONV && ctx->wave_align && ctx->wave_counters && p.tiles_m_per == 0 && tiles >= 2 * clusters &&
                            p.num_kb >= 32;   /* 32 k-blocks: K >= 1024 floats */
    /* Beside a transfer kernel (SMs left to it) the launch stays a plain one: a cooperative launch might be held back
     * until the transfer's blocks have gone.  The waits are then met as soon as all blocks have been placed. */
    const bool cooperative = ctx->wave_align == 1 && ctx->reserved_sms == 0;
    if (want_align) {
        unsigned long long* counter = nullptr; unsigned long long base = 0;
        if (decxb_wave_slot(ctx, s, (unsigned long long)(tiles - clusters), &counter, &base)) {
            pp.wave_counter = counter; pp.wave_base = base;
            attr[1].id = cudaLaunchAttributeCooperative;
            attr[1].val.cooperative = cooperative ? 1 : 0;
            cudaError_t e;
            {
                decxb_launch_scope scope(ctx, s, DECXB_K_GEMM);
                e = cudaLaunchKernelEx(&cfg, kernel, ma_hi, ma_lo, mb_hi, mb_lo, md, pp, ma_x, mb_x);
            }
            if (e == cudaSuccess) return DECXB_OK;
            cudaGetLastError();
            ctx->launches--;                                                        /* that one did not happen */
            decxb_wave_unslot(ctx, s, (unsigned long long)(tiles - clusters));     /* nothing was counted */
            ctx->wave_align = 0;                                                    /* not on this device: stop asking */
            pp.wave_counter = nullptr; pp.wave_base = 0;
        }
    }
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    {
        decxb_launch_scope scope(ctx, s, DECXB_K_GEMM);
        DECXB_CUDA_TRY(ctx, cudaLaunchKernelEx(&cfg, kernel, ma_hi, ma_lo, mb_hi, mb_lo, md, pp, ma_x, mb_x));
    }
    return DECXB_OK;
}

template <int CTAS, int BN, int NSPLIT, int KCH = 0>
int launch_conv_cfg(decxb_ctx* ctx, const decxb_conv_gemm_args& a, cudaStream_t s)
{
    using C = Cfg<CTAS, BN, NSPLIT>;
    /* A CTA's 128 tile rows are nbox patches of bx x by output pixels (one TMA box each): the choice that covers
     * the image with the fewest wasted pixels (56 x 56 cannot be tiled by 128-pixel rectangles with power-of-two
     * sides, 8 x 8 patches tile it exactly), fewer boxes on a tie. */
    int best_bx = 128, best_nbox = 1; int64_t best_area = -1;
    for (int nbox = 1; nbox <= 4; nbox <<= 1) {
        const int P = 128 / nbox;
        for (int bx = P; bx >= 1; bx >>= 1) {
            const int by = P / bx;
            const int64_t area = decxb_ceil_to(a.eq_w, bx) * decxb_ceil_to(a.out_h, by);
            if (best_area < 0 || area < best_area) { best_area = area; best_bx = bx; best_nbox = nbox; }
        }
    }
    const int nbox = best_nbox, bx = best_bx, by = 128 / nbox / best_bx;
    const int64_t dp = a.dp, cblocks = decxb_ceil_div(dp, BK);
    CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
    int rc;
    if ((rc = make_map_conv(ctx, &ma_hi, a.src_hi, dp, a.wp, a.H, a.batch, a.src_img_stride, bx, by))) return rc;
    if ((rc = make_map(ctx, &mb_hi, a.k_hi, a.k_rows, a.k_cols, a.ldk, BN))) return rc;
    if (NSPLIT == 3) {
        if ((rc = make_map_conv(ctx, &ma_lo, a.src_lo, dp, a.wp, a.H, a.batch, a.src_img_stride, bx, by))) return rc;
        if ((rc = make_map(ctx, &mb_lo, a.k_lo, a.k_rows, a.k_cols, a.ldk, BN))) return rc;
    } else { ma_lo = ma_hi; mb_lo = mb_hi; }
    GemmParams p = {};
    p.bx = bx; p.by = by; p.nbox = nbox; p.batch = (int)a.batch;
    p.tiles_x = (int)decxb_ceil_div(a.eq_w, bx);
    p.tiles_y = (int)decxb_ceil_div(a.out_h, by);
    p.out_h = (int)a.out_h; p.eq_w = (int)a.eq_w; p.kw = (int)a.kW; p.off_x = a.off_x; p.off_y = a.off_y;
    p.cblocks = (int)cblocks;
    p.dst_img_stride = a.dst_img_stride;
    const int64_t patches = (int64_t)a.batch * p.tiles_x * p.tiles_y;
    const int64_t tiles_m = decxb_ceil_div(patches, (int64_t)nbox * CTAS);
    p.M = tiles_m * C::UMMA_M;                                     /* rows of the tiled problem; real bounds are per pixel */
    p.N = a.Np; p.K = a.k_cols;
    p.C = nullptr; p.ldc = 0; p.D = a.dst; p.ldd = a.Np;
    p.bias = a.bias; p.act = a.act;
    if (tiles_m > 0x7fffffffLL) return decxb_fail(ctx, DECXB_ERR_TOO_LARGE, "convolution tiles");
    p.tiles_m = (int)tiles_m;
    p.tiles_n = (int)decxb_ceil_div(a.Np, C::UMMA_N);
    p.num_kb = (int)(a.kW * a.kH * cblocks);
    p.wait_limit_ns = ctx->wait_limit_ns;
    p.status = ctx->d_status;
    /* result stores through the copy engine when the destination can be described to it */
    CUtensorMap md = ma_hi;
    if ((reinterpret_cast<uintptr_t>(a.dst) & 15) == 0 && a.Np % 4 == 0 && a.dst_img_stride % 4 == 0) {
        if ((rc = make_map_conv_dst(ctx, &md, a.dst, a.Np, a.eq_w, a.out_h, a.batch, a.dst_img_stride, bx))) return rc;
        p.tma_store = 1;
    }
    return launch_kernel<CTAS, BN, NSPLIT, true, KCH>(ctx, ma_hi, ma_lo, mb_hi, mb_lo, md, p, s);
}

/* rows x K bf16 array with K contiguous and a row pitch of `ld` values; box = 32 values (64 bytes) x box_rows, 64-byte swizzle. */
int make_map_bf16(decxb_ctx* ctx, CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows)
{
    auto fn = get_encode_fn();
    if (!fn) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld % 8))
        return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "TMA bf16 operand must be 16-byte aligned with a pitch that is a multiple of 8 values");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled (bf16) failed: " + std::to_string((int)r));
    return DECXB_OK;
}

template <int CTAS, int BN, int NSPLIT, int KCH = 0>
int launch_cfg(decxb_ctx* ctx, const decxb_gemm_args& a, cudaStream_t s)
{
    using C = Cfg<CTAS, BN, NSPLIT>;
    CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo, ma_x, mb_x;
    int rc;
    const int64_t a_rows = a.nbatch > 1 ? a.m_pad * a.nbatch : a.M;
    const int64_t b_rows = a.nbatch > 1 ? a.n_pad * a.nbatch : a.b_rows;
    if ((rc = make_map(ctx, &ma_hi, a.a_hi, a_rows, a.K, a.lda, BM_CTA))) return rc;
    if ((rc = make_map(ctx, &mb_hi, a.b_hi, b_rows, a.K, a.ldb, BN))) return rc;
    if (NSPLIT == 3) {
        if ((rc = make_map(ctx, &ma_lo, a.a_lo, a_rows, a.K, a.lda, BM_CTA))) return rc;
        if ((rc = make_map(ctx, &mb_lo, a.b_lo, b_rows, a.K, a.ldb, BN))) return rc;
    } else if (NSPLIT == 2) {
        if ((rc = make_map_bf16(ctx, &ma_lo, a.a_lo16, a_rows, a.K, a.ld16, BM_CTA))) return rc;
        if ((rc = make_map_bf16(ctx, &ma_x, a.a_16, a_rows, a.K, a.ld16, BM_CTA))) return rc;
        if ((rc = make_map_bf16(ctx, &mb_lo, a.b_lo16, b_rows, a.K, a.ld16, BN))) return rc;
        if ((rc = make_map_bf16(ctx, &mb_x, a.b_16, b_rows, a.K, a.ld16, BN))) return rc;
    } else { ma_lo = ma_hi; mb_lo = mb_hi; }

    GemmParams p = {};
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.C = a.C; p.ldc = a.ldc; p.D = a.D; p.ldd = a.ldd;
    p.bias = a.bias; p.act = a.act;
    p.tiles_m = (int)decxb_ceil_div(a.M, C::UMMA_M);
    p.tiles_n = (int)decxb_ceil_div(a.N, C::UMMA_N);
    if (a.nbatch > 1) {
        /* stacked operands: every matrix occupies whole tiles (a.m_pad rows of A, a.n_pad rows of B) */
        if (a.m_pad % C::UMMA_M || a.n_pad % C::UMMA_N) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "batched operands not padded to the tile");
        p.tiles_m_per = (int)(a.m_pad / C::UMMA_M);
        if ((int64_t)p.tiles_m_per * a.nbatch > 0x7fffffffLL) return decxb_fail(ctx, DECXB_ERR_TOO_LARGE, "batched tiles");
        p.tiles_m = p.tiles_m_per * (int)a.nbatch;
        p.b_batch_rows = a.n_pad; p.d_batch_stride = a.d_batch_stride; p.c_batch_stride = a.c_batch_stride;
    }
    p.num_kb = (int)decxb_ceil_div(a.K, BK);
    p.wait_limit_ns = ctx->wait_limit_ns;
    p.status = ctx->d_status;
    /* results through TMA stores when the result array can be described to the copy engine
     * (16-byte aligned base and pitch); batched launches and odd layouts store from the threads */
    /* N must be a multiple of 4 as well: the copy engine clips a store at the tensor's edge in whole
     * 16-byte pieces, so a ragged N would have the rest of the last piece of every row written */
    CUtensorMap md = ma_hi;
    if (a.nbatch <= 1 && (reinterpret_cast<uintptr_t>(a.D) & 15) == 0 && a.ldd % 4 == 0 && a.N % 4 == 0) {
        if ((rc = make_map(ctx, &md, a.D, a.M, a.N, a.ldd, 32))) return rc;
        p.tma_store = 1;
    }
    if (NSPLIT == 2) return launch_kernel<CTAS, BN, NSPLIT, false, KCH>(ctx, ma_hi, ma_lo, mb_hi, mb_lo, md, p, s, &ma_x, &mb_x);
    return launch_kernel<CTAS, BN, NSPLIT, false, KCH>(ctx, ma_hi, ma_lo, mb_hi, mb_lo, md, p, s);
}


template <int CTAS, int BN>
int launch_cfg_f16(decxb_ctx* ctx, const decxb_gemm_f16_args& a, cudaStream_t s)
{
    using C = Cfg<CTAS, BN, 16>;
    CUtensorMap ma, mb;
    int rc;
    if ((rc = make_map_f16(ctx, &ma, a.A, a.M, a.K, a.lda, BM_CTA))) return rc;
    if ((rc = make_map_f16(ctx, &mb, a.Bt, a.N, a.K, a.ldbt, BN))) return rc;
    GemmParams p = {};
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.C = reinterpret_cast<const float*>(a.C); p.ldc = a.ldc;
    p.D = reinterpret_cast<float*>(a.D); p.ldd = a.ldd;
    p.bias = nullptr; p.act = a.act;
    p.tiles_m = (int)decxb_ceil_div(a.M, C::UMMA_M);
    p.tiles_n = (int)decxb_ceil_div(a.N, C::UMMA_N);
    p.num_kb = (int)decxb_ceil_div(a.K, 64);
    p.wait_limit_ns = ctx->wait_limit_ns;
    p.status = ctx->d_status;
    return launch_kernel<CTAS, BN, 16, false>(ctx, ma, ma, mb, mb, ma /* unused */, p, s);
}

}  // namespace

int decxb_launch_gemm_f16_tn(decxb_ctx* ctx, const decxb_gemm_f16_args& a, cudaStream_t s)
{
    if (a.M <= 0 || a.N <= 0 || a.K <= 0) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "gemm dims must be positive");
    if (a.M > 0x7fffffffLL || a.N > 0x7fffffffLL || a.K > 0x7fffffffLL) return decxb_fail(ctx, DECXB_ERR_TOO_LARGE, "gemm dims");
    const int64_t t2 = decxb_ceil_div(a.M, 256) * decxb_ceil_div(a.N, 256);
    if (a.N <= 64) return launch_cfg_f16<1, 64>(ctx, a, s);
    if (t2 * 2 < ctx->sm_count / 2 || a.N <= 128 || a.M <= 128) return launch_cfg_f16<1, 128>(ctx, a, s);
    return launch_cfg_f16<2, 128>(ctx, a, s);
}

void* decxb_tensor_map_encoder() { return reinterpret_cast<void*>(get_encode_fn()); }

void decxb_tile_shape(int tile, int* tm, int* tn)
{
    switch (tile) {
    case DECXB_TILE_2CTA_256x256: *tm = 256; *tn = 256; break;
    case DECXB_TILE_1CTA_128x256: *tm = 128; *tn = 256; break;
    case DECXB_TILE_1CTA_128x64:  *tm = 128; *tn = 64; break;
    default: *tm = 128; *tn = 128; break;
    }
}

/* cost = waves x accumulator area per SM x relative cost per unit of area; the relative costs
 * were measured on B200 at M=8192 N=4096 K=2048 and at 1024^3 (bigger tiles move fewer
 * shared-memory bytes per flop; small problems need more tiles than SMs) */
int decxb_pick_tile(decxb_ctx* ctx, int64_t M, int64_t N, int64_t nbatch)
{
    struct Cand { int tile, tm, tn, sms_per_tile; double area, rel; };
    const Cand cands[4] = {{DECXB_TILE_2CTA_256x256, 256, 256, 2, 32768, 1.00}, {DECXB_TILE_1CTA_128x256, 128, 256, 1, 32768, 1.18},
                           {DECXB_TILE_1CTA_128x128, 128, 128, 1, 16384, 1.24}, {DECXB_TILE_1CTA_128x64, 128, 64, 1, 8192, 2.20}};
    double best = -1; int tile = DECXB_TILE_1CTA_128x128;
    for (const Cand& c : cands) {
        const int64_t tiles = decxb_ceil_div(M, c.tm) * decxb_ceil_div(N, c.tn) * (nbatch > 1 ? nbatch : 1);
        const int64_t slots = ctx->sm_count / c.sms_per_tile > 0 ? ctx->sm_count / c.sms_per_tile : 1;
        const double cost = (double)decxb_ceil_div(tiles, slots) * c.area * c.rel;
        if (best < 0 || cost < best * 0.999) { best = cost; tile = c.tile; }
    }
    return tile;
}

int decxb_launch_gemm_tn(decxb_ctx* ctx, const decxb_gemm_args& a, cudaStream_t s)
{
    if (a.M <= 0 || a.N <= 0 || a.K <= 0) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "gemm dims must be positive");
    if (a.M > 0x7fffffffLL || a.N > 0x7fffffffLL || a.K > 0x7fffffffLL) return decxb_fail(ctx, DECXB_ERR_TOO_LARGE, "gemm dims");
    const bool x3 = a.a_lo != nullptr;
    int tile = a.tile;
    if (tile == DECXB_TILE_AUTO) tile = decxb_pick_tile(ctx, a.M, a.N, a.nbatch);
    if (a.a_16) {
        /* TF32 hi * hi plus two bf16 cross products, K accumulated in chunks; two tile shapes */
        if (a.nbatch > 1 || !a.a_lo16 || !a.b_16 || !a.b_lo16) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "bf16 cross-term operands");
        if (tile != DECXB_TILE_2CTA_256x256 || !chunked_regs_ok<2, 128, false, 2>(ctx)) return launch_cfg<1, 128, 2, KCHUNK>(ctx, a, s);
        return launch_cfg<2, 128, 2, KCHUNK>(ctx, a, s);
    }
    /* a K that fits the first chunk gives the same bits either way: take the kernel with fewer threads */
    const bool chunked = a.chunked && decxb_ceil_div(a.K, BK) > 2 * KCHUNK;
    if (a.chunked && !x3) return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "chunked accumulation needs the 3xTF32 operands");
    if (chunked) {
        if ((tile == DECXB_TILE_2CTA_256x256 && !chunked_regs_ok<2, 128, false>(ctx)) ||
            (tile == DECXB_TILE_1CTA_128x256 && !chunked_regs_ok<1, 256, false>(ctx))) {
            if (a.nbatch > 1) return decxb_fail(ctx, DECXB_ERR_CUDA, "chunked GEMM kernel was not compiled to 168 registers");
            tile = DECXB_TILE_1CTA_128x128;
        }
        switch (tile) {
        case DECXB_TILE_1CTA_128x128: return launch_cfg<1, 128, 3, KCHUNK>(ctx, a, s);
        case DECXB_TILE_2CTA_256x256: return launch_cfg<2, 128, 3, KCHUNK>(ctx, a, s);
        case DECXB_TILE_1CTA_128x256: return launch_cfg<1, 256, 3, KCHUNK>(ctx, a, s);
        case DECXB_TILE_1CTA_128x64:  return launch_cfg<1, 64, 3, KCHUNK>(ctx, a, s);
        default: return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "unknown gemm tile");
        }
    }
    switch (tile) {
    case DECXB_TILE_1CTA_128x128: return x3 ? launch_cfg<1, 128, 3>(ctx, a, s) : launch_cfg<1, 128, 1>(ctx, a, s);
    case DECXB_TILE_2CTA_256x256: return x3 ? launch_cfg<2, 128, 3>(ctx, a, s) : launch_cfg<2, 128, 1>(ctx, a, s);
    case DECXB_TILE_1CTA_128x256: return x3 ? launch_cfg<1, 256, 3>(ctx, a, s) : launch_cfg<1, 256, 1>(ctx, a, s);
    case DECXB_TILE_1CTA_128x64:  return x3 ? launch_cfg<1, 64, 3>(ctx, a, s)  : launch_cfg<1, 64, 1>(ctx, a, s);
    default: return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "unknown gemm tile");
    }
}

int decxb_launch_conv_implicit(decxb_ctx* ctx, const decxb_conv_gemm_args& a, cudaStream_t s)
{
    const bool x3 = a.src_lo != nullptr;
    if (a.chunked && !x3) return decxb_fail(ctx, DECXB_ERR_BAD_FLAG, "chunked accumulation needs the 3xTF32 operands");
    if (a.chunked && a.kW * a.kH * decxb_ceil_div(a.dp, BK) > 2 * KCHUNK) {
        if (a.Np <= 64)  return launch_conv_cfg<1, 64, 3, KCHUNK>(ctx, a, s);
        if (a.Np <= 128 || !chunked_regs_ok<2, 128, true>(ctx)) return launch_conv_cfg<1, 128, 3, KCHUNK>(ctx, a, s);
        return launch_conv_cfg<2, 128, 3, KCHUNK>(ctx, a, s);
    }
    if (a.Np <= 64)  return x3 ? launch_conv_cfg<1, 64, 3>(ctx, a, s)  : launch_conv_cfg<1, 64, 1>(ctx, a, s);
    if (a.Np <= 128) return x3 ? launch_conv_cfg<1, 128, 3>(ctx, a, s) : launch_conv_cfg<1, 128, 1>(ctx, a, s);
    return x3 ? launch_conv_cfg<2, 128, 3>(ctx, a, s) : launch_conv_cfg<2, 128, 1>(ctx, a, s);
}

extern "C" int decxb_selftest_bounded_wait(decxb_ctx* ctx, int limit_ms)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (limit_ms <= 0 || limit_ms > 1000) return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "limit must be 1..1000 ms");
    GemmParams p = {};
    p.wait_limit_ns = (long long)limit_ms * 1000000LL;
    p.status = ctx->d_status;
    {
        decxb_launch_scope scope(ctx, ctx->stream, DECXB_K_GEMM);
        decxb_wait_probe_kernel<<<1, 32, 0, ctx->stream>>>(p);
    }
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    DECXB_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return decxb_check_dev_status(ctx);
}
