/*
 * Tensor-core ceiling probe (sm_100a): what the tcgen05 TF32 pipe delivers when nothing but the
 * MMA instruction stream runs.  It gives the GEMM kernel's roofline a measured denominator: the
 * reference publishes no peak, and the vendor's dense TF32 figure is a nominal one.
 *
 * One CTA pair per two SMs (cluster of 2, cta_group::2, the GEMM kernel's 256 x 256 tile).  The
 * operand tiles of one k-block (a_hi, a_lo, b_hi, b_lo: 128 rows x 32 floats each per CTA) are
 * written to shared memory ONCE, then one thread of the leader CTA issues
 * tcgen05.mma.cta_group::2.kind::tf32 256 x 256 x 8 in a loop, with no TMA and no epilogue in
 * the loop:
 *   pattern 0  one MMA per k-step on the same two tiles            -> the TF32 issue peak
 *   pattern 1  the 3xTF32 k-step of the GEMM kernel (a_lo*b_hi, a_hi*b_lo, a_hi*b_hi on four
 *              distinct tiles)                                      -> the ceiling that the
 *              shared-memory operand reads of that pattern leave
 *   pattern 2  pattern 1 with a_hi kept in the collector buffer between its two MMAs
 *   pattern 3, 4, 5  the k-step of pattern 2 on the single-CTA tiles 128 x 64, 128 x 128 and
 *              128 x 256 (cta_group::1), the shapes small problems get
 * The wait for the last MMA is bounded like every wait in this library.
 */
#include "common.h"
#include "tc_ptx.cuh"

using namespace tcptx;

namespace {

constexpr int PROBE_THREADS = 128;
constexpr int TILE_BYTES = 128 * 32 * 4;                 /* 16 KiB: 128 rows of one 128-byte k-block (an A tile) */
/* a_hi, a_lo (128 rows each), b_hi, b_lo (BN rows each), alignment slack, barrier + TMEM slot */
constexpr int probe_smem(int bn) { return 2 * TILE_BYTES + 2 * bn * 128 + 1024 + 64; }

__device__ __forceinline__ uint32_t mix32(uint32_t h)
{
    h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;
    return h;
}

template <int PATTERN, int CTAS, int BN>
__global__ void __launch_bounds__(PROBE_THREADS, 1)
decxb_tensor_probe_kernel(int iters, long long wait_limit_ns, decxb_dev_status* status)
{
    constexpr int UMMA_M = 128 * CTAS, UMMA_N = BN * CTAS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    constexpr int B_BYTES = BN * 128;
    constexpr int OPERAND_BYTES = 2 * TILE_BYTES + 2 * B_BYTES;
    const uint32_t bar = base + OPERAND_BYTES;
    const uint32_t tmem_slot = bar + 8;
    const int warp = threadIdx.x >> 5;
    const uint32_t cta_rank = CTAS == 2 ? cluster_ctarank() : 0u;

    /* operand tiles: values in [-1, 1) for the hi tiles, 2^-12 of that for the lo tiles (the
     * magnitudes a real split produces); any placement will do, the data is random anyway */
    for (int i = threadIdx.x; i < OPERAND_BYTES / 4; i += PROBE_THREADS) {
        const uint32_t u = mix32((uint32_t)i * 0x9E3779B1u + blockIdx.x * 7919u + 1u);
        float v = (float)(u >> 8) * (1.0f / 8388608.0f) - 1.0f;
        const int off = i * 4;
        const bool is_lo = (off >= TILE_BYTES && off < 2 * TILE_BYTES) || off >= 2 * TILE_BYTES + B_BYTES;
        if (is_lo) v *= (1.0f / 4096.0f);               /* the a_lo and b_lo tiles */
        asm volatile("st.shared.f32 [%0], %1;" :: "r"(base + 4u * (uint32_t)i), "f"(v) : "memory");
    }
    fence_proxy_async_smem();
    if (threadIdx.x == 0) { mbar_init(bar, 1); fence_barrier_init(); }
    if (warp == 1) { tmem_alloc<CTAS>(tmem_slot, 512); tmem_relinquish<CTAS>(); }
    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

    if (cta_rank == 0 && threadIdx.x == 0) {
        constexpr uint32_t idesc = make_idesc(UMMA_M, UMMA_N);
        const uint64_t da_hi = make_smem_desc(base), da_lo = make_smem_desc(base + TILE_BYTES);
        const uint64_t db_hi = make_smem_desc(base + 2 * TILE_BYTES), db_lo = make_smem_desc(base + 2 * TILE_BYTES + B_BYTES);
        for (int it = 0; it < iters; ++it) {
            const uint32_t tmem_d = tmem_base + (uint32_t)((it & 1) * UMMA_N);  /* alternate the two accumulators */
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint64_t koff = (uint64_t)((kk * 8 * 4) >> 4);
                const uint32_t acc = (it >= 2 || kk != 0) ? 1u : 0u;
                if (PATTERN == 0) {
                    umma_tf32<CTAS>(tmem_d, da_hi + koff, db_hi + koff, idesc, acc);
                } else {
                    umma_tf32<CTAS>(tmem_d, da_lo + koff, db_hi + koff, idesc, acc);
                    umma_tf32<CTAS, PATTERN == 2 ? 1 : 0>(tmem_d, da_hi + koff, db_lo + koff, idesc, 1u);
                    umma_tf32<CTAS, PATTERN == 2 ? 2 : 0>(tmem_d, da_hi + koff, db_hi + koff, idesc, 1u);
                }
            }
        }
        umma_commit<CTAS>(bar);
    }
    /* both CTAs wait for the commit (it arrives on the barrier at the same offset in each) */
    if (threadIdx.x == 0) {
        const unsigned long long t0 = globaltimer_ns();
        uint32_t spins = 0;
        while (!mbar_try_wait(bar, 0u)) {
            if ((++spins & 255u) == 0 && (long long)(globaltimer_ns() - t0) > wait_limit_ns) {
                if (atomicCAS(&status->code, 0, DECXB_DEVERR_WAIT_EXPIRED) == 0) {
                    status->where = 950; status->block = (int)blockIdx.x; status->detail = iters;
                    __threadfence_system();
                }
                break;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();
    if (warp == 1) { tc_fence_after(); tmem_dealloc<CTAS>(tmem_base, 512); }
}

template <int PATTERN, int CTAS, int BN>
int launch_probe(decxb_ctx* ctx, int iters, cudaStream_t s)
{
    auto kernel = decxb_tensor_probe_kernel<PATTERN, CTAS, BN>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, probe_smem(BN));
    if (e != cudaSuccess) return decxb_fail(ctx, DECXB_ERR_CUDA, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(ctx->sm_count / CTAS * CTAS), 1, 1);
    cfg.blockDim = dim3(PROBE_THREADS, 1, 1);
    cfg.dynamicSmemBytes = probe_smem(BN);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    /* generous limit for the final wait: the loop itself is the measured time */
    const long long limit = 20000000000LL;
    decxb_launch_scope scope(ctx, s, DECXB_K_GEMM);
    DECXB_CUDA_TRY(ctx, cudaLaunchKernelEx(&cfg, kernel, iters, limit, ctx->d_status));
    return DECXB_OK;
}

int launch_probe_any(decxb_ctx* ctx, int pattern, int iters, cudaStream_t s)
{
    switch (pattern) {
    case 0: return launch_probe<0, 2, 128>(ctx, iters, s);
    case 1: return launch_probe<1, 2, 128>(ctx, iters, s);
    case 2: return launch_probe<2, 2, 128>(ctx, iters, s);
    case 3: return launch_probe<2, 1, 64>(ctx, iters, s);
    case 4: return launch_probe<2, 1, 128>(ctx, iters, s);
    default: return launch_probe<2, 1, 256>(ctx, iters, s);
    }
}

}  // namespace

extern "C" int decxb_probe_tensor_peak(decxb_ctx* ctx, int pattern, double target_ms, decxb_tensor_probe* out)
{
    int rc = decxb_bind(ctx);
    if (rc) return rc;
    if (!out || pattern < 0 || pattern > 5 || !(target_ms > 0.0) || target_ms > 5000.0)
        return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "probe: pattern 0..5, 0 < target_ms <= 5000");
    cudaStream_t s = ctx->stream;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    DECXB_CUDA_TRY(ctx, cudaEventCreate(&e0));
    if (cudaEventCreate(&e1) != cudaSuccess) { cudaEventDestroy(e0); return decxb_fail(ctx, DECXB_ERR_CUDA, "cudaEventCreate"); }
    auto timed = [&](int iters, float* ms) -> int {
        cudaEventRecord(e0, s);
        int r = launch_probe_any(ctx, pattern, iters, s);
        cudaEventRecord(e1, s);
        if (r) return r;
        if (cudaStreamSynchronize(s) != cudaSuccess || cudaEventElapsedTime(ms, e0, e1) != cudaSuccess)
            return decxb_fail(ctx, DECXB_ERR_CUDA, std::string("probe: ") + cudaGetErrorString(cudaGetLastError()));
        return decxb_check_dev_status(ctx);
    };
    float ms = 0.f;
    int iters = 4000;
    rc = timed(iters, &ms);                 /* warm-up and calibration */
    if (rc == DECXB_OK) {
        double want = target_ms / (ms > 1e-3 ? ms : 1e-3) * iters;
        if (want > 2.0e9) want = 2.0e9;
        if (want < 1000.0) want = 1000.0;
        iters = (int)want;
        rc = timed(iters, &ms);
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (rc) return rc;
    const int mma_per_kstep = pattern == 0 ? 1 : 3;
    const int ctas = pattern <= 2 ? 2 : 1;
    const double clusters = ctx->sm_count / ctas;
    const double mma_flops = 2.0 * (128 * ctas) * (pattern == 3 ? 64 : pattern == 4 ? 128 : 256) * 8;
    out->ms = ms;
    out->iterations = (int64_t)iters;
    out->sms = (int)(clusters * ctas);
    out->tensor_tflops = clusters * (double)iters * 4 * mma_per_kstep * mma_flops / (ms * 1e-3) / 1e12;
    out->algorithmic_tflops = out->tensor_tflops / mma_per_kstep;
    return DECXB_OK;
}
