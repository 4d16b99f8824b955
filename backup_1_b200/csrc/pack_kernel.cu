/*
 * im2col pack (sm_100a), bit-exact to the reference's cu_sIm2Col_r8_within
 * (srcs/convolution/CUDA/im2col/im2col.cuh:86-178) run on a zero-initialised staging buffer:
 *
 *   I2C[(y*eq_w + x)*Kp + (ky*kW + kx)*dp + c] = S[y + ky + off_y][x + kx + off_x][c]
 *
 * S = tensor value for 0 <= row < H and 0 <= col < wpitch, else 0; (off_y, off_x) =
 * (-(kH/2), -(kW/2)) with the zero-border flag and (0, 0) with the valid flag.
 *
 * The reference stages the tensor into an apron-padded buffer and lets each thread write
 * 16-byte pieces Kp*4 bytes apart (im2col.cuh:166-172).  Here the tensor is read in place
 * (bounds checks give the zero apron) and the work is laid out along the OUTPUT: the column
 * matrix is one flat array whose rows are Kp floats, so consecutive threads write
 * consecutive 16-byte words.  A block owns one output row y of one image and a run of x;
 * thread (ty, tx) keeps its column slot t = tx (+ k*TX) fixed, so tap and channel are
 * computed once, and walks x with stride TY: no division in the inner loop.  Source reads
 * are 16-byte loads that hit L1/L2 (each source word is used kW*kH times); the kernel is
 * bound by the HBM write of the column matrix.
 */
#include "common.h"

#include <cudaTypedefs.h>

#define PACK_X_PER_BLOCK 32

__global__ void __launch_bounds__(256)
decxb_im2col_pack_kernel(const float4* __restrict__ src, float4* __restrict__ i2c,
                         int H, int wp, int dp4, int kW, int kH, int off_y, int off_x,
                         int out_h, int eq_w, int Kp4, int TX, int TY,
                         int64_t src_stride4, int64_t i2c_stride4, const decxb_bounds bnd)
{
    const int tid = threadIdx.x;
    if (tid >= TX * TY) return;
    const int tx = tid % TX, ty = tid / TX;
    const int row = blockIdx.x;                 /* image * out_h + y */
    const int img = row / out_h, y = row - img * out_h;
    const int x_begin = blockIdx.y * PACK_X_PER_BLOCK;
    const int x_end = min(x_begin + PACK_X_PER_BLOCK, eq_w);
    const float4* __restrict__ s_img = src + (int64_t)img * src_stride4;
    float4* __restrict__ o_row = i2c + (int64_t)img * i2c_stride4 + (int64_t)y * eq_w * Kp4;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);

    for (int t = tx; t < Kp4; t += TX) {
        const int tap = t / dp4, c4 = t - tap * dp4;
        const int ky = tap / kW, kx = tap - ky * kW;
        const int r = y + ky + off_y;
        const bool row_ok = (r >= 0) && (r < H);
        const float4* __restrict__ s_row = s_img + ((int64_t)r * wp) * dp4 + c4;
        const int dq = kx + off_x;
#pragma unroll 4
        for (int x = x_begin + ty; x < x_end; x += TY) {
            const int q = x + dq;
            float4 v = zero;
            if (row_ok && q >= 0 && q < wp && DECXB_OK_IN(bnd, s_row + (int64_t)q * dp4, 16)) v = __ldg(s_row + (int64_t)q * dp4);
            if (DECXB_OK_OUT0(bnd, o_row + (int64_t)x * Kp4 + t, 16)) o_row[(int64_t)x * Kp4 + t] = v;
        }
    }
}

/* Staged variant: the kH source rows a block needs (its run of x plus the kW-1 halo, all
 * channels) are loaded ONCE into shared memory with coalesced 16-byte loads, bounds checks
 * giving the zero apron; every output word is then served from shared memory.  Pixels x..x+kW-1
 * of one source row are adjacent in shared memory exactly as the kW*dp floats of tap row ky are
 * adjacent in an output row, so the copy-out is a straight run per (x, ky).  L2 read traffic
 * drops from kW*kH passes over the tensor to one; the kernel is left with the write of the
 * column matrix. */
__global__ void __launch_bounds__(256)
decxb_im2col_pack_staged_kernel(const float4* __restrict__ src, float4* __restrict__ i2c,
                                int H, int wp, int dp4, int kW, int kH, int off_y, int off_x,
                                int out_h, int eq_w, int Kp4, int TX, int TY,
                                int64_t src_stride4, int64_t i2c_stride4, const decxb_bounds bnd)
{
    extern __shared__ float4 stage[];                 /* [kH][PX][dp4], PX = PACK_X_PER_BLOCK + kW - 1 */
    const int tid = threadIdx.x;
    const int row = blockIdx.x;
    const int img = row / out_h, y = row - img * out_h;
    const int x_begin = blockIdx.y * PACK_X_PER_BLOCK;
    const int x_end = min(x_begin + PACK_X_PER_BLOCK, eq_w);
    const int PX = PACK_X_PER_BLOCK + kW - 1;
    const int row4 = PX * dp4;                        /* float4 per staged row */
    const float4* __restrict__ s_img = src + (int64_t)img * src_stride4;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);

    const int q0 = x_begin + off_x;                   /* source pixel of staged pixel 0 */
    const int i_lo = max(0, -q0) * dp4, i_hi = max(0, min(PX, wp - q0)) * dp4;   /* in-range part of a staged row */
    for (int ky = 0; ky < kH; ++ky) {
        const int r = y + ky + off_y;
        const bool row_ok = (r >= 0) && (r < H);
        const float4* __restrict__ s_row = s_img + ((int64_t)r * wp + q0) * dp4;
        float4* st = stage + ky * row4;
        for (int i = tid; i < row4; i += blockDim.x)
            st[i] = (row_ok && i >= i_lo && i < i_hi && DECXB_OK_IN(bnd, s_row + i, 16)) ? __ldg(s_row + i) : zero;
    }
    __syncthreads();

    if (tid >= TX * TY) return;
    const int tx = tid % TX, ty = tid / TX;
    float4* __restrict__ o_row = i2c + (int64_t)img * i2c_stride4 + (int64_t)y * eq_w * Kp4;
    const int seg4 = kW * dp4;                        /* float4 per tap row */
    for (int t = tx; t < Kp4; t += TX) {
        const int ky = t / seg4;
        const float4* st = stage + ky * row4 + (t - ky * seg4);
#pragma unroll 4
        for (int x = x_begin + ty; x < x_end; x += TY)
            if (DECXB_OK_OUT0(bnd, o_row + (int64_t)x * Kp4 + t, 16)) o_row[(int64_t)x * Kp4 + t] = st[(x - x_begin) * dp4];
    }
}

/* TMA variant: no thread touches the data.  One tiled TMA load brings the kH source rows of a
 * block's run of x (plus halo, all channels, box {dp, PX, kH, 1} of the tensor seen as
 * (channel, x, y, image)) into shared memory; pixels outside the tensor are zero-filled by the
 * copy engine, which is the zero apron.  Then every (x, ky) pair is ONE bulk store
 * shared -> global of kW*dp floats: the kW adjacent pixels of staged row ky are exactly tap
 * row ky of output row x.  Threads only compute addresses and issue copies. */
__device__ __forceinline__ uint32_t pk_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__global__ void __launch_bounds__(64)
decxb_im2col_pack_tma_kernel(const __grid_constant__ CUtensorMap src_map, float* __restrict__ i2c,
                             int dp, int kW, int kH, int off_y, int off_x, int out_h, int eq_w, int64_t Kp,
                             int64_t i2c_stride, long long wait_limit_ns, decxb_dev_status* status)
{
    extern __shared__ __align__(128) uint8_t pk_smem[];
    __shared__ __align__(8) uint64_t bar;
    const uint32_t stage = (pk_smem_u32(pk_smem) + 127u) & ~127u;
    const uint32_t b = pk_smem_u32(&bar);
    const int row = blockIdx.x;
    const int img = row / out_h, y = row - img * out_h;
    const int x_begin = blockIdx.y * PACK_X_PER_BLOCK;
    const int nx = min(PACK_X_PER_BLOCK, eq_w - x_begin);
    const int PX = PACK_X_PER_BLOCK + kW - 1;
    const uint32_t bytes = (uint32_t)kH * PX * dp * 4u;

    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(b) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(b), "r"(bytes) : "memory");
        asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
            :: "r"(stage), "l"(&src_map), "r"(b), "r"(0), "r"(x_begin + off_x), "r"(y + off_y), "r"(img) : "memory");
    }
    __syncthreads();
    /* Bounded wait for the load.  On expiry the block records where it gave up, then waits once
     * more, again with a limit, for its own copy (which cannot be cancelled) before it lets go of
     * the shared memory that copy writes, and stores nothing. */
    auto wait_load = [&](long long limit_ns) -> bool {
        unsigned long long t0 = 0; uint32_t spins = 0, done = 0;
        while (true) {
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(b) : "memory");
            if (done) return true;
            if ((++spins & 255u) == 0) {
                unsigned long long now; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                if ((long long)(now - t0) > limit_ns) return false;
            }
        }
    };
    bool ok = wait_load(wait_limit_ns);
    if (!ok) {
        if (atomicCAS(&status->code, 0, DECXB_DEVERR_WAIT_EXPIRED) == 0) {
            status->where = 800; status->block = (int)blockIdx.x; status->detail = (int)blockIdx.y;
        }
        (void)wait_load(wait_limit_ns);
    }
    if (ok) {
        float* o_row = i2c + (int64_t)img * i2c_stride + ((int64_t)y * eq_w + x_begin) * Kp;
        const uint32_t seg_bytes = (uint32_t)kW * dp * 4u;
        for (int i = threadIdx.x; i < nx * kH; i += blockDim.x) {
            const int xi = i / kH, ky = i - xi * kH;
            const uint32_t s_addr = stage + (uint32_t)((ky * PX + xi) * dp) * 4u;
            float* d_addr = o_row + (int64_t)xi * Kp + (int64_t)ky * kW * dp;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                         :: "l"(d_addr), "r"(s_addr), "r"(seg_bytes) : "memory");
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   /* shared memory may go once it has been read */
    }
}

static int launch_pack_tma(decxb_ctx* ctx, const float* src, int64_t H, int64_t wp, int64_t dp, int64_t batch,
                           int64_t src_stride, int kW, int kH, int off_y, int off_x, const decxb_conv_geom& g,
                           float* i2c, int64_t i2c_stride, dim3 grid, size_t stage_bytes, cudaStream_t s)
{
    auto fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(decxb_tensor_map_encoder());
    if (!fn) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
    CUtensorMap map;
    cuuint64_t dims[4] = {(cuuint64_t)dp, (cuuint64_t)wp, (cuuint64_t)H, (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)dp * 4, (cuuint64_t)wp * dp * 4, (cuuint64_t)src_stride * 4};
    cuuint32_t box[4] = {(cuuint32_t)dp, (cuuint32_t)(PACK_X_PER_BLOCK + kW - 1), (cuuint32_t)kH, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(src), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return decxb_fail(ctx, DECXB_ERR_CUDA, "cuTensorMapEncodeTiled (pack) failed: " + std::to_string((int)r));
    static std::once_flag once[DECXB_MAX_DEVICES];
    const int dev = ctx->device;
    std::call_once(once[dev], [] {
        cudaFuncSetAttribute(decxb_im2col_pack_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
    });
    decxb_launch_scope scope(ctx, s, DECXB_K_PACK);
    decxb_im2col_pack_tma_kernel<<<grid, 64, stage_bytes + 128, s>>>(map, i2c, (int)dp, kW, kH, off_y, off_x, (int)g.out_h,
                                                                     (int)g.eq_w, g.Kp, i2c_stride, ctx->wait_limit_ns,
                                                                     ctx->d_status);
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    return DECXB_OK;
}

int decxb_launch_pack(decxb_ctx* ctx, const float* src, int64_t W, int64_t H, int64_t depth,
                      int64_t kW, int64_t kH, int flag, float* i2c, int64_t batch,
                      int64_t src_stride, int64_t i2c_stride, cudaStream_t s)
{
    decxb_conv_geom g;
    int rc = decxb_conv_geometry(W, H, depth, kW, kH, 1, flag, &g);
    if (rc) return decxb_fail(ctx, rc, "im2col pack geometry");
    const int64_t dp = decxb_ceil_to(depth, 4), wp = decxb_ceil_to(W, 4);
    if (batch <= 0) return DECXB_OK;
    if (src_stride == 0) src_stride = H * wp * dp;
    if (i2c_stride == 0) i2c_stride = g.M * g.Kp;
    if (((uintptr_t)src | (uintptr_t)i2c) % 16 || src_stride % 4 || i2c_stride % 4)
        return decxb_fail(ctx, DECXB_ERR_BAD_PARAM, "im2col pack needs 16-byte aligned tensors");
    if (g.out_h * batch > 0x7fffffffLL || g.Kp / 4 > 0x7fffffffLL || H * wp * dp / 4 > 0x7fffffffffLL)
        return decxb_fail(ctx, DECXB_ERR_TOO_LARGE, "im2col pack");
    const int Kp4 = (int)(g.Kp / 4);
    /* column slots per thread row: the fewest passes over Kp4 with at most 256 threads, all
     * passes equally full (Kp4 = 576 -> 3 passes of 192, not 2 full + 1 quarter-full of 256) */
    const int passes = (Kp4 + 255) / 256;
    const int TX = (Kp4 + passes - 1) / passes;
    const int TY = 256 / TX > 0 ? 256 / TX : 1;
    dim3 grid((unsigned)(g.out_h * batch), (unsigned)decxb_ceil_div(g.eq_w, PACK_X_PER_BLOCK));
    const int off_y = flag == DECXB_CONV_ZERO_COMPENSATE ? -(int)(kH / 2) : 0;
    const int off_x = flag == DECXB_CONV_ZERO_COMPENSATE ? -(int)(kW / 2) : 0;
    const int block = (TX * TY + 31) / 32 * 32;
    const size_t stage_bytes = (size_t)kH * (PACK_X_PER_BLOCK + kW - 1) * dp * sizeof(float);
    const decxb_bounds bnd = {ctx->d_status, decxb_make_extent(src, (size_t)((batch - 1) * src_stride + H * wp * dp) * 4),
                              decxb_make_extent(i2c, (size_t)((batch - 1) * i2c_stride + g.M * g.Kp) * 4), {}, DECXB_BK_PACK};
    /* copy-engine path: channels fit one TMA box, the staged rows fit shared memory, batch fits
     * a tensor-map dimension */
    if (ctx->pack_variant == 0 && dp <= 256 && stage_bytes + 128 <= 112 * 1024 && batch <= 0x7fffffffLL)
        return launch_pack_tma(ctx, src, H, wp, dp, batch, src_stride, (int)kW, (int)kH, off_y, off_x, g, i2c, i2c_stride,
                               grid, stage_bytes, s);
    if (ctx->pack_variant != 2 && stage_bytes <= 112 * 1024) {
        static std::once_flag once[DECXB_MAX_DEVICES];
        const int dev = ctx->device;
        std::call_once(once[dev], [] {
            cudaFuncSetAttribute(decxb_im2col_pack_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
        });
        decxb_launch_scope scope(ctx, s, DECXB_K_PACK);
        decxb_im2col_pack_staged_kernel<<<grid, block < 128 ? 128 : block, stage_bytes, s>>>(
            reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(i2c),
            (int)H, (int)wp, (int)(dp / 4), (int)kW, (int)kH, off_y, off_x,
            (int)g.out_h, (int)g.eq_w, Kp4, TX, TY, src_stride / 4, i2c_stride / 4, bnd);
        DECXB_CUDA_TRY(ctx, cudaGetLastError());
        return DECXB_OK;
    }
    decxb_launch_scope scope(ctx, s, DECXB_K_PACK);
    decxb_im2col_pack_kernel<<<grid, block, 0, s>>>(
        reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(i2c),
        (int)H, (int)wp, (int)(dp / 4), (int)kW, (int)kH, off_y, off_x,
        (int)g.out_h, (int)g.eq_w, Kp4, TX, TY, src_stride / 4, i2c_stride / 4, bnd);
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    return DECXB_OK;
}
