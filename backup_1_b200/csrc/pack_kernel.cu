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

#define PACK_X_PER_BLOCK 32

__global__ void __launch_bounds__(256)
decxb_im2col_pack_kernel(const float4* __restrict__ src, float4* __restrict__ i2c,
                         int H, int wp, int dp4, int kW, int kH, int off_y, int off_x,
                         int out_h, int eq_w, int Kp4, int TX, int TY,
                         int64_t src_stride4, int64_t i2c_stride4)
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
            if (row_ok && q >= 0 && q < wp) v = __ldg(s_row + (int64_t)q * dp4);
            o_row[(int64_t)x * Kp4 + t] = v;
        }
    }
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
    const int TX = Kp4 < 256 ? Kp4 : 256;
    const int TY = 256 / TX > 0 ? 256 / TX : 1;
    dim3 grid((unsigned)(g.out_h * batch), (unsigned)decxb_ceil_div(g.eq_w, PACK_X_PER_BLOCK));
    const int off_y = flag == DECXB_CONV_ZERO_COMPENSATE ? -(int)(kH / 2) : 0;
    const int off_x = flag == DECXB_CONV_ZERO_COMPENSATE ? -(int)(kW / 2) : 0;
    const int block = (TX * TY + 31) / 32 * 32;
    decxb_launch_scope scope(ctx, s, DECXB_K_PACK);
    decxb_im2col_pack_kernel<<<grid, block, 0, s>>>(
        reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(i2c),
        (int)H, (int)wp, (int)(dp / 4), (int)kW, (int)kH, off_y, off_x,
        (int)g.out_h, (int)g.eq_w, Kp4, TX, TY, src_stride / 4, i2c_stride / 4);
    DECXB_CUDA_TRY(ctx, cudaGetLastError());
    return DECXB_OK;
}
