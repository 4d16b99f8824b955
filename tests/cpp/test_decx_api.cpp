/*
 * Test program for the C++ de:: layer, written the way the reference's console test programs
 * use the library (test/test/CUDA_GEMM/CUDA_GEMM.cpp:16-117, test/test/generating classes and
 * generating GPU classes), but with assertions instead of printed values.
 *   test_decx_api layout   -- containers, pitches, index formulas, error handles; needs no GPU
 *   test_decx_api gpu      -- GEMM and im2col convolution through every overload on a B200
 */
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "decx/DECX.h"

static int g_fail = 0;
#define CHECK(cond)                                                                   \
    do {                                                                              \
        if (!(cond)) { printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond); ++g_fail; } \
    } while (0)

static float rnd(unsigned& s)   /* uniform [-1, 1) */
{
    s = s * 1664525u + 1013904223u;
    return (float)(s >> 8) * (1.0f / 8388608.0f) - 1.0f;
}

static int test_layout()
{
    /* creating_Matrix.h: fill with i + j, read back; pitch is ceil8(width) */
    de::Matrix<float>& A = de::CreateMatrixRef<float>(13, 7, decx::Page_Default);
    CHECK(A.Width() == 13 && A.Height() == 7 && A.TotalBytes() == 13 * 7 * sizeof(float));
    for (int i = 0; i < 7; ++i) for (int j = 0; j < 13; ++j) A.index(i, j) = (float)(i + j);
    CHECK(&A.index(1, 0) - &A.index(0, 0) == 16);
    CHECK(A.index(6, 12) == 18.0f && A.index(0, 13) == 0.0f);
    /* operator= aliases the storage */
    de::Matrix<float>& A2 = de::CreateMatrixRef<float>();
    A2 = A;
    A2.index(2, 3) = -5.0f;
    CHECK(A.index(2, 3) == -5.0f && A2.Width() == 13);

    /* creating_Tensor.h: A.index(i, j, z) = i + j + z; HWC with dpitch = ceil4(depth), wpitch = ceil4(width) */
    de::Tensor<float>& T = de::CreateTensorRef<float>(10, 6, 3, decx::Page_Default);
    CHECK(T.Width() == 10 && T.Height() == 6 && T.Depth() == 3);
    for (int i = 0; i < 6; ++i) for (int j = 0; j < 10; ++j) for (int z = 0; z < 3; ++z) T.index(i, j, z) = (float)(i + j + z);
    CHECK(&T.index(0, 1, 0) - &T.index(0, 0, 0) == 4);
    CHECK(&T.index(1, 0, 0) - &T.index(0, 0, 0) == 4 * 12);
    CHECK(T.index(0, 0, 3) == 0.0f && T.index(0, 10, 0) == 0.0f);     /* padding is zero */

    de::TensorArray<float>& K = de::CreateTensorArrayRef<float>(3, 3, 3, 5, decx::Page_Default);
    CHECK(K.TensorNum() == 5);
    CHECK(&K.index(0, 0, 0, 1) - &K.index(0, 0, 0, 0) == 4 * 4 * 3);  /* dpitch * wpitch * height */
    K.index(2, 2, 2, 4) = 9.0f;
    CHECK(K.index(2, 2, 2, 4) == 9.0f);

    /* operations before InitCuda return the not-initialised handle (GEMM.h:63-66) */
    de::Matrix<float>& B = de::CreateMatrixRef<float>(4, 13, decx::Page_Default);
    de::Matrix<float>& C = de::CreateMatrixRef<float>();
    de::DH h = de::cuda::GEMM(A, B, C);
    CHECK(h.error_type == decx::DECX_FAIL_not_init && h.error_string != nullptr);
    de::Tensor<float>& D = de::CreateTensorRef<float>();
    h = de::cuda::Conv2_MK_im2col(T, K, D, decx::de_conv_zero_compensate);
    CHECK(h.error_type == decx::DECX_FAIL_not_init);
    A.release(); A2.release(); T.release(); K.release(); B.release();
    return g_fail;
}

/* one ascending-k fp32 fma chain per output: the reference kernels' arithmetic */
static void chain_gemm(de::Matrix<float>& A, de::Matrix<float>& B, de::Matrix<float>* C, std::vector<float>& out)
{
    const int M = A.Height(), K = A.Width(), N = B.Width();
    out.assign((size_t)M * N, 0.f);
    for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j) {
            float c = C ? C->index(i, j) : 0.f;
            for (int k = 0; k < K; ++k) c = fmaf(A.index(i, k), B.index(k, j), c);
            out[(size_t)i * N + j] = c;
        }
}

static double max_err(de::Matrix<float>& X, const std::vector<float>& R)
{
    double m = 0;
    const int M = X.Height(), N = X.Width();
    for (int i = 0; i < M; ++i) for (int j = 0; j < N; ++j) m = fmax(m, fabs((double)X.index(i, j) - R[(size_t)i * N + j]));
    return m;
}

static void test_gemm_known_answer()
{
    /* CUDA_GEMM.cpp:24-42: A[i][j] = 0.1 j, B[i][j] = 0.1 i, every C element = sum_k (0.1 k)^2 */
    const int n = 2048;
    de::Matrix<float>& A = de::CreateMatrixRef<float>(n, n, decx::Page_Locked);
    de::Matrix<float>& B = de::CreateMatrixRef<float>(n, n, decx::Page_Locked);
    de::Matrix<float>& C = de::CreateMatrixRef<float>(n, n, decx::Page_Locked);
    for (int i = 0; i < n; ++i) for (int j = 0; j < n; ++j) { A.index(i, j) = 0.1f * j; B.index(i, j) = 0.1f * i; }
    double expect = 0; for (int k = 0; k < n; ++k) { double v = (double)(0.1f * k); expect += v * v; }
    /* default mode: chunked accumulation, under the 1e-6 bar of K max|a| max|b| on this all-positive case */
    de::DH h = de::cuda::GEMM(A, B, C);
    CHECK(h.error_type == decx::DECX_SUCCESS);
    bool same = true; for (int i = 0; i < n; i += 37) for (int j = 0; j < n; j += 41) same &= C.index(i, j) == C.index(0, 0);
    CHECK(same);
    CHECK(fabs(C.index(n - 1, n - 1) - expect) / ((double)n * 204.7 * 204.7) <= 1e-6);
    /* whole-K tensor-core accumulation (opt-in): looser on same-sign data */
    de::cuda::SetGemmStrictAccumulation(false);
    h = de::cuda::GEMM(A, B, C);
    de::cuda::SetGemmStrictAccumulation(true);
    CHECK(h.error_type == decx::DECX_SUCCESS);
    CHECK(fabs(C.index(n - 1, n - 1) - expect) / expect < 2e-5);
    h = de::cuda::GEMM(A, B, C);
    /* the GPU_Matrix path of the same program (CUDA_GEMM.cpp:60-110) */
    de::GPU_Matrix<float>& dA = de::CreateGPUMatrixRef<float>(n, n);
    de::GPU_Matrix<float>& dB = de::CreateGPUMatrixRef<float>(n, n);
    de::GPU_Matrix<float>& dC = de::CreateGPUMatrixRef<float>();
    dA.Load_from_host(A); dB.Load_from_host(B);
    h = de::cuda::GEMM(dA, dB, dC);
    CHECK(h.error_type == decx::DECX_SUCCESS && dC.Width() == (uint)n && dC.Height() == (uint)n);
    de::Matrix<float>& C2 = de::CreateMatrixRef<float>(n, n, decx::Page_Locked);
    dC.Load_to_host(C2);
    CHECK(C2.index(5, 7) == C.index(5, 7) && C2.index(n - 1, 0) == C.index(0, 0));
    A.release(); B.release(); C.release(); C2.release(); dA.release(); dB.release(); dC.release();
}

static void test_gemm_random_and_errors()
{
    unsigned s = 12345;
    const int M = 203, K = 150, N = 117;                 /* nothing aligned: pitches 152, 120 */
    de::Matrix<float>& A = de::CreateMatrixRef<float>(K, M, decx::Page_Default);
    de::Matrix<float>& B = de::CreateMatrixRef<float>(N, K, decx::Page_Locked);
    de::Matrix<float>& C = de::CreateMatrixRef<float>(N, M, decx::Page_Default);
    de::Matrix<float>& D = de::CreateMatrixRef<float>();
    for (int i = 0; i < M; ++i) for (int k = 0; k < K; ++k) A.index(i, k) = rnd(s);
    for (int k = 0; k < K; ++k) for (int j = 0; j < N; ++j) B.index(k, j) = rnd(s);
    for (int i = 0; i < M; ++i) for (int j = 0; j < N; ++j) C.index(i, j) = rnd(s);
    std::vector<float> R;
    de::DH h = de::cuda::GEMM(A, B, D);
    CHECK(h.error_type == decx::DECX_SUCCESS && D.Width() == (uint)N && D.Height() == (uint)M);
    chain_gemm(A, B, nullptr, R);
    CHECK(max_err(D, R) / K <= 1e-6);
    h = de::cuda::GEMM(A, B, C, D);
    chain_gemm(A, B, &C, R);
    CHECK(h.error_type == decx::DECX_SUCCESS && max_err(D, R) / K <= 1e-6);
    /* plain TF32 is opt-in and visibly less exact */
    de::cuda::SetGemmPlainTF32(true);
    h = de::cuda::GEMM(A, B, C, D);
    const double e1 = max_err(D, R) / K;
    de::cuda::SetGemmPlainTF32(false);
    CHECK(h.error_type == decx::DECX_SUCCESS && e1 > 1e-6 && e1 < 2e-3);
    /* A.width != B.height -> DimsNotMatching (GEMM.h:68-71) */
    h = de::cuda::GEMM(B, B, D);
    CHECK(h.error_type == decx::DECX_FAIL_DimsNotMatching);
    /* device path with addend */
    de::GPU_Matrix<float>& dA = de::CreateGPUMatrixRef<float>(K, M);
    de::GPU_Matrix<float>& dB = de::CreateGPUMatrixRef<float>(N, K);
    de::GPU_Matrix<float>& dC = de::CreateGPUMatrixRef<float>(N, M);
    de::GPU_Matrix<float>& dD = de::CreateGPUMatrixRef<float>();
    dA.Load_from_host(A); dB.Load_from_host(B); dC.Load_from_host(C);
    h = de::cuda::GEMM(dA, dB, dC, dD);
    de::Matrix<float>& D2 = de::CreateMatrixRef<float>(N, M, decx::Page_Default);
    dD.Load_to_host(D2);
    CHECK(h.error_type == decx::DECX_SUCCESS && max_err(D2, R) / K <= 1e-6);
}

/* IEEE half <-> float for the test's own data (round to nearest even; no denormal inputs here) */
static de::Half f2h(float f)
{
    unsigned x; memcpy(&x, &f, 4);
    const unsigned sign = (x >> 16) & 0x8000u;
    int e = (int)((x >> 23) & 0xff) - 127 + 15;
    unsigned m = x & 0x7fffffu;
    de::Half h;
    if (e <= 0) { h.val = (unsigned short)sign; return h; }
    unsigned r = (m >> 13) + ((m & 0x1000u) && ((m & 0x2fffu) != 0) ? 1u : 0u);
    unsigned v = ((unsigned)e << 10) + r;
    h.val = (unsigned short)(sign | (v > 0x7bffu ? 0x7c00u : v));
    return h;
}
static float h2f(de::Half h)
{
    const unsigned sign = (unsigned)(h.val & 0x8000u) << 16, e = (h.val >> 10) & 0x1f, m = h.val & 0x3ffu;
    if (e == 0) { float f = (float)m * 5.9604644775390625e-8f; return (h.val & 0x8000u) ? -f : f; }
    const unsigned x = sign | ((e - 15 + 127) << 23) | (m << 13);
    float f; memcpy(&f, &x, 4); return f;
}

static void test_gemm_half()
{
    /* the fp16 overloads (GEMM.h:33-49): half in, half out; pitch is ceil16(width) */
    unsigned s = 99;
    const int M = 96, K = 80, N = 72;
    de::Matrix<de::Half>& A = de::CreateMatrixRef<de::Half>(K, M, decx::Page_Default);
    de::Matrix<de::Half>& B = de::CreateMatrixRef<de::Half>(N, K, decx::Page_Locked);
    de::Matrix<de::Half>& C = de::CreateMatrixRef<de::Half>(N, M, decx::Page_Default);
    de::Matrix<de::Half>& D = de::CreateMatrixRef<de::Half>();
    CHECK(&A.index(1, 0) - &A.index(0, 0) == 80 && &B.index(1, 0) - &B.index(0, 0) == 80);
    for (int i = 0; i < M; ++i) for (int k = 0; k < K; ++k) A.index(i, k) = f2h(rnd(s));
    for (int k = 0; k < K; ++k) for (int j = 0; j < N; ++j) B.index(k, j) = f2h(rnd(s));
    for (int i = 0; i < M; ++i) for (int j = 0; j < N; ++j) C.index(i, j) = f2h(rnd(s));
    for (int with_c = 0; with_c <= 1; ++with_c) {
        de::DH h = with_c ? de::cuda::GEMM(A, B, C, D) : de::cuda::GEMM(A, B, D);
        CHECK(h.error_type == decx::DECX_SUCCESS && D.Width() == (uint)N && D.Height() == (uint)M);
        double worst = 0;
        for (int i = 0; i < M; ++i) for (int j = 0; j < N; ++j) {
            double e = with_c ? (double)h2f(C.index(i, j)) : 0.0;
            for (int k = 0; k < K; ++k) e += (double)h2f(A.index(i, k)) * (double)h2f(B.index(k, j));
            worst = fmax(worst, fabs((double)h2f(D.index(i, j)) - e) - (fabs(e) * 4.8828125e-4 + K * 2.4e-7 + 6e-8));
        }
        CHECK(worst <= 0.0);
    }
    de::GPU_Matrix<de::Half>& dA = de::CreateGPUMatrixRef<de::Half>(K, M);
    de::GPU_Matrix<de::Half>& dB = de::CreateGPUMatrixRef<de::Half>(N, K);
    de::GPU_Matrix<de::Half>& dD = de::CreateGPUMatrixRef<de::Half>();
    dA.Load_from_host(A); dB.Load_from_host(B);
    de::DH h = de::cuda::GEMM(dA, dB, dD);
    de::Matrix<de::Half>& D2 = de::CreateMatrixRef<de::Half>(N, M, decx::Page_Default);
    dD.Load_to_host(D2);
    de::cuda::GEMM(A, B, D);
    bool same = h.error_type == decx::DECX_SUCCESS;
    for (int i = 0; i < M; ++i) for (int j = 0; j < N; ++j) same &= D2.index(i, j).val == D.index(i, j).val;
    CHECK(same);
}

static void test_gemm3()
{
    /* batched product over MatrixArrays (GEMM3.h:45-114), 5 matrices, nothing aligned */
    unsigned s = 4242;
    const int M = 150, K = 90, N = 70, nb = 5;
    de::MatrixArray<float>& A = de::CreateMatrixArrayRef<float>(K, M, nb, decx::Page_Locked);
    de::MatrixArray<float>& B = de::CreateMatrixArrayRef<float>(N, K, nb, decx::Page_Default);
    de::MatrixArray<float>& C = de::CreateMatrixArrayRef<float>(N, M, nb, decx::Page_Default);
    de::MatrixArray<float>& D = de::CreateMatrixArrayRef<float>();
    for (int b = 0; b < nb; ++b) {
        for (int i = 0; i < M; ++i) for (int k = 0; k < K; ++k) A.index(i, k, b) = rnd(s);
        for (int k = 0; k < K; ++k) for (int j = 0; j < N; ++j) B.index(k, j, b) = rnd(s);
        for (int i = 0; i < M; ++i) for (int j = 0; j < N; ++j) C.index(i, j, b) = rnd(s);
    }
    for (int with_c = 0; with_c <= 1; ++with_c) {
        de::DH h = with_c ? de::cuda::GEMM3(A, B, C, D) : de::cuda::GEMM3(A, B, D);
        CHECK(h.error_type == decx::DECX_SUCCESS && D.MatrixNumber() == (uint)nb && D.Width() == (uint)N && D.Height() == (uint)M);
        double m = 0;
        for (int b = 0; b < nb; ++b) for (int i = 0; i < M; ++i) for (int j = 0; j < N; ++j) {
            float c = with_c ? C.index(i, j, b) : 0.f;
            for (int k = 0; k < K; ++k) c = fmaf(A.index(i, k, b), B.index(k, j, b), c);
            m = fmax(m, fabs((double)D.index(i, j, b) - c));
        }
        CHECK(m / K <= 1e-6);
    }
    de::MatrixArray<float>& B2 = de::CreateMatrixArrayRef<float>(N, K, nb + 1, decx::Page_Default);
    CHECK(de::cuda::GEMM3(A, B2, D).error_type == decx::DECX_FAIL_MNumNotMatching);
}

/* direct cross-correlation in the column order (ky, kx, c) of the reference's column matrix */
static float conv_ref(de::Tensor<float>& S, de::TensorArray<float>& F, int n, int y, int x, int flag)
{
    const int kH = F.Height(), kW = F.Width(), C = S.Depth(), H = S.Height(), W = S.Width();
    const int oy = flag ? -(kH / 2) : 0, ox = flag ? -(kW / 2) : 0;
    float acc = 0.f;
    for (int ky = 0; ky < kH; ++ky) for (int kx = 0; kx < kW; ++kx) for (int c = 0; c < C; ++c) {
        const int r = y + ky + oy, q = x + kx + ox;
        const float v = (r >= 0 && r < H && q >= 0 && q < W) ? S.index(r, q, c) : 0.f;
        acc = fmaf(v, F.index(ky, kx, c, n), acc);
    }
    return acc;
}

static void test_conv()
{
    unsigned s = 777;
    const int W = 21, H = 12, C = 6, N = 5;
    for (int flag = 0; flag <= 1; ++flag) for (int algo = 0; algo <= 1; ++algo) {
        const int kW = flag ? 3 : 5, kH = 3;
        de::cuda::SetConvExplicitPack(algo == 1);
        de::Tensor<float>& S = de::CreateTensorRef<float>(W, H, C, decx::Page_Locked);
        de::TensorArray<float>& F = de::CreateTensorArrayRef<float>(kW, kH, C, N, decx::Page_Default);
        de::Tensor<float>& D = de::CreateTensorRef<float>();
        for (int i = 0; i < H; ++i) for (int j = 0; j < W; ++j) for (int z = 0; z < C; ++z) S.index(i, j, z) = rnd(s);
        for (int n = 0; n < N; ++n) for (int i = 0; i < kH; ++i) for (int j = 0; j < kW; ++j) for (int z = 0; z < C; ++z) F.index(i, j, z, n) = rnd(s);
        de::DH h = de::cuda::Conv2_MK_im2col(S, F, D, flag);
        CHECK(h.error_type == decx::DECX_SUCCESS);
        const int ow = flag ? W : W - (kW / 2) * 2, oh = flag ? H : H - (kH / 2) * 2;
        CHECK((int)D.Width() == ow && (int)D.Height() == oh && (int)D.Depth() == N);
        double m = 0;
        for (int y = 0; y < oh; ++y) for (int x = 0; x < ow; ++x) for (int n = 0; n < N; ++n)
            m = fmax(m, fabs((double)D.index(y, x, n) - conv_ref(S, F, n, y, x, flag)));
        CHECK(m / (kW * kH * C) <= 1e-6);
        /* device-resident overload and the batched TensorArray overload give the same numbers */
        de::GPU_Tensor<float>& dS = de::CreateGPUTensorRef<float>(W, H, C);
        de::GPU_TensorArray<float>& dF = de::CreateGPUTensorArrayRef<float>(kW, kH, C, N);
        de::GPU_Tensor<float>& dD = de::CreateGPUTensorRef<float>();
        dS.Load_from_host(S); dF.Load_from_host(F);
        h = de::cuda::Conv2_MK_im2col(dS, dF, dD, flag);
        de::Tensor<float>& D2 = de::CreateTensorRef<float>(ow, oh, N, decx::Page_Default);
        dD.Load_to_host(D2);
        bool same = h.error_type == decx::DECX_SUCCESS;
        for (int y = 0; y < oh; ++y) for (int x = 0; x < ow; ++x) for (int n = 0; n < N; ++n) same &= D2.index(y, x, n) == D.index(y, x, n);
        CHECK(same);
        de::TensorArray<float>& SB = de::CreateTensorArrayRef<float>(W, H, C, 3, decx::Page_Default);
        for (int b = 0; b < 3; ++b) for (int i = 0; i < H; ++i) for (int j = 0; j < W; ++j) for (int z = 0; z < C; ++z)
            SB.index(i, j, z, b) = b == 1 ? S.index(i, j, z) : rnd(s);
        de::GPU_TensorArray<float>& dSB = de::CreateGPUTensorArrayRef<float>(W, H, C, 3);
        de::GPU_TensorArray<float>& dDB = de::CreateGPUTensorArrayRef<float>();
        dSB.Load_from_host(SB);
        h = de::cuda::Conv2_MK_im2col(dSB, dF, dDB, flag);
        CHECK(h.error_type == decx::DECX_SUCCESS && dDB.TensorNum() == 3 && (int)dDB.Width() == ow);
        de::TensorArray<float>& DB = de::CreateTensorArrayRef<float>(ow, oh, N, 3, decx::Page_Default);
        dDB.Load_to_host(DB);
        same = true;
        for (int y = 0; y < oh; ++y) for (int x = 0; x < ow; ++x) for (int n = 0; n < N; ++n) same &= DB.index(y, x, n, 1) == D.index(y, x, n);
        CHECK(same);
        /* bad kernel / flag */
        h = de::cuda::Conv2_MK_im2col(S, F, D, 7);
        CHECK(h.error_type == decx::DECX_FAIL_ErrorFlag);
    }
    de::cuda::SetConvExplicitPack(false);
    de::Tensor<float>& S = de::CreateTensorRef<float>(8, 8, 4, decx::Page_Default);
    de::TensorArray<float>& F = de::CreateTensorArrayRef<float>(19, 3, 4, 2, decx::Page_Default);   /* radius 9 > 8 */
    de::Tensor<float>& D = de::CreateTensorRef<float>();
    CHECK(de::cuda::Conv2_MK_im2col(S, F, D, 1).error_type == decx::DECX_FAIL_ConvBadKernel);
    de::TensorArray<float>& F2 = de::CreateTensorArrayRef<float>(3, 3, 8, 2, decx::Page_Default);    /* depth mismatch */
    CHECK(de::cuda::Conv2_MK_im2col(S, F2, D, 1).error_type == decx::DECX_FAIL_DimsNotMatching);
}

int main(int argc, char** argv)
{
    if (argc < 2) { printf("usage: %s layout|gpu\n", argv[0]); return 2; }
    if (!strcmp(argv[1], "layout")) { test_layout(); }
    else if (!strcmp(argv[1], "gpu")) {
        de::InitCuda();
        test_gemm_known_answer();
        test_gemm_random_and_errors();
        test_gemm3();
        test_gemm_half();
        test_conv();
        de::release_all_tmp();
    } else return 2;
    printf(g_fail ? "%d check(s) FAILED\n" : "all checks passed\n", g_fail);
    return g_fail ? 1 : 0;
}
