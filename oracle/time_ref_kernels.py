"""Times the REFERENCE'S OWN CUDA kernels (compiled for sm_100a into
oracle/_ref/libdecx_ref_kernels_gpu.so) on the GPU of this machine, for the BASELINE shapes.
TEST INFRASTRUCTURE: prints one JSON line per case; nothing in the product reads it.

    python oracle/time_ref_kernels.py [--big]

Kernels: cu_GEMM_fp32_spec (srcs/GEMM/CUDA/large_squares/GEMM.cuh:31-100) and the convolution
pair cu_sIm2Col_r8_within + cu_conv_eq_mm (srcs/convolution/CUDA/im2col/im2col.cuh:86-178,
eq_GEMM.cuh:109-209), launched with the reference drivers' geometry.  The time is the second
launch of each kernel (the first one brings the managed buffers to the device).
"""
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from oracle import oracle as o  # noqa: E402


def main():
    big = "--big" in sys.argv
    assert o.ref_kernels_gpu() is not None, "oracle/_ref/libdecx_ref_kernels_gpu.so is not built"
    gemms = [("cfg1", 1024, 1024, 1024)] + ([("cfg2", 8192, 4096, 2048)] if big else [])
    for name, M, N, K in gemms:
        A = o.fill_uniform(M * K, 1).reshape(M, K)
        B = o.fill_uniform(K * N, 2).reshape(K, N)
        D = o.ref_gemm_spec(A, B, gpu=True)
        ms = o.ref_last_kernel_ms()
        rows = slice(0, min(M, 64))
        ok = bool((D[rows] == o.gemm_fmaf(A[rows], B)).all())
        print(json.dumps({"case": name, "kernel": "cu_GEMM_fp32_spec", "ms": ms, "tflops": 2.0 * M * N * K / ms / 1e9,
                          "bit_identical_to_oracle": ok}))
    convs = [("cfg3", 224, 224, 64, 3, 64)] + ([("cfg4_one_image", 56, 56, 256, 3, 256)] if big else [])
    for name, W, H, C, k, F in convs:
        src = o.make_tensor(W, H, C, 4)
        flt = o.make_filters(k, k, C, F, 5)
        P = o.ref_im2col_pack(src, W, C, k, k, 1, gpu=True)
        pack_ms = o.ref_last_kernel_ms()
        ok_pack = bool((P.view("u4") == o.im2col_pack(src, W, C, k, k, 1).view("u4")).all())
        o.ref_conv2_im2col(src, W, C, flt, k, 1, gpu=True)
        both_ms = o.ref_last_kernel_ms()
        flops = 2.0 * H * W * k * k * C * F
        print(json.dumps({"case": name, "kernel": "cu_sIm2Col_r8_within + cu_conv_eq_mm", "pack_ms": pack_ms,
                          "pack_plus_gemm_ms": both_ms, "tflops": flops / both_ms / 1e9,
                          "pack_bit_identical_to_oracle": ok_pack}))


if __name__ == "__main__":
    main()
