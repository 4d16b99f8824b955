"""The oracle against the reference's own outputs (golden vectors, and the reference code
itself when oracle/_ref is built).  CPU only."""
import hashlib

import numpy as np
import pytest

from oracle import oracle as o


def _check(z, cases, name, arr):
    arr = np.ascontiguousarray(arr)
    if name in cases["sha256"]:
        assert hashlib.sha256(arr.tobytes()).hexdigest() == cases["sha256"][name], name
        assert np.array_equal(arr.reshape(-1)[::97].view(np.uint32), z[name + "__sample"].view(np.uint32))
    else:
        assert arr.shape == z[name].shape
        assert np.array_equal(arr.view(np.uint32), z[name].view(np.uint32)), name


def test_gemm_chain_matches_reference_kernels(golden):
    z, cases = golden
    for c in cases["gemm"]:
        A = o.fill_uniform(c["M"] * c["K"], 1).reshape(c["M"], c["K"])
        B = o.fill_uniform(c["K"] * c["N"], 2).reshape(c["K"], c["N"])
        Cin = o.fill_uniform(c["M"] * c["N"], 3).reshape(c["M"], c["N"]) if c["with_c"] else None
        _check(z, cases, c["name"], o.gemm_fmaf(A, B, Cin))


def test_gemm_chain_matches_reference_cpu_gemm_config1(golden):
    """BASELINE config 1 (1024^3): bit-identical to decx::sgemm_caller's output."""
    z, cases = golden
    A = o.fill_uniform(1024 * 1024, 1).reshape(1024, 1024)
    B = o.fill_uniform(1024 * 1024, 2).reshape(1024, 1024)
    D = o.gemm_fmaf(A, B)
    assert hashlib.sha256(D.tobytes()).hexdigest() == cases["cpu_gemm_1024_sha256"]
    assert np.array_equal(D[::64, ::64], z["cpu_gemm_1024_sample"])


def test_known_answer_of_reference_test_program():
    """test/test/CUDA_GEMM/CUDA_GEMM.cpp:24-42: A[i][j] = 0.1 j, B[i][j] = 0.1 i, so every
    element of C is sum_k (0.1 k)^2 (here at 256^3 instead of 2048^3)."""
    n = 256
    A = np.tile((0.1 * np.arange(n, dtype=np.float32))[None, :], (n, 1)).astype(np.float32)
    B = np.tile((0.1 * np.arange(n, dtype=np.float32))[:, None], (1, n)).astype(np.float32)
    D = o.gemm_fmaf(A, B)
    expect = float(np.sum((0.1 * np.arange(n, dtype=np.float64)) ** 2))
    assert np.all(D == D[0, 0])
    assert abs(D[0, 0] - expect) / expect < 1e-5


def test_pack_and_conv_match_reference_kernels(golden):
    z, cases = golden
    for c in cases["conv"]:
        src = o.make_tensor(c["W"], c["H"], c["depth"], 4)
        flt = o.make_filters(c["kW"], c["kH"], c["depth"], c["N"], 5)
        _check(z, cases, "pack_" + c["name"], o.im2col_pack(src, c["W"], c["depth"], c["kW"], c["kH"], c["flag"]))
        _check(z, cases, "conv_" + c["name"], o.conv2_im2col(src, c["W"], c["depth"], flt, c["kW"], c["flag"]))


def test_pack_layout_properties():
    """Padding pixels and padding channels of the tensor travel as-is; the apron is zero."""
    W, H, C, kW, kH = 6, 5, 3, 3, 3
    src = o.make_tensor(W, H, C, 4)
    P = o.im2col_pack(src, W, C, kW, kH, 1).reshape(H, 8, kH, kW, 4)
    assert np.array_equal(P[:, :, 1, 1, :], src)                       # centre tap = the tensor itself
    assert np.all(P[0, :, 0, :, :] == 0) and np.all(P[:, 0, :, 0, :] == 0)   # top / left apron
    assert np.all(P[..., 3] == 0)                                      # padding channel


@pytest.mark.skipif(o.ref_kernels() is None, reason="oracle/_ref not built")
def test_against_reference_code_directly():
    rng_cases = [(10, 9, 5, 3, 5, 3, 1), (21, 6, 4, 5, 3, 7, 0), (64, 17, 12, 3, 3, 40, 1)]
    for W, H, C, kW, kH, N, flag in rng_cases:
        src = o.make_tensor(W, H, C, 11)
        flt = o.make_filters(kW, kH, C, N, 12)
        assert np.array_equal(o.im2col_pack(src, W, C, kW, kH, flag).view(np.uint32),
                              o.ref_im2col_pack(src, W, C, kW, kH, flag).view(np.uint32))
        assert np.array_equal(o.conv2_im2col(src, W, C, flt, kW, flag).view(np.uint32),
                              o.ref_conv2_im2col(src, W, C, flt, kW, flag).view(np.uint32))
    A = o.fill_uniform(130 * 40, 7).reshape(130, 40)
    B = o.fill_uniform(40 * 200, 8).reshape(40, 200)
    assert np.array_equal(o.gemm_fmaf(A, B), o.ref_gemm_spec(A, B))


@pytest.mark.skipif(not o.ref_cpu_available(), reason="oracle/_ref not built")
def test_reference_cpu_gemm_runs_and_matches(tmp_path):
    f = str(tmp_path / "c.bin")
    r = o.ref_cpu_gemm(256, 128, 192, reps=1, out=f, split=(2, 2))
    assert r["gflops"] > 0
    A = o.fill_uniform(256 * 192, 1).reshape(256, 192)
    B = o.fill_uniform(192 * 128, 2).reshape(192, 128)
    assert np.array_equal(np.fromfile(f, dtype=np.float32).reshape(256, 128), o.gemm_fmaf(A, B))


def test_activation_restatement_known_values():
    """ReLU / sigmoid / tanh as the reference's operators define them (nn/operators/ReLU.h:48-75,
    sigmoid.h:45-46, tanh.h:41-42), bias added first."""
    x = np.array([[-2.0, -0.0, 0.0, 0.5, 3.0]], dtype=np.float32)
    assert np.array_equal(o.bias_activation(x, None, 1), np.array([[0, 0, 0, 0.5, 3.0]], dtype=np.float32))
    s = o.bias_activation(x, None, 2)
    assert np.allclose(s, 1.0 / (1.0 + np.exp(-x.astype(np.float64))), atol=1e-7) and s[0, 2] == 0.5
    t = o.bias_activation(x, None, 3)
    assert np.allclose(t, np.tanh(x.astype(np.float64)), atol=2e-7) and t[0, 2] == 0.0
    b = np.array([1, 1, 1, 1, -5], dtype=np.float32)
    assert np.array_equal(o.bias_activation(x, b, 1), np.array([[0, 1, 1, 1.5, 0]], dtype=np.float32))


def test_half_chain_restatement():
    """The reference's fp16 GEMM accumulates in half: integer-valued inputs small enough to stay
    exact must reproduce the exact product; random inputs must show half-precision error."""
    A = np.arange(12, dtype=np.float16).reshape(3, 4) - 5
    B = (np.arange(20, dtype=np.float16).reshape(4, 5) % 7) - 3
    assert np.array_equal(o.gemm_f16_half_chain(A, B).astype(np.float64), o.gemm_f16_exact(A, B))
    A = o.fill_uniform(32 * 256, 1).reshape(32, 256); B = o.fill_uniform(256 * 16, 2).reshape(256, 16)
    err = np.abs(o.gemm_f16_half_chain(A, B).astype(np.float64) - o.gemm_f16_exact(A, B)).max()
    assert 1e-4 < err < 0.2
