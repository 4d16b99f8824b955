"""ctypes/numpy front end of the test oracle.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg
import this module; the product package never does.

Three things live behind it:

* ``libdecx_oracle.so``  - the plain-C restatement (``decx_oracle.c``).
* ``_ref/libdecx_ref_kernels_host.so`` - the reference's own CUDA kernel
  sources executed on host threads (``ref_kernels_host.cpp``); optional.
* ``_ref/decx_ref_cpu`` - the reference's own CPU GEMM as a command-line
  program (``ref_cpu_gemm.cpp``); optional, used for the timed CPU baseline.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_F = np.float32


def _build_oracle() -> Path:
    so = HERE / "libdecx_oracle.so"
    src = HERE / "decx_oracle.c"
    if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-s", "-C", str(HERE), "oracle"], check=True)
    return so


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        L = C.CDLL(str(_build_oracle()))
        i64, u64, u32, fp, dp = C.c_int64, C.c_uint64, C.c_uint32, C.c_void_p, C.c_void_p
        L.decxo_fill_uniform.argtypes = [fp, u64, u32, u64]
        L.decxo_fill_uniform_2d.argtypes = [fp, u64, u64, u64, u32, u64]
        L.decxo_gemm_fmaf.argtypes = [i64, i64, i64, fp, i64, fp, i64, fp, i64, fp, i64]
        L.decxo_gemm_fmaf_nt.argtypes = [i64, i64, i64, fp, i64, fp, i64, fp, i64]
        L.decxo_gemm_f64.argtypes = [i64, i64, i64, fp, i64, fp, i64, fp, i64, dp, i64]
        L.decxo_im2col_pack.argtypes = [fp, i64, i64, i64, i64, i64, C.c_int, fp]
        L.decxo_im2col_pack.restype = C.c_int
        L.decxo_kernel_matrix.argtypes = [fp, i64, i64, i64, i64, i64, i64, fp]
        L.decxo_conv2_im2col.argtypes = [fp, i64, i64, i64, fp, i64, i64, i64, C.c_int, fp]
        L.decxo_conv2_im2col.restype = C.c_int
        L.decxo_bias_activation.argtypes = [fp, i64, i64, i64, fp, C.c_int]
        L.decxo_num_threads.restype = C.c_int
        L.decxo_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def ceil4(v: int) -> int:
    return (v + 3) // 4 * 4


# ----------------------------------------------------------------------------
# seeded data
# ----------------------------------------------------------------------------
def fill_uniform(n: int, seed: int, first_index: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=_F)
    lib().decxo_fill_uniform(_p(out), n, seed, first_index)
    return out


def fill_uniform_2d(rows: int, cols: int, pitch: int, seed: int, first_index: int = 0) -> np.ndarray:
    out = np.empty((rows, pitch), dtype=_F)
    lib().decxo_fill_uniform_2d(_p(out), rows, cols, pitch, seed, first_index)
    return out


def make_tensor(W: int, H: int, depth: int, seed: int, first_index: int = 0) -> np.ndarray:
    """A DECX tensor (HWC, padded) as an array [H][wpitch][dpitch]; padding is zero."""
    wp, dp = ceil4(W), ceil4(depth)
    t = np.zeros((H, wp, dp), dtype=_F)
    vals = fill_uniform(H * W * depth, seed, first_index).reshape(H, W, depth)
    t[:, :W, :depth] = vals
    return t


def make_filters(kW: int, kH: int, depth: int, N: int, seed: int) -> np.ndarray:
    """A DECX TensorArray of N filters: [N][kH][ceil4(kW)][dpitch]; padding is zero."""
    kwp, dp = ceil4(kW), ceil4(depth)
    t = np.zeros((N, kH, kwp, dp), dtype=_F)
    vals = fill_uniform(N * kH * kW * depth, seed).reshape(N, kH, kW, depth)
    t[:, :, :kW, :depth] = vals
    return t


# ----------------------------------------------------------------------------
# restated algorithms
# ----------------------------------------------------------------------------
def gemm_fmaf(A: np.ndarray, B: np.ndarray, Cin: np.ndarray | None = None) -> np.ndarray:
    """D = A @ B (+ Cin) as one ascending-k fp32 fma chain per output."""
    A = np.ascontiguousarray(A, dtype=_F)
    B = np.ascontiguousarray(B, dtype=_F)
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    if Cin is not None:
        Cin = np.ascontiguousarray(Cin, dtype=_F)
    D = np.empty((M, N), dtype=_F)
    lib().decxo_gemm_fmaf(M, N, K, _p(A), K, _p(B), N, _p(Cin), N, _p(D), N)
    return D


def gemm_f64(A: np.ndarray, B: np.ndarray, Cin: np.ndarray | None = None) -> np.ndarray:
    A = np.ascontiguousarray(A, dtype=_F)
    B = np.ascontiguousarray(B, dtype=_F)
    M, K = A.shape
    _, N = B.shape
    if Cin is not None:
        Cin = np.ascontiguousarray(Cin, dtype=_F)
    D = np.empty((M, N), dtype=np.float64)
    lib().decxo_gemm_f64(M, N, K, _p(A), K, _p(B), N, _p(Cin), N, _p(D), N)
    return D


def gemm_f16_half_chain(A: np.ndarray, B: np.ndarray, Cin: np.ndarray | None = None) -> np.ndarray:
    """The reference's fp16 GEMM arithmetic: every output is one chain of HALF-precision fused
    multiply-adds in ascending k, c = round_half(a*b + c) (__hfma2 in the macro hfma_8x1,
    srcs/GEMM/CUDA/GEMM_kernel_def.cuh:100-107; accumulators are half2, preloaded from C in the
    A*B+C kernel).  numpy: the product and sum are formed in float64 (exact for half inputs but for
    astronomically rare cases) and rounded to half once per step."""
    A = np.asarray(A, dtype=np.float16); B = np.asarray(B, dtype=np.float16)
    M, K = A.shape
    N = B.shape[1]
    c = np.zeros((M, N), dtype=np.float16) if Cin is None else np.asarray(Cin, dtype=np.float16).copy()
    A64, B64 = A.astype(np.float64), B.astype(np.float64)
    for k in range(K):
        c = (A64[:, k, None] * B64[None, k, :] + c.astype(np.float64)).astype(np.float16)
    return c


def gemm_f16_exact(A: np.ndarray, B: np.ndarray, Cin: np.ndarray | None = None) -> np.ndarray:
    """Exact product of half inputs in float64 (yardstick for both arithmetic variants)."""
    D = np.asarray(A, dtype=np.float16).astype(np.float64) @ np.asarray(B, dtype=np.float16).astype(np.float64)
    return D if Cin is None else D + np.asarray(Cin, dtype=np.float16).astype(np.float64)


def conv_geometry(W, H, depth, kW, kH, flag):
    """(out_w, out_h, eq_w, M, Kp) of the im2col convolution."""
    if flag == 1:
        ow, oh = W, H
    elif flag == 0:
        ow, oh = W - (kW // 2) * 2, H - (kH // 2) * 2
    else:
        raise ValueError("flag")
    eq = ceil4(ow)
    return ow, oh, eq, eq * oh, kW * kH * ceil4(depth)


def im2col_pack(src: np.ndarray, W: int, depth: int, kW: int, kH: int, flag: int) -> np.ndarray:
    src = np.ascontiguousarray(src, dtype=_F)
    H = src.shape[0]
    _, _, _, M, Kp = conv_geometry(W, H, depth, kW, kH, flag)
    out = np.empty((M, Kp), dtype=_F)
    rc = lib().decxo_im2col_pack(_p(src), W, H, depth, kW, kH, flag, _p(out))
    if rc:
        raise ValueError(f"decxo_im2col_pack rc={rc}")
    return out


def kernel_matrix(filters: np.ndarray, kW: int, depth: int, n_rows: int | None = None, ld: int | None = None):
    filters = np.ascontiguousarray(filters, dtype=_F)
    N, kH = filters.shape[0], filters.shape[1]
    Kp = kW * kH * ceil4(depth)
    n_rows = ceil4(N) if n_rows is None else n_rows
    ld = Kp if ld is None else ld
    out = np.empty((n_rows, ld), dtype=_F)
    lib().decxo_kernel_matrix(_p(filters), kW, kH, depth, N, n_rows, ld, _p(out))
    return out


def conv2_im2col(src: np.ndarray, W: int, depth: int, filters: np.ndarray, kW: int, flag: int) -> np.ndarray:
    """Destination tensor in its padded layout [out_h][eq_w][ceil4(N)]."""
    src = np.ascontiguousarray(src, dtype=_F)
    filters = np.ascontiguousarray(filters, dtype=_F)
    H = src.shape[0]
    N, kH = filters.shape[0], filters.shape[1]
    _, oh, eq, _, _ = conv_geometry(W, H, depth, kW, kH, flag)
    out = np.empty((oh, eq, ceil4(N)), dtype=_F)
    rc = lib().decxo_conv2_im2col(_p(src), W, H, depth, _p(filters), kW, kH, N, flag, _p(out))
    if rc:
        raise ValueError(f"decxo_conv2_im2col rc={rc}")
    return out


def bias_activation(X: np.ndarray, bias: np.ndarray | None, act: int) -> np.ndarray:
    """act(X + bias[column]) over the last axis, in place on a copy (1 ReLU, 2 sigmoid, 3 tanh)."""
    Y = np.ascontiguousarray(X, dtype=_F).copy()
    cols = Y.shape[-1]
    b = None if bias is None else np.ascontiguousarray(bias, dtype=_F)
    lib().decxo_bias_activation(_p(Y), Y.size // cols, cols, cols, _p(b), act)
    return Y


def norm_err(X: np.ndarray, R: np.ndarray, K: int, amax: float, bmax: float) -> float:
    """The parity figure: max|X - R| / (K * max|a| * max|b|)."""
    d = np.abs(X.astype(np.float64) - R.astype(np.float64)).max()
    return float(d / (K * amax * bmax))


# ----------------------------------------------------------------------------
# the reference's own code (optional: present when oracle/_ref was built)
# ----------------------------------------------------------------------------
_ref = None


def ref_kernels():
    """The reference's CUDA kernels on host threads, or None when not built."""
    global _ref
    so = HERE / "_ref" / "libdecx_ref_kernels_host.so"
    if _ref is None and so.exists():
        L = C.CDLL(str(so))
        u, fp = C.c_uint, C.c_void_p
        L.decx_ref_im2col_pack.argtypes = [fp, u, u, u, u, u, C.c_int, fp]
        L.decx_ref_conv2_im2col.argtypes = [fp, u, u, u, fp, u, u, u, C.c_int, fp]
        L.decx_ref_gemm_spec.argtypes = [u, u, u, fp, u, fp, u, fp, u, fp, u]
        _ref = L
    return _ref


_ref_gpu = None


def ref_kernels_gpu():
    """The reference's CUDA kernels compiled for sm_100a (real launches), or None when not
    built.  Only for use on a machine with a GPU."""
    global _ref_gpu
    so = HERE / "_ref" / "libdecx_ref_kernels_gpu.so"
    if _ref_gpu is None and so.exists():
        L = C.CDLL(str(so))
        u, fp = C.c_uint, C.c_void_p
        L.decx_ref_im2col_pack.argtypes = [fp, u, u, u, u, u, C.c_int, fp]
        L.decx_ref_conv2_im2col.argtypes = [fp, u, u, u, fp, u, u, u, C.c_int, fp]
        L.decx_ref_gemm_spec.argtypes = [u, u, u, fp, u, fp, u, fp, u, fp, u]
        L.decx_ref_last_kernel_ms.restype = C.c_float
        _ref_gpu = L
    return _ref_gpu


def ref_last_kernel_ms() -> float:
    """Device time of the kernel(s) of the last ref_* call made with gpu=True."""
    return float(ref_kernels_gpu().decx_ref_last_kernel_ms())


def _ref_lib(gpu: bool):
    return ref_kernels_gpu() if gpu else ref_kernels()


def ref_im2col_pack(src, W, depth, kW, kH, flag, gpu=False):
    src = np.ascontiguousarray(src, dtype=_F)
    H = src.shape[0]
    _, _, _, M, Kp = conv_geometry(W, H, depth, kW, kH, flag)
    out = np.empty((M, Kp), dtype=_F)
    rc = _ref_lib(gpu).decx_ref_im2col_pack(_p(src), W, H, depth, kW, kH, flag, _p(out))
    if rc:
        raise ValueError(f"decx_ref_im2col_pack rc={rc}")
    return out


def ref_conv2_im2col(src, W, depth, filters, kW, flag, gpu=False):
    src = np.ascontiguousarray(src, dtype=_F)
    filters = np.ascontiguousarray(filters, dtype=_F)
    H = src.shape[0]
    N, kH = filters.shape[0], filters.shape[1]
    _, oh, eq, _, _ = conv_geometry(W, H, depth, kW, kH, flag)
    out = np.empty((oh, eq, ceil4(N)), dtype=_F)
    rc = _ref_lib(gpu).decx_ref_conv2_im2col(_p(src), W, H, depth, _p(filters), kW, kH, N, flag, _p(out))
    if rc:
        raise ValueError(f"decx_ref_conv2_im2col rc={rc}")
    return out


def ref_gemm_spec(A, B, Cin=None, gpu=False):
    A = np.ascontiguousarray(A, dtype=_F)
    B = np.ascontiguousarray(B, dtype=_F)
    M, K = A.shape
    _, N = B.shape
    if Cin is not None:
        Cin = np.ascontiguousarray(Cin, dtype=_F)
    D = np.empty((M, N), dtype=_F)
    rc = _ref_lib(gpu).decx_ref_gemm_spec(M, N, K, _p(A), K, _p(B), N, _p(Cin), N, _p(D), N)
    if rc:
        raise ValueError(f"decx_ref_gemm_spec rc={rc}")
    return D


def ref_cpu_available() -> bool:
    return (HERE / "_ref" / "decx_ref_cpu").exists()


def ref_cpu_threads(M: int, N: int) -> tuple[int, int]:
    """Largest thread split <TX,TY> the reference entry accepts for (M, N) on
    the CPUs this process may use (the reference's pool arrays hold 16 slots)."""
    ncpu = min(len(os.sched_getaffinity(0)), 16)
    for tx, ty in ((4, 4), (3, 4), (4, 2), (2, 2), (1, 1)):
        if tx * ty <= ncpu and M % tx == 0 and (M // tx) % 32 == 0 and (N // 16) // ty >= 1:
            return tx, ty
    return 1, 1


def ref_cpu_gemm(M: int, N: int, K: int, A="seed:1", B="seed:2", reps: int = 3, out: str = "-",
                 split: tuple[int, int] | None = None, timeout: float = 600.0) -> dict:
    """Run the reference's CPU GEMM in a child process limited to <=16 CPUs.
    A/B are 'seed:<n>' or file names of raw float32 data."""
    tx, ty = split or ref_cpu_threads(M, N)
    # The reference's pool starts hardware_concurrency() workers into arrays of 16 slots
    # (thread_pool.h:18, :144-150, :246) and aborted inside glibc on hosts with more than 16 CPUs
    # online; the driver program now caps the count it reports (see ref_cpu_gemm.cpp).  The
    # repeat-then-degrade loop below stays as a guard: the pool also starts its workers while
    # the queues are still being constructed (thread_pool.h:126-137).
    attempts = [(tx, ty)] * 3 + [(a, b) for a, b in ((4, 2), (2, 2), (1, 1))
                                  if a * b < tx * ty and M % a == 0 and (M // a) % 32 == 0 and (N // 16) // b >= 1]
    err = ""
    for tx, ty in attempts:
        cmd = [str(HERE / "_ref" / "decx_ref_cpu"), "gemm", str(M), str(N), str(K), f"{tx}x{ty}", str(reps), A, B, out]
        env = dict(os.environ, DECX_REF_CPUS=str(max(tx * ty, 1)))
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
        if r.returncode == 0:
            break
        err = f"decx_ref_cpu failed rc={r.returncode}: {r.stderr.strip()}"
    else:
        raise RuntimeError(err)
    res = json.loads(r.stdout.strip().splitlines()[-1])
    res["split"] = f"{tx}x{ty}"
    return res
