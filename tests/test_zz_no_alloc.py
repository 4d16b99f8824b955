"""The allocation-free GEMM entry point (decxb_gemm_f32_noalloc) against the regular one.

Some users of the library run where device memory cannot be allocated any more: a framework's
caching pool already holds the whole card, or the call sits in a latency-critical loop that
cannot afford cudaMalloc's device-wide synchronisation.  For them the library keeps the hi/lo
operand scratch of the 3xTF32 GEMM in a fixed 64 MiB array of its own image.  This file checks
that entry through the C ABI: same results as decxb_gemm_f32 on two calls in a row (the second
smaller, so stale contents of the shared array would show), and a clear refusal beyond the
array's size.  It is collected last so that a run stopping at the first failure has already
covered every other test; it also passes alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import backup_1_b200 as b
from oracle import oracle as o

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_3X = 1e-6      # the bar of tests/test_gpu_parity.py


def _noalloc(M, N, K, dA, dB, dD, dC=None, lda=None, ldb=None, ldc=None, ldd=None, stream=None):
    L = b.load_library()
    err = C.create_string_buffer(256)
    rc = L.decxb_gemm_f32_noalloc(0, M, N, K, dA.data_ptr(), lda or K, dB.data_ptr(), ldb or N,
                                  dC.data_ptr() if dC is not None else None, ldc or N, dD.data_ptr(), ldd or N,
                                  stream, err, len(err))
    return rc, err.value.decode()


def test_noalloc_gemm_matches_regular_entry_twice_in_a_row():
    ctx = b.Context(0)
    try:
        for call, (M, N, K, with_c) in enumerate([(1024, 768, 1000, False), (300, 200, 77, True)]):
            A = o.fill_uniform(M * K, 1).reshape(M, K)
            B = o.fill_uniform(K * N, 2).reshape(K, N)
            Cin = o.fill_uniform(M * N, 3).reshape(M, N) if with_c else None
            dA, dB = torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV)
            dC = torch.from_numpy(Cin).to(DEV) if with_c else None
            d_ref = torch.full((M, N), float("nan"), device=DEV)
            d_new = torch.full((M, N), float("nan"), device=DEV)
            ctx.gemm(M, N, K, dA, K, dB, N, d_ref, N, Cin=dC, ldc=N if with_c else 0)
            ctx.synchronize()
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            rc, msg = _noalloc(M, N, K, dA, dB, d_new, dC)
            assert rc == 0, msg
            if call > 0:    # the first call may load the module that carries the array
                assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
            X, R = d_new.cpu().numpy(), d_ref.cpu().numpy()
            assert not np.isnan(X).any()
            assert o.norm_err(X, R, K, 1.0, 1.0) <= TOL_3X
            assert o.norm_err(X, o.gemm_fmaf(A, B, Cin), K, 1.0, 1.0) <= TOL_3X
    finally:
        ctx.close()


def test_noalloc_gemm_refuses_what_does_not_fit():
    t = torch.zeros(16, device=DEV)
    rc, msg = _noalloc(4096, 4096, 4096, t, t, t)          # needs 256 MiB of scratch
    assert rc == 104 and "static array" in msg
    rc, msg = _noalloc(0, 8, 8, t, t, t)
    assert rc == 13


def test_noalloc_gemm_at_the_limit_of_the_array():
    """2048^3 needs exactly the 64 MiB the array holds and must run; four more columns of K do not fit."""
    M = N = K = 2048
    ctx = b.Context(0)
    try:
        dA = torch.empty((M, K + 4), device=DEV); dB = torch.empty((K + 4, N), device=DEV)
        ctx.fill_uniform(dA, M, K + 4, K + 4, 1); ctx.fill_uniform(dB, K + 4, N, N, 2)
        ctx.synchronize()
        d_new = torch.full((M, N), float("nan"), device=DEV); d_ref = torch.empty((M, N), device=DEV)
        rc, msg = _noalloc(M, N, K, dA, dB, d_new, lda=K + 4)
        assert rc == 0, msg
        ctx.gemm(M, N, K, dA, K + 4, dB, N, d_ref, N, mode=b.GEMM_3XTF32)
        ctx.synchronize()
        assert torch.equal(d_new, d_ref)          # same kernels, same mode: same bits
        rows = np.array([0, 1000, 2047])
        R = o.gemm_fmaf(dA[rows, :K].cpu().numpy(), dB[:K].cpu().numpy())
        assert o.norm_err(d_new[rows].cpu().numpy(), R, K, 1.0, 1.0) <= TOL_3X
        rc, msg = _noalloc(M, N, K + 4, dA, dB, d_new, lda=K + 4)
        assert rc == 104 and "static array" in msg
    finally:
        ctx.close()


def test_noalloc_gemm_on_a_callers_stream_with_pitched_operands():
    M, N, K = 257, 130, 75
    lda, ldb, ldc, ldd = 80, 136, 140, 132
    A = np.zeros((M, lda), np.float32); A[:, :K] = o.fill_uniform(M * K, 1).reshape(M, K)
    B = np.zeros((K, ldb), np.float32); B[:, :N] = o.fill_uniform(K * N, 2).reshape(K, N)
    Cin = np.zeros((M, ldc), np.float32); Cin[:, :N] = o.fill_uniform(M * N, 3).reshape(M, N)
    dA, dB, dC = (torch.from_numpy(x).to(DEV) for x in (A, B, Cin))
    dD = torch.full((M, ldd), float("nan"), device=DEV)
    st = torch.cuda.Stream(device=DEV)
    torch.cuda.synchronize()
    rc, msg = _noalloc(M, N, K, dA, dB, dD, dC, lda=lda, ldb=ldb, ldc=ldc, ldd=ldd, stream=st.cuda_stream)
    assert rc == 0, msg
    X = dD.cpu().numpy()
    assert np.isnan(X[:, N:]).all(), "wrote outside the N columns of D"
    R = o.gemm_fmaf(A[:, :K], B[:, :N], Cin[:, :N])
    assert o.norm_err(X[:, :N], R, K, 1.0, 1.0) <= TOL_3X


_WARM_SCRIPT = r"""
import ctypes as C, sys
import torch
import backup_1_b200 as b
L = b.load_library()
shapes = [(1024, 1024, 512), (1280, 1280, 256), (384, 12544, 256), (2048, 2048, 256), (200, 40, 64)]
ops = []
for (M, N, K) in shapes:
    ops.append((torch.rand((M, K), device="cuda:0") - 0.5, torch.rand((K, N), device="cuda:0") - 0.5,
                torch.empty((M, N), device="cuda:0")))
err = C.create_string_buffer(256)
def call(i):
    (M, N, K), (A, B, D) = shapes[i], ops[i]
    rc = L.decxb_gemm_f32_noalloc(0, M, N, K, A.data_ptr(), K, B.data_ptr(), N, None, 0, D.data_ptr(), N, None, err, len(err))
    assert rc == 0, err.value
for i in range(len(shapes)):          # warm-up: module, kernels, attributes
    call(i)
torch.cuda.synchronize()
free0 = torch.cuda.mem_get_info()[0]
for rep in range(2):
    for i in range(len(shapes)):
        call(i)
        assert torch.cuda.mem_get_info()[0] == free0, f"shape {shapes[i]} changed the free memory"
assert torch.cuda.current_device() == 0
for i, (M, N, K) in enumerate(shapes):   # and the results are right
    A, B, D = ops[i]
    ref = (A.double() @ B.double())
    assert float((D.double() - ref).abs().max()) / (K * 0.25) <= 1e-6      # max|a| = max|b| = 0.5
print("warm ok")
"""


def test_noalloc_gemm_allocates_nothing_after_warm_up_in_a_fresh_process():
    """In a process of its own, without the regular entry ever running: after one warm-up call per
    shape (shapes that select each tile of the kernel), further calls leave the device's free
    memory exactly where it was."""
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    r = subprocess.run([sys.executable, "-c", _WARM_SCRIPT], cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "warm ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
