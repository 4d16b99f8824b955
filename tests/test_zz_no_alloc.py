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


def _noalloc(M, N, K, dA, dB, dD, dC=None):
    L = b.load_library()
    err = C.create_string_buffer(256)
    rc = L.decxb_gemm_f32_noalloc(0, M, N, K, dA.data_ptr(), K, dB.data_ptr(), N,
                                  dC.data_ptr() if dC is not None else None, N, dD.data_ptr(), N,
                                  None, err, len(err))
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
