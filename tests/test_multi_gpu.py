"""The gathering entries over real NCCL, one process per GPU (needs at least two GPUs; with one GPU
only the single-rank cases run).  No rank fails here: failure detection is tested on the host in
tests/test_comm_host.py."""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import backup_1_b200 as b
from oracle import oracle as o

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def test_single_rank_communicator_runs_the_panel_groups(ctx):
    """world = 1: NCCL is loaded and joined, nothing travels; the row-panel groups assemble the product."""
    M, N, K = 1500, 264, 200
    A = o.fill_uniform(M * K, 1).reshape(M, K); B = o.fill_uniform(K * N, 2).reshape(K, N)
    dA, dB = torch.from_numpy(A).to("cuda:0"), torch.from_numpy(B).to("cuda:0")
    comm = b.Comm(ctx, 1, 0, b.Comm.unique_id(), timeout_ms=20000)
    try:
        want = torch.empty((M, N), device="cuda:0")
        ctx.gemm(M, N, K, dA, K, dB, N, want, N)
        for groups in (1, 4):
            full = torch.full((M, N), float("nan"), device="cuda:0")
            comm.gemm_rowshard_gather(M, N, K, dA, K, dB, N, full, groups=groups)
            comm.synchronize(); ctx.synchronize()
            assert torch.equal(full, want)
        assert o.norm_err(want[:32].cpu().numpy(), o.gemm_fmaf(A[:32], B), K, 1.0, 1.0) <= 1e-6
    finally:
        comm.close()


def test_single_rank_host_resident_product_with_b_in_shares(ctx):
    """world = 1: the host-resident sharded entry uploads 'its share' (all) of each column block of B, gathers it
    (nothing travels) and returns the bits of the device-resident product; a CUDA call that fails in the middle
    (injected on the host) is reported, and the same call then succeeds."""
    comm = b.Comm(ctx, 1, 0, b.Comm.unique_id(), timeout_ms=20000)
    try:
        for (M, N, K) in [(1500, 264, 200), (700, 3001, 70), (11000, 2304, 36)]:
            A = o.fill_uniform(M * K, 1).reshape(M, K); B = o.fill_uniform(K * N, 2).reshape(K, N)
            dA, dB = torch.from_numpy(A).to("cuda:0"), torch.from_numpy(B).to("cuda:0")
            want = torch.empty((M, N), device="cuda:0")
            ctx.gemm(M, N, K, dA, K, dB, N, want, N)
            ctx.synchronize()
            hD = np.full((M, N + 5), np.nan, dtype=np.float32)
            comm.gemm_rowshard_host(M, N, K, A, K, B, N, hD, N + 5)
            assert np.array_equal(hD[:, :N], want.cpu().numpy())
            assert np.isnan(hD[:, N:]).all()
        M, N, K = 1500, 264, 200
        A = o.fill_uniform(M * K, 1).reshape(M, K); B = o.fill_uniform(K * N, 2).reshape(K, N)
        hD = np.full((M, N), np.nan, dtype=np.float32)
        good = hD.copy()
        comm.gemm_rowshard_host(M, N, K, A, K, B, N, good, N)
        L = b.load_library()
        for nth in (0, 3, 6):
            assert L.decxb_inject_pipeline_error(ctx.h, nth) == 0
            with pytest.raises(b.DecxbError):
                comm.gemm_rowshard_host(M, N, K, A, K, B, N, hD, N)
            L.decxb_inject_pipeline_error(ctx.h, -1)
            hD[:] = np.nan
            comm.gemm_rowshard_host(M, N, K, A, K, B, N, hD, N)
            assert np.array_equal(hD, good)
    finally:
        comm.close()


def test_prepared_b_gives_the_bits_of_the_plain_entry(ctx):
    M, N, K = 700, 328, 260
    A = o.fill_uniform(M * K, 1).reshape(M, K); B = o.fill_uniform(K * N, 2).reshape(K, N)
    Cin = o.fill_uniform(M * N, 3).reshape(M, N); bias = o.fill_uniform(N, 9)
    dA, dB, dC, dbias = (torch.from_numpy(x).to("cuda:0") for x in (A, B, Cin, bias))
    for mode in (b.GEMM_DEFAULT, b.GEMM_3XTF32, b.GEMM_1XTF32):
        want = torch.empty((M, N), device="cuda:0"); got = torch.full((M, N), float("nan"), device="cuda:0")
        ctx.gemm_act(M, N, K, dA, K, dB, N, want, N, Cin=dC, ldc=N, bias=dbias, act=b.ACT_RELU, mode=mode)
        pb = ctx.prepare_b(K, N, dB, N, mode=mode)
        ctx.synchronize()                                 # the preparation runs on the context's stream
        dB_saved = dB.clone(); dB.zero_()                 # B itself is no longer needed once prepared
        torch.cuda.synchronize()
        for _ in range(2):
            ctx.gemm_prepared(M, dA, K, pb, got, N, Cin=dC, ldc=N, bias=dbias, act=b.ACT_RELU)
        ctx.synchronize()
        dB.copy_(dB_saved)
        assert torch.equal(got, want)
        with pytest.raises(b.DecxbError):
            ctx.gemm_prepared(M, dA, K - 1, pb, got, N)   # lda < K
        ctx.release_b(pb)


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("world", [2, 4, 8])
def test_gather_over_nccl_one_process_per_gpu(world, tmp_path):
    if _ngpu() < world:
        pytest.skip(f"needs {world} GPUs")
    rdv = tmp_path / "nccl_id.bin"
    procs = [subprocess.Popen([sys.executable, str(HERE / "multi_gpu_worker.py"), str(world), str(r), str(rdv)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} ok" in out, f"rank {r}:\n{out[-3000:]}"


_NEVER_JOINS = r"""
import sys, time
import torch
import backup_1_b200 as b
ctx = b.Context(0)
uid = b.Comm.unique_id()
t0 = time.perf_counter()
try:
    b.Comm(ctx, 2, 0, uid, timeout_ms=1500)        # rank 1 of 2 is never started
    print("joined?!"); sys.exit(1)
except b.DecxbError as e:
    dt = time.perf_counter() - t0
    assert e.status == 103, e
    assert 1.4 <= dt < 30.0, dt
# the context (and NCCL) are still usable: a single-rank communicator and a product
c = b.Comm(ctx, 1, 0, b.Comm.unique_id(), timeout_ms=20000)
A = torch.rand((256, 64), device="cuda:0"); B = torch.rand((64, 256), device="cuda:0"); D = torch.empty((256, 256), device="cuda:0")
c.gemm_rowshard_gather(256, 256, 64, A, 64, B, 256, D, groups=2)
c.synchronize(); ctx.synchronize()
assert float((D.double() - A.double() @ B.double()).abs().max()) / 64 <= 1e-6
c.close(); ctx.close()
print("never-joins ok")
"""


def test_a_rank_that_never_joins_times_out_with_the_real_library():
    """Over the real NCCL: rank 0 of 2 waits for a rank that is never started; the join gives up after its
    limit with DECXB_ERR_TIMEOUT (no kernel is in flight at that point, nothing on the GPU is touched), and the
    process goes on to use the GPU.  Runs in a child process so that a stuck join could not stall the suite."""
    r = subprocess.run([sys.executable, "-c", _NEVER_JOINS], cwd=HERE.parent, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0 and "never-joins ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
