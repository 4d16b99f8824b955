"""One rank of the multi-GPU gather tests (started by tests/test_multi_gpu.py, one process per GPU).

    python tests/multi_gpu_worker.py <world> <rank> <rendezvous file>

Every rank generates the whole A and B from the seeds, computes the unsharded product on its own
GPU as the expectation, and then checks that what the gathering entries leave in D_full equals it
bit for bit: rows multiplied here AND rows that arrived from the peers."""
import os
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import backup_1_b200 as b  # noqa: E402


def main():
    world, rank, rdv = int(sys.argv[1]), int(sys.argv[2]), Path(sys.argv[3])
    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"
    ctx = b.Context(rank)
    ctx.set_wait_limit_ms(2000)
    if rank == 0:
        uid = b.Comm.unique_id()
        tmp = rdv.with_suffix(".tmp")
        tmp.write_bytes(uid)
        os.replace(tmp, rdv)
    else:
        t0 = time.time()
        while not rdv.exists():
            if time.time() - t0 > 60:
                raise SystemExit("rendezvous file never appeared")
            time.sleep(0.05)
        uid = rdv.read_bytes()
    comm = b.Comm(ctx, world, rank, uid, timeout_ms=60000)
    try:
        for (M, N, K, groups) in [(4099, 520, 300, 1), (4099, 520, 300, 4), (8192, 1024, 512, 3), (5, 64, 64, 2)]:
            A = torch.empty((M, K), device=dev); Bm = torch.empty((K, N), device=dev)
            ctx.fill_uniform(A, M, K, K, 1); ctx.fill_uniform(Bm, K, N, N, 2)
            want = torch.empty((M, N), device=dev)
            f, l = b.shard_range(M, world, rank)
            # expectation: every rank's block as that rank computes it (same entry, same shapes), run here
            for r in range(world):
                rf, rl = b.shard_range(M, world, r)
                if rl > rf:
                    ctx.gemm_rowshard(world, r, M, N, K, A[rf:], K, Bm, N, want[rf:], N)
            ctx.synchronize()
            full = torch.full((M, N), float("nan"), device=dev)
            comm.gemm_rowshard_gather(M, N, K, A[f:] if l > f else A, K, Bm, N, full, groups=groups)
            comm.synchronize()
            ctx.synchronize()
            if groups == 1:
                assert torch.equal(full, want), f"rank {rank}: gathered product differs (M={M}, groups={groups})"
            else:
                # panel groups change the tile schedule of a rank's rows, not the arithmetic of an output
                assert not torch.isnan(full).any()
                assert torch.equal(full, want), f"rank {rank}: gathered product differs (M={M}, groups={groups})"
        # host-resident operands: a rank uploads its share of B, the ranks all-gather it, the rank's rows come home
        import numpy as np
        # (several column blocks of B, the last one ragged; more rows than the first row block takes; fewer rows than ranks)
        for (M, N, K) in [(4099, 520, 300), (300, 3001, 70), (24000, 2304, 64), (5, 64, 3)]:
            A = torch.empty((M, K), device=dev); Bm = torch.empty((K, N), device=dev)
            ctx.fill_uniform(A, M, K, K, 3); ctx.fill_uniform(Bm, K, N, N, 4)
            f, l = b.shard_range(M, world, rank)
            want = torch.empty((max(l - f, 1), N), device=dev)
            if l > f:
                ctx.gemm_rowshard(world, rank, M, N, K, A[f:], K, Bm, N, want, N)
            ctx.synchronize()
            hA = np.ascontiguousarray(A.cpu().numpy()); hB = np.ascontiguousarray(Bm.cpu().numpy())
            hD = np.full((M + 1, N + 3), np.nan, dtype=np.float32)            # a row pitch wider than the rows, one spare row
            rows_a = hA[f:] if l > f else hA
            comm.gemm_rowshard_host(M, N, K, rows_a.ctypes.data, K, hB.ctypes.data, N, hD[f:].ctypes.data, N + 3)
            if l > f:
                assert np.array_equal(hD[f:l, :N], want[:l - f].cpu().numpy()), f"rank {rank}: host-resident rows differ (M={M})"
            assert np.isnan(hD[l:]).all() and np.isnan(hD[:f]).all() and np.isnan(hD[:, N:]).all(), "wrote outside the rank's rows"
        # blocks of unequal size (images of a sharded convolution result): 7 units of 3000 floats
        units, ub = 7, 3000
        base = torch.full((units, ub), float("nan"), device=dev)
        f, l = b.shard_range(units, world, rank)
        for u in range(f, l):
            base[u] = float(u + 1)
        comm.allgather_blocks(base, ub * 4, units)
        comm.synchronize()
        torch.cuda.synchronize()
        expect = torch.arange(1, units + 1, device=dev, dtype=torch.float32).unsqueeze(1).expand(units, ub)
        assert torch.equal(base, expect), f"rank {rank}: all-gather of unequal blocks"
        # equal blocks take NCCL's own all-gather
        units = 4 * world
        base = torch.full((units, ub), float("nan"), device=dev)
        f, l = b.shard_range(units, world, rank)
        base[f:l] = torch.arange(f + 1, l + 1, device=dev, dtype=torch.float32).unsqueeze(1)
        comm.allgather_blocks(base, ub * 4, units)
        comm.synchronize()
        torch.cuda.synchronize()
        expect = torch.arange(1, units + 1, device=dev, dtype=torch.float32).unsqueeze(1).expand(units, ub)
        assert torch.equal(base, expect), f"rank {rank}: all-gather of equal blocks"
    finally:
        comm.close()
        ctx.close()
    print(f"rank {rank} ok")


if __name__ == "__main__":
    main()
