"""The N>1 path on CPU: two gloo ranks shard a GEMM by rows and a convolution by images, compute
their shards with the oracle (the stand-in for the per-rank GPU call) and all-gather the
result; the gathered tensor must equal the unsharded computation bit for bit."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from backup_1_b200 import shard
from oracle import oracle as o


def test_block_range_partitions_exactly():
    for total in (0, 1, 7, 256, 8192, 32768):
        for world in (1, 2, 3, 4, 8):
            spans = [shard.block_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert shard.gemm_row_shard(32768, 8, 3) == (12288, 16384)
    assert shard.conv_batch_shard(256, 8, 7) == (224, 256)


def test_library_partition_rule_equals_the_python_one():
    """The C-ABI rule (decxb_shard_range, what a non-Python host binds) and shard.block_range
    must be the same function."""
    import backup_1_b200 as b
    for total in (0, 1, 5, 7, 255, 256, 257, 8192, 32768, 10 ** 12 + 7):
        for world in (1, 2, 3, 4, 5, 8, 16):
            for rank in range(world):
                assert b.shard_range(total, world, rank) == shard.block_range(total, world, rank)
    for bad in ((10, 0, 0), (10, 2, 2), (10, 2, -1), (-1, 2, 0)):
        try:
            b.shard_range(*bad)
        except b.DecxbError:
            continue
        raise AssertionError(f"{bad} accepted")


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 101, 64, 48                       # 101 rows: uneven shards
        A = o.fill_uniform(M * K, 1).reshape(M, K)
        B = o.fill_uniform(K * N, 2).reshape(K, N)
        r0, r1 = shard.gemm_row_shard(M, world, rank)
        local = torch.from_numpy(o.gemm_fmaf(A[r0:r1], B))
        full = shard.all_gather_blocks(local, M)
        ok_gemm = np.array_equal(full.numpy(), o.gemm_fmaf(A, B))
        W, H, C, kW, F, nb = 10, 6, 4, 3, 8, 4      # even shards: the single-call gather path
        imgs = np.stack([o.make_tensor(W, H, C, 4, first_index=i * 1009) for i in range(nb)])
        flt = o.make_filters(kW, kW, C, F, 5)
        b0, b1 = shard.conv_batch_shard(nb, world, rank)
        loc = torch.from_numpy(np.stack([o.conv2_im2col(imgs[i], W, C, flt, kW, 1) for i in range(b0, b1)]))
        fullc = shard.all_gather_blocks(loc, nb)
        ref = np.stack([o.conv2_im2col(imgs[i], W, C, flt, kW, 1) for i in range(nb)])
        ok_conv = np.array_equal(fullc.numpy(), ref)
        q.put((rank, ok_gemm, ok_conv))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_gather():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] and r[2] for r in res)
