"""The C-ABI library: builds, loads, exports every symbol the header declares, and its host
logic (geometry, argument checks) behaves.  No compute calls: CPU only."""
import ctypes as C
import re
from pathlib import Path

import pytest

import backup_1_b200 as b
from backup_1_b200 import lib as blib
from oracle import oracle as o

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "decxb.h").read_text()
    return sorted(set(re.findall(r"DECXB_API\s+[\w\s\*]+?\b(decxb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = b.load_library()
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/decxb.h but not exported"
    assert set(names) == set(blib.SIGNATURES), "python prototypes out of sync with the header"


def test_status_strings_and_version():
    L = b.load_library()
    assert L.decxb_version().startswith(b"decxb")
    assert b"initialized" in L.decxb_status_string(1)
    assert b"dims" in L.decxb_status_string(3)


def test_no_device_fails_loudly():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(b.DecxbError) as e:
        b.Context(0)
    assert e.value.status in (101, 102)


@pytest.mark.parametrize("W,H,depth,kW,kH,N,flag", [
    (224, 224, 64, 3, 3, 64, 1), (56, 56, 256, 3, 3, 256, 1), (22, 19, 6, 3, 5, 5, 0), (9, 7, 3, 3, 3, 2, 1),
])
def test_conv_geometry_matches_oracle(W, H, depth, kW, kH, N, flag):
    g = b.conv_geometry(W, H, depth, kW, kH, N, flag)
    ow, oh, eq, M, Kp = o.conv_geometry(W, H, depth, kW, kH, flag)
    assert (g.out_w, g.out_h, g.eq_w, g.M, g.Kp, g.Np) == (ow, oh, eq, M, Kp, o.ceil4(N))


def test_conv_geometry_rejects_bad_input():
    for args, status in [((8, 8, 4, 19, 3, 1, 1), 5), ((8, 8, 4, 3, 3, 1, 7), 11), ((2, 2, 4, 3, 3, 1, 0), 5), ((0, 8, 4, 3, 3, 1, 1), 13)]:
        with pytest.raises(b.DecxbError) as e:
            b.conv_geometry(*args)
        assert e.value.status == status


def test_config_sizes_of_baseline():
    g3 = b.conv_geometry(224, 224, 64, 3, 3, 64, 1)
    assert (g3.M, g3.Kp) == (50176, 576) and g3.M * g3.Kp * 4 == 115605504
    g4 = b.conv_geometry(56, 56, 256, 3, 3, 256, 1)
    assert (g4.M, g4.Kp) == (3136, 2304) and g4.M * g4.Kp * 4 == 28901376


def _host_plan(L, M, N, K, world):
    n = L.decxb_gemm_host_plan(M, N, K, world, None, 0)
    assert n >= 1
    buf = (C.c_int64 * (3 * n))()
    assert L.decxb_gemm_host_plan(M, N, K, world, buf, n) == n
    t = [tuple(buf[3 * i:3 * i + 3]) for i in range(n)]
    return [x[1:] for x in t if x[0] == 0], [x[1:] for x in t if x[0] == 1], [x[1:] for x in t if x[0] == 2]


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("dims", [(32768, 32768, 32768), (8192, 4096, 2048), (1, 1, 1), (5, 64, 3), (24000, 2304, 64),
                                  (700, 3001, 70), (4099, 520, 300), (10241, 2047, 9000), (0, 128, 128)])
def test_host_pipeline_plan_covers_every_row_and_column_once(world, dims):
    """The cut of the host-resident product (pure host arithmetic): the column blocks of B tile [0, N), the pieces
    of the first row-block followed by the later row-blocks tile [0, M), nothing is empty, and the blocks that
    the peers complete start on a 16-byte boundary of the row."""
    L = b.load_library()
    M, N, K = dims
    if M == 0 and world == 1:
        M = 1
    cols, pieces, rows = _host_plan(L, M, N, K, world)
    at = 0
    for first, count in cols:
        assert first == at and count > 0
        assert first % 4 == 0
        at += count
    assert at == N
    at = 0
    for first, count in pieces + rows:
        assert first == at and count > 0
        at += count
    assert at == M
    if M > 0:
        assert len(pieces) >= 1 and len(pieces) <= 4
    # the first row-block shrinks with the number of ranks that share the host link, never below a quarter of a tile wave
    first_rows = sum(c for _, c in pieces)
    assert first_rows <= max(10240, -(-M // 8 // 256) * 256, 512)
    if world > 1 and M >= 10240 and K >= 10240:
        assert first_rows < 10240


def test_host_pipeline_plan_rejects_bad_arguments():
    L = b.load_library()
    assert L.decxb_gemm_host_plan(-1, 8, 8, 1, None, 0) == -1
    assert L.decxb_gemm_host_plan(8, 0, 8, 1, None, 0) == -1
    assert L.decxb_gemm_host_plan(8, 8, 8, 0, None, 0) == -1
    assert L.decxb_gemm_host_plan(8, 8, 8, 1, None, 4) == -1


@pytest.mark.parametrize("world", [2, 4, 8])
def test_host_pipeline_plan_gives_every_rank_the_same_column_blocks(world):
    """Ranks of a sharded host-resident product complete each column block of B together (one collective per block),
    so the blocks must not depend on how many rows a rank owns: unequal shards, and ranks without rows, included."""
    L = b.load_library()
    for (M, N, K) in [(32768, 32768, 32768), (4099, 3001, 300), (5, 64, 3), (24001, 2304, 64)]:
        plans = []
        for rank in range(world):
            f, l = b.shard_range(M, world, rank)
            plans.append(_host_plan(L, l - f, N, K, world)[0])
        assert all(p == plans[0] for p in plans)
        # and the shares of B's rows that the ranks upload tile [0, K)
        at = 0
        for rank in range(world):
            f, l = b.shard_range(K, world, rank)
            assert f == at
            at = l
        assert at == K
