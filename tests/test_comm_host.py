"""Failure detection of the gather layer, on the host: a rank that never arrives, a communicator
that reports an asynchronous error.  The other ranks are played by a stand-in for libnccl
(tests/fake_nccl.c) that the library loads in place of the real one; no GPU and no network are
involved, and nothing faults.  The joining half of decxb_comm_init runs as it does in production:
non-blocking init, bounded poll of ncclCommGetAsyncError, abort on expiry."""
import ctypes as C
import os
import subprocess
import time
from pathlib import Path

import pytest

import backup_1_b200 as b

HERE = Path(__file__).resolve().parent


@pytest.fixture(scope="module")
def fake(tmp_path_factory):
    so = tmp_path_factory.mktemp("fake_nccl") / "libfake_nccl.so"
    subprocess.run(["gcc", "-O1", "-shared", "-fPIC", "-fvisibility=hidden", "-o", str(so), str(HERE / "fake_nccl.c")], check=True)
    lib = C.CDLL(str(so))
    lib.fake_nccl_count.argtypes = [C.c_int]
    return str(so), lib


def handshake(path, mode, timeout_ms, world=2, rank=0):
    os.environ["FAKE_NCCL_MODE"] = mode
    L = b.load_library()
    err = C.create_string_buffer(300)
    t0 = time.perf_counter()
    rc = L.decxb_comm_selftest_handshake(path.encode(), world, rank, b"\x5a" * 128, timeout_ms, err, len(err))
    return rc, err.value.decode(), time.perf_counter() - t0


def test_all_ranks_join(fake):
    path, lib = fake
    lib.fake_nccl_reset()
    rc, msg, _ = handshake(path, "ok", 500)
    assert rc == 0, msg
    assert lib.fake_nccl_count(0) == 1 and lib.fake_nccl_count(1) == 0 and lib.fake_nccl_count(2) == 1


def test_a_rank_that_arrives_late_within_the_limit(fake):
    path, lib = fake
    lib.fake_nccl_reset()
    rc, msg, dt = handshake(path, "late", 2000)
    assert rc == 0, msg
    assert 0.14 <= dt < 1.5 and lib.fake_nccl_count(3) > 10 and lib.fake_nccl_count(1) == 0


def test_a_rank_that_never_arrives_times_out_and_the_communicator_is_aborted(fake):
    path, lib = fake
    lib.fake_nccl_reset()
    rc, msg, dt = handshake(path, "never", 200)
    assert rc == 103 and "did not complete within 200 ms" in msg and "aborted" in msg
    assert 0.19 <= dt < 1.5
    assert lib.fake_nccl_count(1) == 1 and lib.fake_nccl_count(2) == 0      # aborted, not destroyed


def test_an_asynchronous_error_aborts_the_communicator(fake):
    path, lib = fake
    lib.fake_nccl_reset()
    rc, msg, dt = handshake(path, "fail", 5000)
    assert rc == 105 and "system error" in msg
    assert dt < 1.0 and lib.fake_nccl_count(1) == 1


def test_bad_arguments_and_missing_library(fake):
    path, _ = fake
    assert handshake(path, "ok", 100, world=2, rank=2)[0] == 13
    rc, msg, _ = handshake("/nonexistent/libnccl.so", "ok", 100)
    assert rc == 105 and "cannot load" in msg
