"""The debug bounds build (libdecxb_bounds.so, -DDECXB_BOUNDS): the library's memory-bound kernels with every
global load and store checked against the extent of its array.  The seeded random-geometry parity tests are
run once more against that build in a child process: they pass only if no access left its array (a caught
violation surfaces as DECXB_ERR_BOUNDS at the next synchronisation).  The self-test shows that the check
trips when it should: an extent declared one row short, on memory that is really there."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

import backup_1_b200 as b

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
BOUNDS_LIB = ROOT / "backup_1_b200" / "libdecxb_bounds.so"

_SELFTEST = r"""
import backup_1_b200 as b
L = b.load_library()
assert L.decxb_bounds_build() == 1
ctx = b.Context(0)
rc = L.decxb_selftest_bounds(ctx.h)
msg = L.decxb_last_error(ctx.h).decode()
assert rc == 106 and "bounds check" in msg and "kernel 2" in msg, (rc, msg)
ctx.synchronize()                      # the status word was cleared: the context is usable
import torch
A = torch.rand((300, 77), device="cuda:0"); B = torch.rand((77, 130), device="cuda:0"); D = torch.empty((300, 130), device="cuda:0")
ctx.gemm(300, 130, 77, A, 77, B, 130, D, 130)
ctx.synchronize()
assert float((D.double() - A.double() @ B.double()).abs().max()) / 77 <= 1e-6
ctx.close()
print("bounds selftest ok")
"""


def _env():
    return dict(os.environ, DECXB_LIBRARY=str(BOUNDS_LIB))


def test_regular_library_is_not_the_bounds_build(ctx):
    L = b.load_library()
    assert L.decxb_bounds_build() == 0
    assert L.decxb_selftest_bounds(ctx.h) == 11          # refused: built without the checks


@pytest.mark.skipif(not BOUNDS_LIB.exists(), reason="libdecxb_bounds.so not built")
def test_bounds_check_trips_on_an_extent_declared_too_short():
    r = subprocess.run([sys.executable, "-c", _SELFTEST], cwd=ROOT, env=_env(), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "bounds selftest ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.skipif(not BOUNDS_LIB.exists(), reason="libdecxb_bounds.so not built")
def test_random_geometry_parity_tests_stay_inside_their_arrays():
    sel = "random or pitched or pack or batched or fp16 or conv_matches or addend or prepared or fill"
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gpu_parity.py", "-m", "gpu", "-x", "-q", "-k", sel,
                        "-p", "no:cacheprovider"], cwd=ROOT, env=_env(), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-1500:]
    assert " passed" in r.stdout and "failed" not in r.stdout
