"""Drives the C++ test program of the de:: layer (tests/cpp/test_decx_api.cpp)."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
EXE = ROOT / "tests" / "cpp" / "test_decx_api"


def _build():
    subprocess.run(["make", "-s", "-C", str(ROOT / "backup_1_b200" / "csrc")], check=True)
    subprocess.run(["make", "-s", "-C", str(ROOT / "backup_1_b200" / "host")], check=True)


def _run(mode):
    _build()
    r = subprocess.run([str(EXE), mode], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all checks passed" in r.stdout


def test_containers_layout_and_not_init_handles():
    _run("layout")


@pytest.mark.gpu
def test_gemm_and_conv_through_the_cpp_api():
    _run("gpu")
