"""bench.py prints ONE JSON line with the agreed keys: the reference arm on the host cores
(runs anywhere the reference's CPU GEMM was built) and the GPU arm on a B200."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

from oracle import oracle as o

ROOT = Path(__file__).resolve().parent.parent
COMMON = {"metric", "unit", "n_gpus", "steps", "warmup", "higher_is_better", "scaling", "vs_baseline", "dtype", "data",
          "config", "value", "ms_per_step", "cpu_baseline", "e2e", "gpu_launches"}


def run_bench(*args, timeout=600):
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.strip().splitlines() if ln.startswith("{")]
    assert len(lines) == 1, f"expected one JSON line, got {len(lines)}"
    return json.loads(lines[0])


@pytest.mark.skipif(not o.ref_cpu_available(), reason="oracle/_ref/decx_ref_cpu not built (reference tree absent at build time)")
def test_reference_arm_times_the_reference_cpu_gemm():
    j = run_bench("--impl", "reference", "--workload", "cfg1", "--steps", "1", "--warmup", "1")
    assert j["impl"] == "reference"
    if "unavailable" in j:
        pytest.fail("reference arm unavailable here: " + j["unavailable"])
    assert COMMON <= set(j)
    assert j["metric"] == "fp32_gemm_conv_tflops" and j["unit"] == "TFLOP/s" and j["higher_is_better"] is True
    assert j["config"]["workload"] == "cfg1" and j["gpu_launches"] == 0
    assert j["value"] > 0 and j["cpu_baseline"]["kind"] == "reference" and j["cpu_baseline"]["value"] == j["value"]
    assert 1 <= j["cpu_baseline"]["cores"] <= 16
    assert j["e2e"] == {"value": j["value"], "unit": j["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


@pytest.mark.gpu
def test_gpu_arm_prints_the_contract_line():
    j = run_bench("--workload", "cfg1", "--steps", "5", "--warmup", "3", "--no-cpu-baseline")
    assert COMMON | {"roofline", "clocks", "also", "max_norm_err"} <= set(j)
    assert j["max_norm_err"] <= 1e-6
    assert {a["workload"] for a in j["also"]} == {"gemm16k", "cfg2", "cfg3", "cfg4"}
    for a in j["also"]:
        assert "failed" not in a, a
        assert a["value"] > 0 and a["max_norm_err"] <= 1e-6
    assert j["roofline"]["tf32_peak_probe"]["burst_tflops"] > 300 and j["roofline"]["x3_ceiling_probe"]["burst_tflops"] > 100
    assert j["config"] == run_bench("--impl", "reference", "--workload", "cfg1", "--steps", "1", "--warmup", "1")["config"] \
        or not o.ref_cpu_available()
    assert j["n_gpus"] == 1 and j["steps"] == 5 and j["warmup"] == 3 and j["vs_baseline"] is None
    assert j["value"] > 0 and j["gpu_launches"] > 0
    rf = j["roofline"]
    assert {"bound", "achieved", "peak", "unit", "frac", "traffic"} <= set(rf)
    assert rf["bound"] in ("hbm", "tensor") and abs(rf["frac"] - rf["achieved"] / rf["peak"]) < 1e-9
    e = j["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] == 2 * 1024 * 1024 * 4 and e["d2h_bytes_per_step"] == 1024 * 1024 * 4
    assert e["value"] < j["value"], "the host-resident leg includes the PCIe copies"
    assert {"sm_mhz", "sm_max_mhz", "reasons"} <= set(j["clocks"])
