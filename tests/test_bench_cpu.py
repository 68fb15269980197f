"""CPU: the reference arm of bench.py (the oracle's CPU form of the workload,
timed on the host cores) prints one JSON line with the contract's keys."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def test_reference_arm_prints_contract_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "dual_fp8_gemm_tflops" and line["unit"] == "TFLOP/s"
    assert line["higher_is_better"] is True and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["e2e"]["value"] == line["value"]
    assert "workload" in line["config"]
    # whole passes, reported as run: no extrapolation from a slice, no echoed step count
    assert line["steps"] == 1 and line["warmup"] == 0 and "whole pass" in line["cpu_baseline"]["sample"]
    assert line["ms_per_step"] > 0 and abs(line["value"] - 4 * 8192**3 / (line["ms_per_step"] * 1e-3) / 1e12) < 1e-6 * line["value"] + 1e-9
    # both arms describe the workload with the same config keys
    import bench

    assert set(line["config"]) == set(bench._config(1))


def test_roofline_traffic_is_read_from_the_kept_profile():
    import bench

    traffic, src = bench._profiled_traffic()
    assert src == "profiles/dual_gemm_pair_mxf8_8192_bench.md" and 4.48e8 < traffic < 2e9


def test_cpu_list_parsing_for_the_multi_rank_host_binding():
    import bench

    assert bench._parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert bench._parse_cpulist("") == set()
    assert bench._bind_near_gpu(0) is None      # no GPU here: nothing to bind to, no exception
