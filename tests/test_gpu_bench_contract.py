"""The benchmark's own arm on the smallest configuration: one JSON line with the keys the contract asks for."""

import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_native_arm_line_on_the_smallest_configuration():
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--workload", "cfg1", "--steps", "3",
                           "--warmup", "3", "--skip-others", "--cpu-seconds", "1", "--e2e-steps", "1",
                           "--e2e-chunks", "4"], capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "roofline", "cpu_baseline", "e2e", "clocks", "gpu_launches"):
        assert key in line, key
    assert line["value"] > 0 and line["n_gpus"] == 1 and line["steps"] == 3 and line["dtype"] == "f64"
    assert line["config"]["workload"] == "cfg1" and "model" not in line["config"]
    roofline = line["roofline"]
    assert roofline["bound"] == "hbm" and roofline["unit"] == "GB/s" and roofline["peak"] > 0
    assert abs(roofline["frac"] - roofline["achieved"] / roofline["peak"]) < 1e-9
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    e2e = line["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] > 0
    assert e2e["api"] == "HostStreamedConv.step"
    assert line["gpu_launches"] >= 2 * line["steps"] and line["device_status"] is None
