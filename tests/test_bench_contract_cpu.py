"""The benchmark's reference arm runs without a GPU: its JSON line is checked here for the keys the contract asks for
(the native arm needs a GPU; its line has the same head and is printed by the same code)."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                           "--warmup", "0", "--cpu-seconds", "1"], capture_output=True, text=True, cwd=ROOT, env=env,
                          timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "uvu_conv_fwd_bwd_edges_per_s"
    assert line["unit"] == "edges/s" and line["higher_is_better"] is True and line["value"] > 0
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 0
    assert line["config"]["workload"] == "cfg2" and line["config"]["atoms_per_gpu"] == 50000
    baseline = line["cpu_baseline"]
    assert baseline["kind"] == "port" and baseline["cores"] >= 1 and baseline["value"] == line["value"]
    assert "destination nodes" in baseline["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "edges/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0
    assert "unavailable" in line["reference_gpu"]  # no GPU here
