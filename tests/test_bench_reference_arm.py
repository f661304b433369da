"""CPU: `bench.py --impl reference` — the reference's own x86 path timed on the host cores — prints the one JSON line
of the bench contract, with no GPU and no CUDA library involved."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1"],
                         cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    line = json.loads(run.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    if "unavailable" in line:  # no reference build and no port on this machine: the contract's one-line answer
        assert isinstance(line["unavailable"], str) and line["unavailable"]
        return
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["unit"] == "GB/s" and line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 2
    assert line["vs_baseline"] is None and line["data"] == "synthetic"
    assert line["config"]["workload"].startswith("C5 FP8-E4M3 Linear M=1 K=8192 N=28672")
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] and line["value"] > 0
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # the metric is bytes of the whole weight per step over the step time
    assert abs(line["value"] - line["config"]["algorithmic_bytes_per_step"] / (line["ms_per_step"] * 1e-3) / 1e9) < 0.02 * line["value"]
