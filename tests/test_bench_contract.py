"""The benchmark's CPU arm runs without a GPU and prints one JSON line with the agreed keys."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run(
        [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "c1", "--steps", "1",
         "--warmup", "1"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in line, key
    assert line["impl"] == "reference" and line["value"] > 0 and line["gpu_launches"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert line["config"]["workload"].startswith("c1")


def test_other_ranks_of_the_reference_arm_do_nothing():
    out = subprocess.run(
        [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "c1", "--gpus", "2"],
        capture_output=True, text=True, timeout=120, cwd=ROOT,
        env={**__import__("os").environ, "RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_reference_arm_covers_the_prefill_workload_with_the_same_config_echo():
    """`--impl reference --workload c4` runs (a bounded sample of the oracle's prefill) and echoes
    the same `config`, `steps` and `warmup` the GPU arm prints for that workload."""
    out = subprocess.run(
        [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "c4", "--steps", "1",
         "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([ln for ln in out.stdout.splitlines() if ln.startswith("{")][0])
    assert line["impl"] == "reference" and line["metric"] == "paged_prefill_tensor_throughput"
    assert line["unit"] == "TFLOP/s" and line["value"] > 0 and (line["steps"], line["warmup"]) == (1, 0)
    sys.path.insert(0, str(ROOT))
    import bench
    from llama_lite_npu_b200 import workloads as W

    assert line["config"] == bench.workload_config(W.C4)
    assert "requests" in line["cpu_baseline"]["sample"]
