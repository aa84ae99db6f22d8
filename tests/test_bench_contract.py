"""bench.py without a GPU: the reference arm (the CPU restatement of the reference's GEMM, kind
"port") prints one JSON line with the keys the benchmark contract names, its `config` is the one
the GPU arm reports, the other ranks of a multi-rank launch stay silent, and the table of ncu
captures answers only for the exact kernel configuration and problem."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _run(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, env=e, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    return r.stdout


def test_reference_arm_line():
    import bench
    out = _run("--impl", "reference", "--steps", "1", "--warmup", "0").strip().splitlines()
    assert len(out) == 1
    line = json.loads(out[0])
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC and line["unit"] == "TFLOP/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["config"] == bench.config_dict(1)  # the same workload description as the GPU arm's
    assert line["value"] > 0 and line["ms_per_step"] > 0
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and "rows" in cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0


def test_reference_arm_other_ranks_are_silent():
    out = _run("--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0",
               env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert out.strip() == ""


def test_traffic_table_answers_only_for_the_captured_kernel():
    import bench
    t = bench.committed_traffic(10, 8192, 8192, 8192, "bf16", "bf16")
    assert t is not None and 4.0e8 < t < 3.0e9  # above the algorithmic 402.7 MB, the same order of magnitude
    assert bench.committed_traffic(4, 8192, 8192, 8192, "bf16", "bf16") is None   # another tile shape
    assert bench.committed_traffic(10, 4096, 4096, 4096, "bf16", "bf16") is None  # another problem
    assert bench.committed_traffic(10, 8192, 8192, 8192, "f16", "f16") is None    # another element type
