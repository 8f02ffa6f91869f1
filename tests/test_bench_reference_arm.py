"""The reference arm of the benchmark runs without a GPU (the reference bench's f32 loop on the host cores): one short
run must print exactly one JSON line with the contract's keys, the same metric, unit and workload name as the native arm
declares, and a cpu_baseline that describes this very run."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 1 and d["steps"] == 1 and d["warmup"] == 1
    assert d["unit"] == "GB/s" and d["higher_is_better"] is True and d["value"] > 0
    sys.path.insert(0, ROOT)
    import bench

    assert d["metric"] == bench.METRIC and d["config"] == {"workload": bench.workload_name(1)}
    cpu = d["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] >= 1 and cpu["value"] == d["value"] and "sample" in cpu
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
