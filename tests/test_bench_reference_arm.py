"""The benchmark's reference arm (CPU only): one JSON line with the keys the
driver reads, on a batch-1 sample of the conv3 workload."""
import json
import os
import subprocess
import sys

from conftest import ROOT


def test_reference_arm_prints_one_json_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "conv3",
                          "--cpu-sample-batch", "1", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "am_lut_gemm_throughput" and d["unit"] == "GMAC/s"
    assert d["value"] > 0 and d["higher_is_better"] is True and d["gpu_launches"] == 0
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["single_thread_value"] > 0
    assert d["e2e"] == {"value": d["value"], "unit": "GMAC/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
