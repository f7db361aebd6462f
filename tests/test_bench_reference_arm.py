"""The reference arm of `bench.py` (`--impl reference`): it runs on the host cores alone, prints exactly one JSON line on
stdout and carries the keys the benchmark contract names. Runs without a GPU (a bounded sample, a few seconds)."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _run(*extra):
    env = dict(os.environ, OMP_NUM_THREADS=os.environ.get("OMP_NUM_THREADS", "4"))
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1", *extra],
                         cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, lines   # stdout carries the JSON line and nothing else
    return json.loads(lines[0])


def test_reference_arm_line_for_the_projection_microbench():
    d = _run("--tokens", "2048", "--cpu-sample-tokens", "256")
    assert d["impl"] == "reference" and d["metric"] == "projection GEMM TFLOP/s" and d["unit"] == "TFLOP/s"
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["higher_is_better"] is True and d["vs_baseline"] is None
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "256 of the 2048" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["config"]["workload"].startswith("ModernBERT-base projection microbench")


def test_reference_arm_honours_the_workload():
    d = _run("--workload", "base")
    assert d["impl"] == "reference" and d["metric"] == "encoder tokens/s" and d["unit"] == "tokens/s"
    assert d["value"] > 0 and d["ms_per_step"] > 0
    assert "22 layers" in d["cpu_baseline"]["sample"] and d["cpu_baseline"]["kind"] == "port"
