"""What bench.py answers without a GPU: more than one GPU is refused with one line and exit code 2,
and the reference arm says in one JSON line why it is unavailable (or runs, where the reference
can be imported)."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
  return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                        timeout=300)


def test_more_than_one_gpu_is_refused_in_one_line():
  r = run("--gpus", "2", "--steps", "2", "--warmup", "3")
  assert r.returncode == 2
  lines = [l for l in (r.stdout + r.stderr).splitlines() if l.strip()]
  assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_prints_one_json_line():
  r = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3")
  assert r.returncode == 0
  lines = [l for l in r.stdout.splitlines() if l.strip()]
  assert len(lines) == 1
  line = json.loads(lines[0])
  assert line["impl"] == "reference"
  assert "unavailable" in line or "value" in line


def test_measured_peaks_are_found_flat_or_nested(tmp_path, monkeypatch):
  sys.path.insert(0, ROOT)
  import bench

  assert bench._find_number({"hbm_gbs": 6700.5}, "hbm_gbs") == 6700.5
  assert bench._find_number({"peaks": {"bf16_tflops": {"value": 1600, "clock_mhz": 1900}}}, "bf16_tflops") == 1600.0
  assert bench._find_number({"runs": [{"x": 1}, {"hbm_gbs": 6600}]}, "hbm_gbs") == 6600.0
  assert bench._find_number({"hbm_gbs": "n/a"}, "hbm_gbs") is None
  monkeypatch.setattr(bench, "ROOT", str(tmp_path))
  assert bench.load_peaks() == (bench.FALLBACK_PEAKS, "fallback")
  (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6800, "bf16_tflops": 1500}))
  peaks, where = bench.load_peaks()
  assert where == "measured" and peaks["hbm_gbs"] == 6800.0 and peaks["bf16_tflops_sustained"] == 1500.0
