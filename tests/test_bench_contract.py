"""What bench.py promises on a machine without a GPU: more than one GPU is refused with one line
and exit code 2, and the reference arm always ends with one JSON line and exit code 0."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_in_one_line():
    p = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert p.returncode == 2
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    assert json.loads(lines[0])["n_gpus"] == 2


def test_the_reference_arm_prints_one_json_line():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert p.returncode == 0
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert "unavailable" in line or "value" in line


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    """The roofline's denominators: a measured file beside bench.py wins, anything unreadable in it
    falls back to the stated figures."""
    sys.path.insert(0, str(ROOT))
    try:
        import bench
    finally:
        sys.path.pop(0)
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    assert bench.load_peaks()["source"] == "fallback"
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6560.0, "bf16_tflops": 1620.0, "bf16_tflops_sustained": 1480.0}))
    got = bench.load_peaks()
    assert got["source"] == "measured" and got["hbm_gbs"] == 6560.0 and got["bf16_tflops"] == 1620.0
    for broken in ('{"hbm_gbs": {"value": 1}}', '{"hbm_gbs": 1.0}', "not json"):
        (tmp_path / "MEASURED_PEAKS.json").write_text(broken)
        assert bench.load_peaks() == bench.FALLBACK_PEAKS
