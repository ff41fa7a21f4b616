"""What bench.py promises: more than one GPU is refused with one line and exit code 2; the
reference arm always ends with one JSON line and exit code 0, which says why it could not run on
a machine without a GPU and carries a measured value on one with a GPU and the installed
reference."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REF_INSTALLED = (ROOT / "baseline" / "_ref" / "torchllms" / "messages" / "configs").is_dir()


def run(*args, timeout=300):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=timeout)


def test_more_than_one_gpu_is_refused_in_one_line():
    p = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert p.returncode == 2
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    assert json.loads(lines[0])["n_gpus"] == 2


def test_the_reference_arm_says_why_it_cannot_run_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("this machine has a GPU: the arm runs (see the test below)")
    p = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3", "--layers", "1")
    assert p.returncode == 0
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and "value" not in line
    why = line["unavailable"]
    assert ("not installed" in why or "lacks" in why) if not REF_INSTALLED else "exited" in why


@pytest.mark.gpu
def test_the_reference_arm_measures_the_installed_reference():
    """Two layers of the shape and a few dozen steps (fewer are lost in the spread of the prefill's time,
    which both sides of the difference contain): enough to see that the reference's own ``LLM`` ran its
    stock path and that the line carries what the full run's line carries."""
    if not REF_INSTALLED:
        pytest.skip("the reference is not installed under baseline/_ref")
    p = run("--impl", "reference", "--gpus", "1", "--steps", "48", "--warmup", "3", "--layers", "2", timeout=1500)
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" not in line, line
    assert line["value"] > 0 and line["e2e"]["value"] > 0 and line["ms_per_step"] > 0 and line["prefill"]["ms"] > 0
    assert all(way["ms_per_step"] > 0 for way in line["decode_ways"].values())
    assert line["config"]["n_layers"] == 2 and line["config"]["n_layers_full"] == 32 and "LLM.generate" in line["config"]["level"]
    assert line["steps"] == 48 and line["dtype"] == "bf16" and line["gpu_launches"] == 0


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
