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
