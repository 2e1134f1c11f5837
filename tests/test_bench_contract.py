"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with a line and exit
code 2, and the reference arm answers with one JSON line that says why it is unavailable."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_with_a_line():
    done = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert done.returncode == 2
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_the_reference_arm_says_why_it_is_unavailable():
    done = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert done.returncode == 0
    record = json.loads(done.stdout.strip().splitlines()[-1])
    assert record["impl"] == "reference" and isinstance(record["unavailable"], str) and record["unavailable"]


def test_the_command_line_passes_bench_arguments_through():
    done = subprocess.run([sys.executable, "-m", "kernel_rush_kawk_b200.cli", "bench", "--impl", "reference"],
                          capture_output=True, text=True, timeout=120, cwd=str(ROOT))
    assert done.returncode == 0 and json.loads(done.stdout.strip().splitlines()[-1])["impl"] == "reference"
