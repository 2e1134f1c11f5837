"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with a line and exit
code 2, and the reference arm answers with one JSON line: its measurement where a CUDA device and a copy
of the reference are present, else the reason why it cannot run there."""

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


def test_the_reference_arm_names_the_missing_device_on_a_machine_without_one():
    import torch

    if torch.cuda.is_available():
        import pytest

        pytest.skip("with a CUDA device the reference arm measures (minutes): bench.py --impl reference")
    done = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert done.returncode == 0
    record = json.loads(done.stdout.strip().splitlines()[-1])
    assert record["impl"] == "reference"
    assert "CUDA" in record["unavailable"] or "baseline/_ref" in record["unavailable"]


def test_the_command_line_passes_bench_arguments_through():
    done = subprocess.run([sys.executable, "-m", "kernel_rush_kawk_b200.cli", "bench", "--gpus", "3"],
                          capture_output=True, text=True, timeout=120, cwd=str(ROOT))
    assert done.returncode == 2 and "one GPU" in done.stdout
