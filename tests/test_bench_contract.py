"""The benchmark's answers that need no GPU: more than one GPU is refused with one line and exit code 2, and the
reference arm says in one JSON line why it cannot run."""
import json
import subprocess
import sys

from conftest import ROOT


def run_bench(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_in_one_line():
    done = run_bench("--gpus", "2", "--steps", "3", "--warmup", "3")
    assert done.returncode == 2
    lines = [l for l in done.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "--gpus 2" in lines[0] and "one GPU" in lines[0]


def test_the_reference_arm_says_why_it_is_unavailable():
    done = run_bench("--impl", "reference", "--gpus", "1", "--steps", "3", "--warmup", "3")
    assert done.returncode == 0
    lines = [l for l in done.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and "\n" not in rec["unavailable"]
