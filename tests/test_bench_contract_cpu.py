"""The edges of bench.py's contract that need no GPU: more than one GPU is refused with one line
and exit code 2; the reference arm prints its one JSON line and exits 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=300, cwd=ROOT)


def test_more_than_one_gpu_is_refused_with_one_line():
    r = run("--gpus", "2", "--steps", "1", "--warmup", "1")
    assert r.returncode == 2
    assert len([l for l in r.stdout.splitlines() if l.strip()]) == 1 and "single-GPU" in r.stdout


def test_reference_arm_says_why_it_is_unavailable():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "1", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]
