"""What ``bench.py`` promises without a GPU: more than one GPU is refused with one line and
exit code 2, and the reference arm answers with its ``unavailable`` line and exit code 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          cwd=ROOT, timeout=900)      # a cold machine pages the libraries in first


def test_more_than_one_gpu_is_refused_with_one_line():
    r = _run("--gpus", "2", "--steps", "1", "--warmup", "1")
    assert r.returncode == 2
    lines = [ln for ln in (r.stdout + r.stderr).splitlines() if ln.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "1", "--warmup", "1")
    assert r.returncode == 0
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and rec["unavailable"]
    assert "\n" not in rec["unavailable"]
