"""What ``bench.py`` promises without a GPU: one line and exit code 2 for more than one GPU,
and the reference arm's ``unavailable`` line."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT,
                          stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_in_one_line():
    p = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    lines = [l for l in (p.stdout + p.stderr).splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]
