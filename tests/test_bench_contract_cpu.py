"""The parts of the bench contract that need no GPU: the reference arm's line and the published numbers."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_and_exits_zero():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 0
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]


def test_published_numbers_match_the_baseline_record():
    sys.path.insert(0, ROOT)
    import importlib
    bench = importlib.import_module("bench")
    with open(os.path.join(ROOT, "BASELINE.md")) as f:
        text = f.read()
    assert bench.BASELINE_TOK_S[1] == 27.9 and "27.9" in text
    assert bench.BASELINE_TTFT_S[1] == 3.773 and "3.773" in text
