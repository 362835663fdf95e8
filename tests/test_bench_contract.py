"""The parts of the benchmark driver contract that need no GPU."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_reports_unavailable_and_exits_zero():
    # the reference is a Metal/MPS package that refuses to build on Linux: its arm says so in one JSON line
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                        "--warmup", "1"], capture_output=True, text=True, timeout=300, cwd=str(ROOT))
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_bench_help_lists_the_contract_flags():
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True, text=True, timeout=300,
                       cwd=str(ROOT))
    assert p.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--no-compare", "--optim-in-backward"):
        assert flag in p.stdout, flag
