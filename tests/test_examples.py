"""The example driver runs end to end on CPU ranks (gloo-free: backend mccl, host transport)."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _run(args, env=None, timeout=240):
    e = dict(os.environ); e.update(env or {})
    return subprocess.run([sys.executable] + args, cwd=ROOT, env=e, capture_output=True, text=True, timeout=timeout)


def test_ddp_dummy_train_two_cpu_ranks(tmp_path):
    stats = tmp_path / "ddp.json"
    r = _run(["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
              "--master-port", "29871", "examples/ddp_dummy_train.py", "--cpu", "--model", "gpt2-tiny", "--steps", "6",
              "--warmup", "1", "--batch-size", "2", "--save-stats", str(stats)])
    assert r.returncode == 0, r.stderr[-2000:]
    s = json.loads(stats.read_text())
    assert s["world_size"] == 2 and len(s["step_times"]) == 6 and s["mode"] == "ddp-mccl"
    base = tmp_path / "base.json"
    r = _run(["examples/ddp_dummy_train.py", "--cpu", "--baseline", "--model", "gpt2-tiny", "--steps", "4", "--warmup", "1",
              "--batch-size", "2", "--save-stats", str(base)])
    assert r.returncode == 0, r.stderr[-2000:]
    r = _run(["examples/benchmark_throughput.py", str(base), str(stats), "--out", str(tmp_path / "bench")])
    assert r.returncode == 0 and "throughput ratio" in r.stdout, r.stderr[-1000:]
    assert (tmp_path / "bench.npz").exists()


def test_shell_scripts_parse():
    import glob, os, subprocess
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
    scripts = sorted(glob.glob(os.path.join(root, "*.sh")))
    assert len(scripts) >= 4
    for s in scripts:
        subprocess.run(["bash", "-n", s], check=True)
