"""pytest configuration: markers and import path.

``gpu`` marks tests that need a CUDA device (run with ``-m gpu`` on a B200 box);
everything else runs on CPU.  ``multigpu`` tests additionally need >= 2 devices
and skip themselves otherwise.
"""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault("MCCL_LOG_LEVEL", "WARN")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "slow: long-running soak/stress test")
    config.addinivalue_line("markers", "timeout: per-test wall-clock limit (pytest-timeout)")


@pytest.fixture(scope="session")
def native():
    import mccl_b200
    return mccl_b200.require_native()


def _cuda_count():
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


def pytest_collection_modifyitems(config, items):
    n = None
    for item in items:
        need = item.get_closest_marker("gpu")
        if need is None:
            continue
        if n is None:
            n = _cuda_count()
        want = need.kwargs.get("count", 1)
        if n < want:
            item.add_marker(pytest.mark.skip(reason=f"needs {want} CUDA device(s), found {n}"))


def pytest_terminal_summary(terminalreporter, exitstatus, config):
    """With ``MCCL_TEST_SUMMARY=<file>``: per-file pass / fail / skip counts, the GPU count and the
    commit, as JSON (the durable record of a multi-GPU run)."""
    path = os.environ.get("MCCL_TEST_SUMMARY")
    if not path:
        return
    import json
    import subprocess
    per_file = {}
    for outcome in ("passed", "failed", "skipped", "error"):
        for rep in terminalreporter.stats.get(outcome, []):
            nodeid = getattr(rep, "nodeid", "") or ""
            f = nodeid.split("::")[0]
            if not f or (outcome != "skipped" and getattr(rep, "when", "call") != "call" and outcome == "passed"):
                continue
            per_file.setdefault(f, {"passed": 0, "failed": 0, "skipped": 0, "error": 0})[outcome] += 1
    try:
        commit = subprocess.run(["git", "rev-parse", "--short", "HEAD"], capture_output=True, text=True, cwd=str(ROOT)).stdout.strip()
    except Exception:
        commit = ""
    gpus, name = _cuda_count(), ""
    try:
        import torch
        name = torch.cuda.get_device_name(0) if gpus else ""
    except Exception:
        pass
    out = {"gpus": gpus, "gpu_name": name, "commit": commit or os.environ.get("MCCL_COMMIT", ""), "exitstatus": int(exitstatus),
           "per_file": per_file, "totals": {k: sum(v[k] for v in per_file.values()) for k in ("passed", "failed", "skipped", "error")}}
    with open(path, "w") as fh:
        json.dump(out, fh, indent=1, sort_keys=True)
