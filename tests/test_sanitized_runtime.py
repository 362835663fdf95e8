"""CPU-rank workloads under the sanitizer-instrumented build of the native layer.

``MCCL_SANITIZE=address python -m mccl_b200._build`` produces ``mccl_b200/_C_asan.so`` (host code
compiled with ``-fsanitize=address``); ``thread`` produces ``_C_tsan.so``.  Each test here starts
child processes that preload the sanitizer runtime, load that library through ``MCCL_NATIVE_LIB``
and run real traffic over the host transport: collectives on CPU tensors at 2 and 3 ranks, the
framed-TCP path with CRC and tiny chunks, the engine / watchdog / memory-pool unit hooks, and a
rank that leaves early (the failure path frees in-flight receives).  A sanitizer report in any
rank's stderr fails the test.  The tests skip when the instrumented library has not been built
(it takes a few minutes), so the regular CPU tier stays fast; CI builds it explicitly.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

from mccl_b200 import _build
from mccl_b200.utils.spawn import run_workers

ROOT = Path(__file__).resolve().parents[1]


def _env(kind):
    lib = _build.sanitized_target(kind)
    if not lib.exists():
        pytest.skip(f"{lib.name} not built (MCCL_SANITIZE={kind} python -m mccl_b200._build)")
    rt = _build.sanitizer_runtime(kind)
    if not rt:
        pytest.skip("sanitizer runtime library not found next to the compiler")
    env = {"MCCL_NATIVE_LIB": str(lib), "LD_PRELOAD": rt, "MCCL_NO_AUTOBUILD": "1"}
    if kind == "address":
        # python and torch are not instrumented: their leaks are not ours to report, and the CUDA
        # runtime needs the shadow gap unprotected even when no GPU is touched
        env["ASAN_OPTIONS"] = "detect_leaks=0:protect_shadow_gap=0:abort_on_error=0:halt_on_error=1:exitcode=66"
    else:
        env["TSAN_OPTIONS"] = "report_signal_unsafe=0:exitcode=66:halt_on_error=0"
    return env


def _no_reports(results, marker):
    for r, res in enumerate(results):
        assert marker not in (res.stderr or ""), f"rank {r}:\n{res.stderr[-4000:]}"
        assert res.returncode == 0, f"rank {r} rc={res.returncode}\n{res.stderr[-2000:]}"


def _traffic(rank, ws):
    import torch, torch.distributed as dist
    for dtype in (torch.float32, torch.bfloat16, torch.int64):
        for n in (1, 33, 4097, 300_001):
            t = (torch.arange(n) % 13).to(dtype) * (rank + 1)
            dist.all_reduce(t)
            assert t[n - 1].item() == ((n - 1) % 13) * sum(range(1, ws + 1))
    big = torch.ones(3_000_000) * (rank + 1)      # two-shot / segmented pair path
    dist.all_reduce(big, op=dist.ReduceOp.AVG)
    assert abs(big[0].item() - (ws + 1) / 2) < 1e-6
    b = torch.arange(70_001, dtype=torch.float32) if rank == 0 else torch.zeros(70_001)
    dist.broadcast(b, 0)
    outs = [torch.empty(257) for _ in range(ws)]
    dist.all_gather(outs, torch.full((257,), float(rank)))
    assert [o[0].item() for o in outs] == [float(r) for r in range(ws)]
    o = torch.empty(100)
    dist.reduce_scatter(o, [torch.full((100,), float(rank + i)) for i in range(ws)])
    works = [dist.all_reduce(torch.ones(10_000), async_op=True) for _ in range(16)]
    for w in works:
        w.wait()
    if ws >= 2:
        if rank == 0:
            dist.send(torch.arange(1000.), 1, tag=3)
        elif rank == 1:
            got = torch.empty(1000)
            dist.recv(got, 0, tag=3)
            assert got[999].item() == 999
    dist.barrier()
    m = mccl.get_metrics()
    assert m.total_ops > 0 and m.total_errors == 0


@pytest.mark.parametrize("ws", [2, 3])
def test_cpu_collectives_under_asan(ws):
    res = run_workers(_traffic, ws, timeout=300, env=_env("address"), expect_failure=True)
    _no_reports(res, "ERROR: AddressSanitizer")


def test_crc_and_tiny_frames_under_asan():
    env = dict(_env("address"), MCCL_TRANSPORT_CRC="1", MCCL_CHUNK_BYTES="4096")
    res = run_workers(_traffic, 2, timeout=300, env=env, expect_failure=True)
    _no_reports(res, "ERROR: AddressSanitizer")


def _leaver(rank, ws):
    import os, time, torch, torch.distributed as dist
    t = torch.ones(1000)
    dist.all_reduce(t)
    if rank == 1:
        sys.stdout.flush()
        os._exit(0)          # leaves between collectives, without a goodbye
    time.sleep(0.5)
    try:
        for _ in range(50):
            dist.all_reduce(torch.ones(100_000))
            time.sleep(0.05)
        raise SystemExit("the survivor never noticed that its peer left")
    except RuntimeError:
        pass                 # poisoned group: the expected outcome


def test_peer_exit_path_under_asan():
    res = run_workers(_leaver, 2, timeout=300, env=dict(_env("address"), MCCL_HEARTBEAT_INTERVAL_MS="200"),
                      expect_failure=True)
    for r, out in enumerate(res):
        assert "ERROR: AddressSanitizer" not in (out.stderr or ""), f"rank {r}:\n{out.stderr[-4000:]}"
    assert res[0].returncode == 0, res[0].stderr[-2000:]


def test_runtime_unit_hooks_under_asan():
    env = dict(os.environ, **_env("address"))
    code = (
        "import mccl_b200 as m; n = m.require_native();"
        "assert n._test_watchdog(50, True, 300) == 1;"
        "o, d, e = n._test_engine(3, 2, 40, 0); assert d == 40 and e == 0;"
        "n._test_mempool(); print('ok')"
    )
    p = subprocess.run([sys.executable, "-c", code], env=env, cwd=str(ROOT), capture_output=True, text=True, timeout=300)
    assert "ERROR: AddressSanitizer" not in p.stderr, p.stderr[-4000:]
    assert p.returncode == 0 and "ok" in p.stdout, p.stderr[-2000:]


@pytest.mark.slow
@pytest.mark.parametrize("ws", [2])
def test_cpu_collectives_under_tsan(ws):
    # Opt-in (MCCL_RUN_TSAN=1): several minutes under ThreadSanitizer.  Python and torch are not
    # instrumented, so happens-before edges that run through them are invisible to the tool: reports
    # about objects whose lifetime is managed by torch's intrusive_ptr reference counts (released in
    # libtorch_python) are of that kind and are not counted.
    if os.environ.get("MCCL_RUN_TSAN") != "1":
        pytest.skip("set MCCL_RUN_TSAN=1 to run the ThreadSanitizer pass")
    res = run_workers(_traffic, ws, timeout=900, env=dict(_env("thread"), MCCL_WATCHDOG_TIMEOUT_MS="600000"), expect_failure=True)
    for r, out in enumerate(res):
        rep = out.stderr or ""
        blocks = [blk for blk in rep.split("==================") if "WARNING: ThreadSanitizer" in blk and "mccl::" in blk]
        ours = [blk for blk in blocks if "intrusive_ptr" not in blk]
        assert not ours, f"rank {r}:\n{ours[0][-4000:]}"
