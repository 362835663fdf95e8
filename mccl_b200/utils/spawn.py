"""Multi-process test harness: run ``fn(rank, world_size)`` in N local worker processes.

The worker function's *source* is serialised into a ``python -c`` script (so it
needs no importable module and can be defined inside a test), every worker
joins a ``mccl`` process group over 127.0.0.1, and a hard wall-clock timeout
kills the whole group and fails the test -- a hung collective can never hang
the test session.  ``device="cpu"`` runs CPU-tensor ranks (no GPU needed);
``device="cuda"`` binds rank r to ``cuda:r``.

Modelled on the strategy of the reference's ``tests/mccl_test_utils.py:47-126``.
"""
from __future__ import annotations

import inspect
import os
import random
import signal
import subprocess
import sys
import textwrap
import time
from pathlib import Path
from typing import Callable, Dict, List, Optional

_REPO_ROOT = str(Path(__file__).resolve().parents[2])
_port_counter = 0


def next_port() -> int:
    """A rendezvous port unlikely to collide across concurrently running tests."""
    global _port_counter
    _port_counter += 1
    base = 20000 + (os.getpid() * 13) % 20000
    return base + (_port_counter * 7 + random.randint(0, 5)) % 9000


_WORKER_TEMPLATE = """
import os, sys, traceback
sys.path.insert(0, {repo_root!r})
rank = int(sys.argv[1]); world_size = int(sys.argv[2])
os.environ['RANK'] = str(rank); os.environ['WORLD_SIZE'] = str(world_size)
os.environ['LOCAL_RANK'] = str(rank)
os.environ['MASTER_ADDR'] = '127.0.0.1'; os.environ['MASTER_PORT'] = {port!r}
os.environ.setdefault('MCCL_LISTEN_ADDR', '127.0.0.1')
import datetime
import torch
import torch.distributed as dist
import mccl_b200 as mccl
DEVICE = {device!r}
if DEVICE == 'cuda':
    torch.cuda.set_device(rank % torch.cuda.device_count())
    device = torch.device('cuda', rank % torch.cuda.device_count())
else:
    device = torch.device('cpu')

{fn_source}

code = 0
try:
    if {init_pg!r}:
        kw = dict(backend={backend!r}, rank=rank, world_size=world_size,
                  timeout=datetime.timedelta(seconds={pg_timeout}))
        if DEVICE == 'cuda' and {bind_device!r}:
            kw['device_id'] = device
        dist.init_process_group(**kw)
    {fn_name}(rank, world_size)
    if {init_pg!r} and dist.is_initialized():
        dist.destroy_process_group()
except BaseException:
    traceback.print_exc()
    code = 1
    # leave in order even after a failure: the group's shutdown drains the streams and releases
    # device memory that peers can reach (all its waits are bounded)
    try:
        if {init_pg!r} and dist.is_initialized():
            dist.destroy_process_group()
    except BaseException:
        pass
sys.stdout.flush(); sys.stderr.flush()
os._exit(code)
"""


class WorkerFailure(AssertionError):
    pass


def run_workers(
    fn: Callable[[int, int], None],
    world_size: int,
    *,
    env: Optional[Dict[str, str]] = None,
    timeout: float = 120.0,
    device: str = "cpu",
    backend: str = "mccl",
    expect_failure: bool = False,
    init_pg: bool = True,
    pg_timeout: int = 60,
    bind_device: bool = False,
) -> List[subprocess.CompletedProcess]:
    """Runs ``fn`` on ``world_size`` local ranks; raises ``WorkerFailure`` on error/timeout.

    With ``expect_failure`` the call returns the per-rank results instead of
    raising when some rank exits non-zero (a timeout still raises: "fails
    cleanly" never means "hangs").
    """
    src = textwrap.dedent(inspect.getsource(fn))
    script = _WORKER_TEMPLATE.format(
        repo_root=_REPO_ROOT, port=str(next_port()), device=device, fn_source=src, fn_name=fn.__name__,
        backend=backend, init_pg=init_pg, pg_timeout=pg_timeout, bind_device=bind_device)
    child_env = dict(os.environ)
    child_env.setdefault("MCCL_LOG_LEVEL", "WARN")
    child_env.setdefault("MCCL_DEVICE_WAIT_US", "5000000")
    child_env.setdefault("OMP_NUM_THREADS", "1")
    # NVLS (NVLink multicast) stays off in test workers unless a test asks for it: a rank that
    # leaves abnormally while its memory is bound to a multicast object can fault its peers' GPUs.
    child_env.setdefault("MCCL_NVLS", "0")
    if env:
        child_env.update({k: str(v) for k, v in env.items()})
    procs = []
    for r in range(world_size):
        procs.append(subprocess.Popen(
            [sys.executable, "-c", script, str(r), str(world_size)],
            env=child_env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
            start_new_session=True))
    deadline = time.time() + timeout
    results: List[Optional[subprocess.CompletedProcess]] = [None] * world_size
    timed_out = False
    for r, p in enumerate(procs):
        left = deadline - time.time()
        try:
            out, err = p.communicate(timeout=max(left, 0.1))
            results[r] = subprocess.CompletedProcess(p.args, p.returncode, out, err)
        except subprocess.TimeoutExpired:
            timed_out = True
            break
    if timed_out:
        for p in procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGKILL)  # exactly the group this harness started
                except ProcessLookupError:
                    pass
        tails = []
        for r, p in enumerate(procs):
            try:
                out, err = p.communicate(timeout=5)
            except Exception:
                out, err = "", ""
            tails.append(f"--- rank {r} (rc={p.returncode}) ---\n{(err or '')[-1500:]}")
        raise WorkerFailure(f"workers exceeded the {timeout}s wall-clock limit and were killed\n" + "\n".join(tails))
    bad = [r for r, res in enumerate(results) if res is not None and res.returncode != 0]
    if bad and not expect_failure:
        msg = "\n".join(
            f"--- rank {r} (rc={results[r].returncode}) ---\n{results[r].stdout[-1500:]}\n{results[r].stderr[-3000:]}"
            for r in bad)
        raise WorkerFailure(f"ranks {bad} failed\n{msg}")
    return results  # type: ignore[return-value]
