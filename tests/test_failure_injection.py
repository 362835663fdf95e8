"""Failure detection without touching a GPU: faults are injected on the host among CPU ranks.

A rank that exits, a watchdog limit, and back-pressure without spurious aborts
(reference tests/test_failure_injection.py:17-74).  Survivors must get a Python exception,
never a hang and never std::terminate.
"""
import pytest

from mccl_b200.utils.spawn import run_workers


def _peer_exits(rank, ws):
    import os, time, torch, torch.distributed as dist
    t = torch.ones(1000); dist.all_reduce(t); assert t[0].item() == ws
    if rank == ws - 1:
        os._exit(0)  # leaves between steps, nothing in flight
    time.sleep(0.5)
    try:
        for _ in range(3):
            t = torch.ones(100000); dist.all_reduce(t)
        print("NO_EXCEPTION")
        os._exit(3)
    except RuntimeError as e:
        print("GOT_EXCEPTION", str(e)[:120])
    try:
        dist.barrier()
        os._exit(4)
    except RuntimeError:
        pass  # a failed group fails fast afterwards
    os._exit(0)


@pytest.mark.parametrize("ws", [2, 3])
def test_survivors_raise_when_a_peer_exits(ws):
    res = run_workers(_peer_exits, ws, timeout=90, expect_failure=True,
                      env={"MCCL_HEARTBEAT_INTERVAL_MS": "200", "MCCL_RECV_TIMEOUT_MS": "5000"})
    for r in range(ws - 1):
        assert res[r].returncode == 0, (r, res[r].stdout, res[r].stderr[-800:])
        assert "GOT_EXCEPTION" in res[r].stdout


def _rank_never_joins(rank, ws):
    import os, time, torch, torch.distributed as dist
    if rank == 1:
        time.sleep(4)  # skips the collective while the others wait, then leaves
        os._exit(0)
    try:
        t = torch.ones(10); dist.all_reduce(t)
        os._exit(3)
    except RuntimeError as e:
        print("TIMEOUT_OK", str(e)[:100])
        os._exit(0)


def test_watchdog_turns_a_missing_rank_into_an_exception():
    res = run_workers(_rank_never_joins, 2, timeout=60, expect_failure=True,
                      env={"MCCL_WATCHDOG_TIMEOUT_MS": "1500", "MCCL_RECV_TIMEOUT_MS": "1500"})
    assert res[0].returncode == 0 and "TIMEOUT_OK" in res[0].stdout, res[0].stderr[-800:]


def _backpressure(rank, ws):
    import torch, torch.distributed as dist
    works, ts = [], []
    for i in range(200):
        t = torch.full((1 << 20,), float(i))  # 4 MB each, queued behind each other
        ts.append(t); works.append(dist.all_reduce(t, async_op=True))
    for w in works:
        w.wait()
    assert all(ts[i][0].item() == i * ws for i in range(200))
    assert mccl.get_metrics().total_errors == 0


def test_queued_operations_do_not_trip_the_watchdog():
    # queue time is far above the 3 s limit in aggregate; deadlines arm only when an op starts executing
    run_workers(_backpressure, 2, timeout=180, env={"MCCL_WATCHDOG_TIMEOUT_MS": "3000"})


def _abort_propagates(rank, ws):
    import os, time, torch, torch.distributed as dist
    be = mccl.get_backend(device="cpu")
    dist.barrier()
    if rank == 0:
        be.abort()
    else:
        time.sleep(1.0)
    try:
        dist.all_reduce(torch.ones(4))
        os._exit(3)
    except RuntimeError:
        assert be.poisoned
    os._exit(0)


def test_abort_reaches_every_rank():
    res = run_workers(_abort_propagates, 3, timeout=60, expect_failure=True)
    assert [r.returncode for r in res] == [0, 0, 0], [r.stderr[-300:] for r in res]
