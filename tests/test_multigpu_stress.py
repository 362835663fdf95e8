"""Race / stress runs on real GPUs: compute interleaved with collectives without host syncs,
mixed operation streams, skewed ranks, many outstanding works (reference
tests/test_race_stress.py and tests/test_ddp_consumer_release.py)."""
import pytest
import torch

from mccl_b200.utils.spawn import run_workers

pytestmark = [pytest.mark.gpu(count=2)]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _stress(rank, ws):
    import time
    import torch, torch.distributed as dist
    # 1. producer fence + consumer release with no host synchronisation anywhere
    n = 1 << 20
    acc = torch.zeros(n, device=device)
    a = torch.randn(2048, 2048, device=device)
    for i in range(40):
        b = a @ a.t()                       # keeps the SMs busy around the collective
        t = torch.full((n,), float(i + rank), device=device) + b[0, 0] * 0
        dist.all_reduce(t)                  # sync op: the current stream waits on-device only
        acc += t                            # consumer kernel right behind it
    torch.cuda.synchronize()
    want = sum(i * ws + sum(range(ws)) for i in range(40))
    assert acc[0].item() == want and acc[-1].item() == want, (acc[0].item(), want)
    # 2. mixed operation stream, several dtypes and sizes, async handles kept alive
    works, checks = [], []
    for it in range(30):
        sz = [17, 4099, 300001, 1 << 21][it % 4]
        kind = it % 5
        if kind == 0:
            t = torch.full((sz,), 1.0, device=device, dtype=[torch.float32, torch.bfloat16, torch.float16][it % 3])
            works.append(dist.all_reduce(t, async_op=True)); checks.append((t, float(ws)))
        elif kind == 1:
            t = torch.full((sz,), float(it), device=device) if rank == it % ws else torch.zeros(sz, device=device)
            works.append(dist.broadcast(t, it % ws, async_op=True)); checks.append((t, float(it)))
        elif kind == 2:
            o = torch.empty(sz * ws, device=device); i_ = torch.full((sz,), float(rank), device=device)
            works.append(dist.all_gather_into_tensor(o, i_, async_op=True)); checks.append((o[-sz:], float(ws - 1)))
        elif kind == 3:
            i_ = torch.ones(sz * ws, device=device); o = torch.empty(sz, device=device)
            works.append(dist.reduce_scatter_tensor(o, i_, async_op=True)); checks.append((o, float(ws)))
        else:
            dist.barrier()
    for w in works:
        w.wait()
    torch.cuda.synchronize()
    for t, v in checks:
        assert t.float()[0].item() == v and t.float()[-1].item() == v
    # 3. skewed ranks: a late rank must be waited for, not timed out on
    for i in range(4):
        if rank == i % ws:
            time.sleep(0.3)
        t = torch.ones(100000, device=device); dist.all_reduce(t)
        assert t[0].item() == ws
    m = mccl.get_metrics()
    assert m.total_errors == 0


@pytest.mark.parametrize("ws", [2, 4, 8])
def test_stress_mixed_streams(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    run_workers(_stress, ws, device="cuda", timeout=300)


def _skip_launch(rank, ws):
    import os, torch, torch.distributed as dist
    t = torch.ones(1000, device=device); dist.all_reduce(t); torch.cuda.synchronize()
    be = mccl.get_backend(device=device)
    if rank == 1:
        be._test_skip_next_launch()   # host-injected fault: this rank never launches the next collective
    t = torch.ones(1000, device=device)
    try:
        dist.all_reduce(t)
        dist.barrier()                 # blocking: surfaces the device-side timeout on the other ranks
        torch.cuda.synchronize()
        if rank != 1:
            os._exit(3)
    except RuntimeError as e:
        print("DEVICE_TIMEOUT_REPORTED", str(e)[:100])
    y = torch.ones(8, device=device).sum().item()   # context is still usable
    assert y == 8.0
    os._exit(0)


def test_bounded_device_wait_is_reported_across_gpus():
    # NVLS is not used by these kernels (plain peer loads/stores); every wait gives up after 1 s
    res = run_workers(_skip_launch, 2, device="cuda", timeout=120, expect_failure=True,
                      env={"MCCL_DEVICE_WAIT_US": "1000000", "NCCL_NVLS_ENABLE": "0"})
    assert res[0].returncode == 0, res[0].stderr[-1500:]
    assert "DEVICE_TIMEOUT_REPORTED" in res[0].stdout
