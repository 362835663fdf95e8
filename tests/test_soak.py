"""Soak: thousands of collectives through one group without leaks, drift or spurious errors
(a short form of the reference's tests/test_soak.py; set MCCL_SOAK_ITERS to lengthen it)."""
import os

import pytest

from mccl_b200.utils.spawn import run_workers


def _soak_cpu(rank, ws):
    import os, torch, torch.distributed as dist
    iters = int(os.environ.get("MCCL_SOAK_ITERS", "2000"))
    t = torch.zeros(64)
    for i in range(iters):
        t.fill_(float(i % 7))
        dist.all_reduce(t)
        assert t[0].item() == (i % 7) * ws
    big = torch.ones(4 << 20)
    for i in range(10):
        big.fill_(1.0); dist.all_reduce(big)
        assert big[-1].item() == ws
    for i in range(200):   # mixed ops
        if i % 3 == 0:
            dist.broadcast(t, i % ws)
        elif i % 3 == 1:
            outs = [torch.empty(64) for _ in range(ws)]; dist.all_gather(outs, t)
        else:
            dist.barrier()
    m = mccl.get_metrics()
    assert m.total_errors == 0 and m.total_ops >= iters
    pool = mccl.staging_pool_bytes()
    assert pool < (256 << 20), f"staging pool grew to {pool} bytes"


@pytest.mark.slow
def test_soak_cpu_ranks():
    run_workers(_soak_cpu, 3, timeout=300)


def _soak_gpu(rank, ws):
    import os, torch, torch.distributed as dist
    iters = int(os.environ.get("MCCL_SOAK_ITERS", "3000"))
    t = torch.zeros(1024, device=device)
    for i in range(iters):           # epochs wrap through the four data buffers and both lanes many times
        t.fill_(float(i % 5)); dist.all_reduce(t)
    torch.cuda.synchronize()
    assert t[0].item() == ((iters - 1) % 5) * ws
    big = torch.ones(25 << 20, device=device)   # 100 MB: two segments per call
    for i in range(20):
        big.fill_(1.0); dist.all_reduce(big)
    torch.cuda.synchronize()
    assert big[0].item() == ws and big[-1].item() == ws
    assert mccl.get_metrics().total_errors == 0


@pytest.mark.slow
@pytest.mark.gpu(count=2)
def test_soak_gpu_ranks():
    run_workers(_soak_gpu, 2, device="cuda", timeout=300)
