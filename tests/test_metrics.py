"""Metrics are populated by real traffic on every rank and cleared by reset (reference tests/test_metrics.py:23-91)."""
from mccl_b200.utils.spawn import run_workers


def _metrics(rank, ws):
    import torch, torch.distributed as dist
    for n in (10, 100000, 1000000):
        t = torch.ones(n); dist.all_reduce(t)
    b = torch.ones(50000); dist.broadcast(b, 0)
    outs = [torch.zeros(10) for _ in range(ws)]; dist.all_gather(outs, torch.ones(10))
    dist.barrier()
    m = mccl.get_metrics()
    assert m.total_ops >= 6, m.total_ops
    assert m.total_bytes_sent > 0 and m.total_errors == 0
    assert m.avg_latency_ms > 0 and m.p50_latency_ms > 0 and m.p99_latency_ms >= m.p50_latency_ms
    assert m.peak_throughput_gbps > 0 and m.avg_network_ms > 0 and m.avg_execution_ms > 0
    assert m.avg_queue_wait_ms >= 0 and m.avg_reduce_ms >= 0 and m.avg_sync_ms >= 0
    mccl.log_metrics()
    mccl.reset_metrics()
    m2 = mccl.get_metrics()
    assert m2.total_ops == 0 and m2.total_bytes_sent == 0
    assert mccl.staging_pool_bytes() > 0
    mccl.trim_staging_pool()


def test_metrics_populated_and_reset():
    run_workers(_metrics, 3, timeout=120)
