"""Reference test scenarios on the GPU data plane (one process per GPU, >= 2 devices).

* train -> barrier -> rank-skewed validation -> train with no host synchronisation between backward
  and the optimizer step (reference tests/test_ddp_consumer_release.py)
* convolution backward overlapped with bucketed allreduce, against a single-process run on the
  union batch (reference tests/test_ddp_conv_overlap.py)
* Lightning-style set-up traffic: broadcast_object_list, int64 all_gather at 5..8 ranks,
  DDP(init_sync=True), a 512 KiB uint8 broadcast of a CPU tensor
  (reference tests/test_broadcast_object_list.py:206-223)
* device metrics: every summary field is populated on every rank after real traffic
  (reference tests/test_metrics.py:23-91)
* the host-staged fallback (MCCL_ALGO=staged) and two process groups used side by side
"""
import pytest
import torch

from mccl_b200.utils.spawn import run_workers

pytestmark = [pytest.mark.gpu(count=2)]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _world_sizes(cands=(2, 4, 8)):
    return [w for w in cands if w <= max(_ngpu(), 2)]


def _consumer_release(rank, ws):
    import time
    import torch, torch.distributed as dist
    from mccl_b200.parallel import wrap_ddp
    def make():
        torch.manual_seed(11)
        return torch.nn.Sequential(torch.nn.Linear(256, 1024), torch.nn.ReLU(), torch.nn.Linear(1024, 1024),
                                   torch.nn.ReLU(), torch.nn.Linear(1024, 32)).to(device)
    model = wrap_ddp(make(), device_ids=[device.index], bucket_cap_mb=1)
    ref = make()
    opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
    g = torch.Generator().manual_seed(5)

    def train(steps):
        for _ in range(steps):
            xs = torch.randn(8 * ws, 256, generator=g); ys = torch.randint(0, 32, (8 * ws,), generator=g)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(xs[rank * 8:(rank + 1) * 8].to(device)), ys[rank * 8:(rank + 1) * 8].to(device)).backward()
            opt.step()                       # no synchronize(), no .item(): ordering is on the device only
            ref_opt.zero_grad()
            torch.nn.functional.cross_entropy(ref(xs.to(device)), ys.to(device)).backward()
            ref_opt.step()

    train(6)
    dist.barrier()
    # validation with a different amount of work per rank, then a reduction of the metric
    model.eval()
    with torch.no_grad():
        tot = torch.zeros(1, device=device)
        for i in range(2 + 3 * rank):
            tot += model(torch.randn(64, 256, device=device)).square().mean()
        if rank == 0:
            time.sleep(0.2)
        cnt = torch.tensor([float(2 + 3 * rank)], device=device)
        dist.all_reduce(tot); dist.all_reduce(cnt)
        assert cnt.item() == sum(2 + 3 * r for r in range(ws))
    model.train()
    # burst of barriers and small allreduces right before training resumes
    for i in range(10):
        dist.barrier()
        t = torch.full((1000,), float(i), device=device); dist.all_reduce(t)
    train(6)
    torch.cuda.synchronize()
    for p, q in zip(model.module.parameters(), ref.parameters()):
        assert torch.allclose(p, q, rtol=2e-4, atol=2e-5), (p - q).abs().max()


@pytest.mark.parametrize("ws", _world_sizes())
def test_train_barrier_skewed_validation_train_without_host_sync(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    run_workers(_consumer_release, ws, device="cuda", timeout=300)


def _conv_overlap(rank, ws):
    import torch, torch.distributed as dist
    from mccl_b200.parallel import wrap_ddp
    def make():
        torch.manual_seed(2)
        return torch.nn.Sequential(
            torch.nn.Conv2d(3, 32, 3, padding=1), torch.nn.ReLU(), torch.nn.Conv2d(32, 64, 3, padding=1, stride=2),
            torch.nn.ReLU(), torch.nn.Conv2d(64, 64, 3, padding=1), torch.nn.ReLU(), torch.nn.AdaptiveAvgPool2d(4),
            torch.nn.Flatten(), torch.nn.Linear(1024, 512), torch.nn.ReLU(), torch.nn.Linear(512, 10)).to(device)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    model = wrap_ddp(make(), device_ids=[device.index], bucket_cap_mb=1)   # several buckets in flight during backward
    ref = make()
    opt = torch.optim.SGD(model.parameters(), lr=0.02)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.02)
    g = torch.Generator().manual_seed(9)
    for step in range(5):
        xs = torch.randn(4 * ws, 3, 32, 32, generator=g); ys = torch.randint(0, 10, (4 * ws,), generator=g)
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(xs[rank * 4:(rank + 1) * 4].to(device)), ys[rank * 4:(rank + 1) * 4].to(device)).backward()
        # gradient parity against one process on the union batch, every step
        ref_opt.zero_grad()
        torch.nn.functional.cross_entropy(ref(xs.to(device)), ys.to(device)).backward()
        for p, q in zip(model.module.parameters(), ref.parameters()):
            assert torch.allclose(p.grad, q.grad, rtol=2e-3, atol=2e-5), (step, (p.grad - q.grad).abs().max())
        opt.step(); ref_opt.step()
    # replicas stay bit-identical
    flat = torch.cat([p.detach().reshape(-1) for p in model.module.parameters()])
    outs = [torch.empty_like(flat) for _ in range(ws)]
    dist.all_gather(outs, flat)
    for o in outs:
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("ws", _world_sizes((2, 4, 8)))
def test_conv_backward_overlaps_bucketed_allreduce(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    run_workers(_conv_overlap, ws, device="cuda", timeout=300)


def _lightning_setup(rank, ws):
    import torch, torch.distributed as dist
    objs = [{"seed": 1234, "name": "run-7", "nested": [1, 2, 3]}, "text", 42] if rank == 0 else [None, None, None]
    dist.broadcast_object_list(objs, src=0, device=device)
    assert objs[0]["nested"] == [1, 2, 3] and objs[1] == "text" and objs[2] == 42
    out = [None] * ws
    dist.all_gather_object(out, {"rank": rank, "pad": "x" * (rank * 37)})
    assert [o["rank"] for o in out] == list(range(ws))
    # int64 metadata allgather (what the DDP constructor and Lightning do)
    mine = torch.tensor([rank * 1000 + 7, rank], dtype=torch.int64, device=device)
    got = [torch.empty_like(mine) for _ in range(ws)]
    dist.all_gather(got, mine)
    assert [int(t[0]) for t in got] == [r * 1000 + 7 for r in range(ws)]
    # CPU uint8 512 KiB broadcast through the same group (host transport)
    payload = (torch.arange(512 * 1024) % 251).to(torch.uint8) if rank == 1 % ws else torch.zeros(512 * 1024, dtype=torch.uint8)
    dist.broadcast(payload, 1 % ws)
    assert int(payload[-1]) == (512 * 1024 - 1) % 251
    # DDP(init_sync=True): parameters that differ before construction are equal after it
    torch.manual_seed(100 + rank)
    m = torch.nn.Linear(64, 64).to(device)
    ddp = torch.nn.parallel.DistributedDataParallel(m, device_ids=[device.index], init_sync=True)
    w = ddp.module.weight.detach().clone()
    ws_list = [torch.empty_like(w) for _ in range(ws)]
    dist.all_gather(ws_list, w)
    for o in ws_list:
        assert torch.equal(o, ws_list[0])


@pytest.mark.parametrize("ws", _world_sizes((2, 5, 8)))
def test_object_lists_int64_allgather_init_sync_and_cpu_broadcast(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    run_workers(_lightning_setup, ws, device="cuda", timeout=300)


def _device_metrics(rank, ws):
    import torch, torch.distributed as dist
    mccl.reset_metrics()
    for n in (10, 100_000, 4_000_000, 20_000_000):      # one-shot, two-shot (and segmented) kernels
        for _ in range(3):
            t = torch.ones(n, device=device); dist.all_reduce(t)
    b = torch.ones(500_000, device=device); dist.broadcast(b, 0)
    o = torch.empty(1000 * ws, device=device); dist.all_gather_into_tensor(o, torch.ones(1000, device=device))
    rs = torch.empty(1000, device=device); dist.reduce_scatter_tensor(rs, torch.ones(1000 * ws, device=device))
    dist.barrier()
    torch.cuda.synchronize()
    import time; time.sleep(1.2)              # two watchdog polls retire the timed collectives
    m = mccl.get_metrics()
    assert m.total_ops >= 15 and m.total_errors == 0, (m.total_ops, m.total_errors)
    assert m.total_bytes_sent > 0 and m.total_bytes_recv > 0
    assert m.avg_latency_ms > 0 and m.p50_latency_ms > 0 and m.p99_latency_ms >= m.p50_latency_ms
    assert m.peak_throughput_gbps > 0
    assert m.avg_sync_ms > 0, "host time spent fencing streams"
    assert m.avg_network_ms > 0, "device time of the transfer phases"
    assert m.avg_reduce_ms > 0, "device time of the reduction phase (in-kernel stamps)"
    assert m.avg_execution_ms > 0 and m.avg_queue_wait_ms >= 0
    mccl.reset_metrics()
    m2 = mccl.get_metrics()
    assert m2.total_ops == 0 and m2.total_bytes_sent == 0


def test_device_metrics_every_field_populated():
    run_workers(_device_metrics, 2, device="cuda", timeout=240, env={"MCCL_DEVICE_TIMING": "1"})


def _staged(rank, ws):
    import torch, torch.distributed as dist
    be = mccl.get_backend(device=device)
    t = torch.arange(100_003, device=device, dtype=torch.float32) * (rank + 1)
    dist.all_reduce(t)
    assert be.data_plane() == "host-staged", be.data_plane()
    assert torch.equal(t, torch.arange(100_003, device=device, dtype=torch.float32) * sum(range(1, ws + 1)))
    b = torch.full((70_001,), 7.0, device=device) if rank == 1 else torch.zeros(70_001, device=device)
    dist.broadcast(b, 1)
    assert b[-1].item() == 7.0
    o = torch.empty(257 * ws, device=device)
    dist.all_gather_into_tensor(o, torch.full((257,), float(rank), device=device))
    assert [o[r * 257].item() for r in range(ws)] == [float(r) for r in range(ws)]
    r_out = torch.empty(100, device=device)
    dist.reduce_scatter_tensor(r_out, torch.ones(100 * ws, device=device) * (rank + 1))
    assert r_out[0].item() == sum(range(1, ws + 1))
    dist.barrier()


def test_host_staged_fallback_on_gpus():
    run_workers(_staged, 2, device="cuda", timeout=240, env={"MCCL_ALGO": "staged"})


def _two_groups(rank, ws):
    import torch, torch.distributed as dist
    # a second CUDA process group next to the default one: both keep their kernels small enough to
    # be co-resident, and collectives of the two groups are issued back to back and interleaved
    g2 = dist.new_group(backend="mccl")
    xs = [torch.full((50_000,), float(rank + i), device=device) for i in range(8)]
    ys = [torch.full((50_000,), float(2 * rank + i), device=device) for i in range(8)]
    works = []
    for i in range(8):
        works.append(dist.all_reduce(xs[i], async_op=True))
        works.append(dist.all_reduce(ys[i], group=g2, async_op=True))
    for w in works:
        w.wait()
    torch.cuda.synchronize()
    for i in range(8):
        assert xs[i][0].item() == sum(r + i for r in range(ws))
        assert ys[i][-1].item() == sum(2 * r + i for r in range(ws))
    b = torch.full((1000,), 3.0, device=device) if rank == 0 else torch.zeros(1000, device=device)
    dist.broadcast(b, 0, group=g2)
    assert b[5].item() == 3.0
    dist.barrier(group=g2); dist.barrier()
    assert mccl.get_backend(group=g2, device=device).data_plane().startswith("nvlink-p2p")


def test_two_cuda_process_groups_side_by_side():
    run_workers(_two_groups, 2, device="cuda", timeout=240,
                env={"MCCL_COMM_CTAS": "16", "MCCL_DEVICE_WAIT_US": "3000000"})


def _ctas_clamped(rank, ws):
    import torch, torch.distributed as dist
    t = torch.ones(30_000_000, device=device)
    for _ in range(4):
        dist.all_reduce(t)      # two lanes in flight; a request for 128 CTAs is clamped to 64 each
    torch.cuda.synchronize()
    assert t[0].item() == float(ws) ** 4
    assert mccl.get_metrics().total_errors == 0


def test_oversized_cta_request_is_clamped_not_timed_out():
    run_workers(_ctas_clamped, 2, device="cuda", timeout=240, env={"MCCL_COMM_CTAS": "128", "MCCL_DEVICE_WAIT_US": "3000000"})


def _info_lines(rank, ws):
    import time
    import torch, torch.distributed as dist
    t = torch.ones(2_000_000, device=device); dist.all_reduce(t)
    t = torch.ones(1000, device=device); dist.all_reduce(t)
    b = torch.ones(300_000, device=device); dist.broadcast(b, 0)
    o = torch.empty(1000 * ws, device=device); dist.all_gather_into_tensor(o, torch.ones(1000, device=device))
    rs = torch.empty(1000, device=device); dist.reduce_scatter_tensor(rs, torch.ones(1000 * ws, device=device))
    torch.cuda.synchronize()
    time.sleep(1.2)   # the watchdog poll retires the timed collectives and prints their lines


def test_one_info_line_per_collective_with_variant_time_and_busbw():
    import re
    res = run_workers(_info_lines, 2, device="cuda", timeout=240,
                      env={"MCCL_LOG_LEVEL": "INFO", "MCCL_DEVICE_TIMING": "1"})
    err = res[0].stderr
    for name, algo in (("mccl:all_reduce", "twoshot|oneshot|nvls"), ("mccl:broadcast", "direct|twohop|nvls"),
                       ("mccl:all_gather", "push"), ("mccl:reduce_scatter", ".*")):
        pat = re.compile(rf"{name} seq=\d+ algo=({algo})\S* bytes=\d+ device_us=[0-9.]+ busbw=[0-9.]+ GB/s")
        assert pat.search(err), f"no INFO line for {name}:\n{err[-3000:]}"
