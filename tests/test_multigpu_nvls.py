"""NVLS (NVLink multicast) kernels on real GPUs: allreduce reduced inside the NVSwitch
(``multimem.ld_reduce`` + ``multimem.st``), allgather and broadcast moved with one
``multimem.st`` per unit.  One process per GPU; needs >= 2 CUDA devices behind an NVSwitch.

Oracles: float64 analytic sums, bitwise identity across ranks (each element is reduced by exactly
one rank), distinct-value patterns for the byte movers, and the point-to-point kernels of the same
library as a differential reference.  Every worker runs to completion and tears the multicast
binding down in ``destroy_process_group``; no failure is injected while NVLS is on.
"""
import pytest
import torch

from mccl_b200.utils.spawn import run_workers

pytestmark = [pytest.mark.gpu(count=2)]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _world_sizes():
    return [w for w in (2, 4, 8) if w <= max(_ngpu(), 2)]


def _skip_if_unavailable(results):
    if any("NVLS_UNAVAILABLE" in (r.stdout or "") for r in results):
        pytest.skip("this box offers no NVLink multicast (the group fell back to the peer-memory kernels)")


def _nvls_allreduce_worker(rank, ws):
    import torch, torch.distributed as dist
    be = mccl.get_backend(device=device)
    warm = torch.ones(8, device=device)
    dist.all_reduce(warm)
    if be.data_plane() != "nvlink-p2p+nvls":
        print("NVLS_UNAVAILABLE", be.data_plane(), flush=True)
        return
    sizes = [1, 3, 1023, 4097, 70001, 262147, 2100001, 20_000_003]
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for n in sizes:
            base = (torch.arange(n, device=device) % 17).to(dtype)
            t = base * (rank + 1)
            dist.all_reduce(t)
            want = base.double() * sum(range(1, ws + 1))
            assert torch.allclose(t.double(), want, rtol=2e-2 if dtype != torch.float32 else 1e-6), (dtype, n)
            t = base * (rank + 1)
            dist.all_reduce(t, op=dist.ReduceOp.AVG)
            assert torch.allclose(t.double(), want / ws, rtol=2e-2 if dtype != torch.float32 else 1e-6), (dtype, n, "avg")
    # random data: float64 oracle through an all_gather of the inputs, and bitwise identity
    for n in (300007, 9_000_001):
        g = torch.Generator(device="cpu").manual_seed(rank * 7 + n)
        x = torch.randn(n, generator=g).to(device)
        ins = [torch.empty_like(x) for _ in range(ws)]
        dist.all_gather(ins, x)
        want = torch.stack([i.double() for i in ins]).sum(0)
        dist.all_reduce(x)
        assert (x.double() - want).abs().max().item() <= 1e-5 * max(1.0, want.abs().max().item()) * ws
        outs = [torch.empty_like(x) for _ in range(ws)]
        dist.all_gather(outs, x)
        for o in outs:
            assert torch.equal(o, outs[0])
    # dtypes / ops the switch does not reduce fall back to the peer-memory kernels
    t = torch.full((100001,), rank + 1, device=device, dtype=torch.int64)
    dist.all_reduce(t)
    assert t[0].item() == sum(range(1, ws + 1))
    t = torch.full((100001,), float(rank), device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t[-1].item() == ws - 1
    # buffer reuse: many back-to-back epochs of alternating sizes through the four NVLS buffers
    for it in range(40):
        n = [17, 500_000, 4097, 3_000_000][it % 4]
        t = torch.full((n,), float(it + rank), device=device)
        dist.all_reduce(t)
        if it % 8 == 7:
            torch.cuda.synchronize()
            assert t[0].item() == sum(it + r for r in range(ws)) and t[-1].item() == t[0].item()
    m = mccl.get_metrics()
    assert m.total_errors == 0


@pytest.mark.parametrize("ws", _world_sizes())
def test_nvls_allreduce(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    res = run_workers(_nvls_allreduce_worker, ws, device="cuda", timeout=300,
                      env={"MCCL_NVLS": "1", "MCCL_ALGO": "nvls"})
    _skip_if_unavailable(res)


def _nvls_tiles_worker(rank, ws):
    import torch, torch.distributed as dist
    be = mccl.get_backend(device=device)
    dist.all_reduce(torch.ones(8, device=device))
    if be.data_plane() != "nvlink-p2p+nvls":
        print("NVLS_UNAVAILABLE", flush=True)
        return
    # small tiles: every CTA runs many stage / reduce / copy-out iterations; wire cast on
    for n in (70001, 5_000_011):
        for rep in range(3):
            g = torch.Generator(device="cpu").manual_seed(rank + 10 * rep)
            x = torch.randn(n, generator=g).to(device)
            ins = [torch.empty_like(x) for _ in range(ws)]
            dist.all_gather(ins, x)
            acc = ins[0].bfloat16().float()
            for i in ins[1:]:
                acc = acc + i.bfloat16().float()
            dist.all_reduce(x, op=dist.ReduceOp.AVG)
            want = (acc.double() / ws)
            assert torch.allclose(x.double(), want, rtol=2e-2, atol=2e-2), (n, rep)
            outs = [torch.empty_like(x) for _ in range(ws)]
            dist.all_gather(outs, x)
            for o in outs:
                assert torch.equal(o, outs[0])


@pytest.mark.parametrize("ws", _world_sizes()[:1] + _world_sizes()[-1:])
def test_nvls_allreduce_small_tiles_and_wire_cast(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    res = run_workers(_nvls_tiles_worker, ws, device="cuda", timeout=300,
                      env={"MCCL_NVLS": "1", "MCCL_ALGO": "nvls", "MCCL_TILE_BYTES": "32768", "MCCL_WIRE_DTYPE": "bf16"})
    _skip_if_unavailable(res)


def _nvls_movers_worker(rank, ws):
    import torch, torch.distributed as dist
    be = mccl.get_backend(device=device)
    dist.all_reduce(torch.ones(8, device=device))
    if be.data_plane() != "nvlink-p2p+nvls":
        print("NVLS_UNAVAILABLE", flush=True)
        return
    for root in range(ws):
        for n in (1, 4096, 1_000_003, 40_000_001):
            b = (torch.arange(n, device=device, dtype=torch.float32) + root) if rank == root else torch.zeros(n, device=device)
            dist.broadcast(b, root)
            assert b[0].item() == root and b[n - 1].item() == float(torch.tensor(n - 1 + root, dtype=torch.float32)), (root, n)
            if n <= 1_000_003:
                assert torch.equal(b, torch.arange(n, device=device, dtype=torch.float32) + root)
    for dtype, n in ((torch.int64, 1), (torch.int64, 513), (torch.float16, 70001), (torch.uint8, 1_000_003), (torch.float32, 9_000_001)):
        i = (torch.arange(n, device=device) % 251 + rank).to(dtype)
        o = torch.empty(n * ws, dtype=dtype, device=device)
        dist.all_gather_into_tensor(o, i)
        want = torch.cat([(torch.arange(n, device=device) % 251 + r).to(dtype) for r in range(ws)])
        assert torch.equal(o, want), (dtype, n)
    # a per-rank block larger than one staging slot goes slice by slice, each slice in place
    n = 12_000_000
    i = torch.full((n,), float(rank), device=device)
    o = torch.empty(n * ws, device=device)
    dist.all_gather_into_tensor(o, i)
    assert [o[r * n].item() for r in range(ws)] == [float(r) for r in range(ws)]
    assert [o[(r + 1) * n - 1].item() for r in range(ws)] == [float(r) for r in range(ws)]
    assert mccl.get_metrics().total_errors == 0


@pytest.mark.parametrize("ws", _world_sizes())
def test_nvls_broadcast_and_allgather(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    res = run_workers(_nvls_movers_worker, ws, device="cuda", timeout=300,
                      env={"MCCL_NVLS": "1", "MCCL_ALGO": "nvls"})
    _skip_if_unavailable(res)


def _nvls_auto_ddp_worker(rank, ws):
    import torch, torch.distributed as dist
    from mccl_b200.parallel import wrap_ddp
    # tuner-driven choice (auto): small buckets take the one-shot kernel, large ones NVLS where the
    # table says so; replicas must stay bit-identical and match a single process on the union batch
    def make():
        torch.manual_seed(42)
        return torch.nn.Sequential(torch.nn.Linear(512, 4096), torch.nn.ReLU(), torch.nn.Linear(4096, 4096),
                                   torch.nn.ReLU(), torch.nn.Linear(4096, 10)).to(device)
    ref = make()
    model = wrap_ddp(make(), device_ids=[device.index], bucket_cap_mb=25)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(7)
    for step in range(5):
        xs = torch.randn(8 * ws, 512, generator=g)
        ys = torch.randint(0, 10, (8 * ws,), generator=g)
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(xs[rank * 8:(rank + 1) * 8].to(device)), ys[rank * 8:(rank + 1) * 8].to(device)).backward()
        opt.step()
        ref_opt.zero_grad()
        torch.nn.functional.cross_entropy(ref(xs.to(device)), ys.to(device)).backward()
        ref_opt.step()
    for p, q in zip(model.module.parameters(), ref.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=1e-5), (p - q).abs().max()
    flat = torch.cat([p.detach().reshape(-1) for p in model.module.parameters()])
    outs = [torch.empty_like(flat) for _ in range(ws)]
    dist.all_gather(outs, flat)
    for o in outs:
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("ws", _world_sizes())
def test_ddp_with_nvls_auto(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    run_workers(_nvls_auto_ddp_worker, ws, device="cuda", timeout=300,
                env={"MCCL_NVLS": "1", "MCCL_NVLS_MIN_BYTES": "1048577"})


def _inplace_worker(rank, ws):
    import torch, torch.distributed as dist
    from mccl_b200.parallel.ddp import _nvls_bucket_pool
    from mccl_b200.parallel import wrap_ddp
    native = mccl.require_native()
    be = mccl.get_backend(device=device)
    dist.all_reduce(torch.ones(8, device=device))
    if not be.data_plane().endswith("+nvls"):
        print("NVLS_UNAVAILABLE", flush=True)
        return
    # 1. raw tensors from the multicast-bound pool are reduced in place by the switch
    holder = torch.nn.Linear(4096, 4096).to(device)          # sizes the pool (about 64 MiB x 4 + slack)
    pool = _nvls_bucket_pool(holder, None)
    assert pool is not None
    with torch.cuda.use_mem_pool(pool):
        bufs = {dt: torch.empty(3_000_000, dtype=dt, device=device) for dt in (torch.float32, torch.bfloat16, torch.float16)}
        small = torch.empty(1000, device=device)
    for dt, buf in bufs.items():
        assert native._nvls_pool_contains(buf)
        for rep in range(3):
            g = torch.Generator().manual_seed(rank * 31 + rep)
            x = torch.randn(buf.numel(), generator=g).to(device).to(dt)
            ins = [torch.empty_like(x) for _ in range(ws)]
            dist.all_gather(ins, x)
            want = torch.stack([i.double() for i in ins]).sum(0)
            buf.copy_(x)
            dist.all_reduce(buf, op=dist.ReduceOp.AVG if rep == 1 else dist.ReduceOp.SUM)
            if rep == 1:
                want = want / ws
            tol = 1e-5 if dt == torch.float32 else 3e-2
            assert (buf.double() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item()) * ws, (dt, rep)
            outs = [torch.empty_like(buf) for _ in range(ws)]
            dist.all_gather(outs, buf)
            for o in outs:
                assert torch.equal(o, outs[0])
        # a view whose byte length is not a multiple of 16 takes the staged path and leaves its neighbours alone
        buf.fill_(1)
        v = buf[5:5 + 1001]
        dist.all_reduce(v)
        assert buf[4].item() == 1 and buf[5].item() == ws and buf[5 + 1000].item() == ws and buf[5 + 1001].item() == 1
    small.fill_(2.0); dist.all_reduce(small); assert small[0].item() == 2.0 * ws    # below the in-place floor
    # 2. DDP buckets land in the pool (before and after DDP re-buckets) and training matches one process
    def make():
        torch.manual_seed(42)
        return torch.nn.Sequential(torch.nn.Linear(512, 2048), torch.nn.ReLU(), torch.nn.Linear(2048, 2048),
                                   torch.nn.ReLU(), torch.nn.Linear(2048, 10)).to(device)
    ref = make()
    model = wrap_ddp(make(), device_ids=[device.index], bucket_cap_mb=4)
    assert getattr(model, "_mccl_nvls_pool", None) is not None
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(7)
    for step in range(5):
        xs = torch.randn(8 * ws, 512, generator=g); ys = torch.randint(0, 10, (8 * ws,), generator=g)
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(xs[rank * 8:(rank + 1) * 8].to(device)), ys[rank * 8:(rank + 1) * 8].to(device)).backward()
        in_pool = [native._nvls_pool_contains(p.grad) for p in model.module.parameters()]
        assert all(in_pool), (step, in_pool)
        opt.step()
        ref_opt.zero_grad()
        torch.nn.functional.cross_entropy(ref(xs.to(device)), ys.to(device)).backward()
        ref_opt.step()
    for p, q in zip(model.module.parameters(), ref.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=1e-5), (p - q).abs().max()
    assert mccl.get_metrics().total_errors == 0


@pytest.mark.parametrize("ws", _world_sizes())
def test_nvls_in_place_allreduce_on_pool_tensors_and_ddp_buckets(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    res = run_workers(_inplace_worker, ws, device="cuda", timeout=300,
                      env={"MCCL_NVLS": "1", "MCCL_LOG_LEVEL": "INFO", "MCCL_DEVICE_TIMING": "1", "MCCL_NVLS_BUCKETS_MIN_WORLD": "2",
                           "MCCL_NVLS_INPLACE_MIN_BYTES": "1048576"})
    _skip_if_unavailable(res)
    if "NVLS_UNAVAILABLE" not in res[0].stdout:
        assert "algo=nvls-inplace" in res[0].stderr, res[0].stderr[-2000:]
