"""Real multi-GPU runs of the NVLink peer-memory data plane (one process per GPU).

Worker source is serialised into child processes with a hard wall-clock limit
(mccl_b200.utils.spawn).  Needs >= 2 CUDA devices; world sizes above the
device count are skipped.
"""
import pytest
import torch

from mccl_b200.utils.spawn import run_workers

pytestmark = [pytest.mark.gpu(count=2)]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _world_sizes():
    return [w for w in (2, 4, 8) if w <= max(_ngpu(), 2)]


def _collectives_worker(rank, ws):
    import torch, torch.distributed as dist
    be = mccl.get_backend(device=device)
    sizes = [1, 3, 1023, 4097, 70001, 262147, 2100001]
    for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.int64, torch.int32):
        for n in sizes:
            base = (torch.arange(n, device=device) % 17).to(dtype)
            t = base * (rank + 1) if dtype.is_floating_point else base * (rank + 1)
            dist.all_reduce(t)
            want = (base.double() * sum(range(1, ws + 1)))
            assert torch.allclose(t.double(), want, rtol=2e-2 if dtype != torch.float32 else 1e-6), (dtype, n)
    assert be.data_plane() == "nvlink-p2p", be.data_plane()
    # ops
    for op, fn in ((dist.ReduceOp.MAX, max), (dist.ReduceOp.MIN, min)):
        t = torch.full((5000,), float(rank), device=device)
        dist.all_reduce(t, op=op)
        assert t[0].item() == fn(range(ws))
    t = torch.full((100001,), float(rank + 1), device=device)
    dist.all_reduce(t, op=dist.ReduceOp.AVG)
    assert abs(t[0].item() - (ws + 1) / 2) < 1e-6
    # bitwise identity across ranks
    g = torch.Generator(device="cpu").manual_seed(rank)
    x = torch.randn(300007, generator=g).to(device)
    dist.all_reduce(x)
    gathered = [torch.empty_like(x) for _ in range(ws)]
    dist.all_gather(gathered, x)
    for o in gathered:
        assert torch.equal(o, gathered[0])
    # broadcast from every root
    for root in range(ws):
        for n in (1, 4096, 1000003):
            b = torch.arange(n, device=device, dtype=torch.float32) + root if rank == root else torch.zeros(n, device=device)
            dist.broadcast(b, root)
            assert b[n - 1].item() == n - 1 + root
    # all_gather_into_tensor / reduce_scatter_tensor
    inp = torch.full((70001,), float(rank), device=device)
    out = torch.empty(70001 * ws, device=device)
    dist.all_gather_into_tensor(out, inp)
    assert [out[i * 70001].item() for i in range(ws)] == [float(i) for i in range(ws)]
    rs_in = torch.arange(ws * 1001, device=device, dtype=torch.float32)
    rs_out = torch.empty(1001, device=device)
    dist.reduce_scatter_tensor(rs_out, rs_in)
    assert torch.equal(rs_out, rs_in[rank * 1001:(rank + 1) * 1001] * ws)
    lst = [torch.full((33,), float(rank * 10 + i), device=device) for i in range(ws)]
    o2 = torch.empty(33, device=device)
    dist.reduce_scatter(o2, lst)
    assert o2[0].item() == sum(r * 10 + rank for r in range(ws))
    dist.barrier()
    # send / recv of CUDA tensors (NCCL p2p on a side stream), while an allreduce is in flight
    nxt, prv = (rank + 1) % ws, (rank - 1) % ws
    big = torch.ones(8_000_000, device=device)
    w_ar = dist.all_reduce(big, async_op=True)
    payload = torch.full((100003,), float(rank), device=device)
    got = torch.empty(100003, device=device)
    if rank % 2 == 0:
        dist.send(payload, nxt); dist.recv(got, prv)
    else:
        dist.recv(got, prv); dist.send(payload, nxt)
    w_ar.wait()
    torch.cuda.synchronize()
    assert got[0].item() == prv and got[-1].item() == prv and big[0].item() == ws
    # async burst: many outstanding works
    works = []
    ts = [torch.full((65536,), float(i), device=device) for i in range(24)]
    for t in ts:
        works.append(dist.all_reduce(t, async_op=True))
    for w in works:
        w.wait()
    torch.cuda.synchronize()
    assert all(ts[i][0].item() == i * ws for i in range(24))
    m = mccl.get_metrics()
    assert m.total_ops > 0 and m.total_bytes_sent > 0 and m.total_errors == 0


@pytest.mark.parametrize("ws", _world_sizes())
def test_collectives_over_nvlink(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    run_workers(_collectives_worker, ws, device="cuda", timeout=240)


def _push_gather_worker(rank, ws):
    import torch, torch.distributed as dist
    # two-shot with owners pushing the reduced chunks; back-to-back calls exercise both lanes and
    # the reuse of the arena's second half
    for dtype in (torch.float32, torch.bfloat16):
        for n in (1, 4097, 262147, 2100001, 12_000_001):
            for rep in range(3):
                base = (torch.arange(n, device=device) % 13).to(dtype)
                t = base * (rank + 1 + rep)
                dist.all_reduce(t)
                want = base.double() * sum(r + 1 + rep for r in range(ws))
                assert torch.allclose(t.double(), want, rtol=2e-2 if dtype != torch.float32 else 1e-6), (dtype, n, rep)
    g = torch.Generator(device="cpu").manual_seed(rank)
    x = torch.randn(3_000_007, generator=g).to(device)
    dist.all_reduce(x, op=dist.ReduceOp.AVG)
    outs = [torch.empty_like(x) for _ in range(ws)]
    dist.all_gather(outs, x)
    for o in outs:
        assert torch.equal(o, outs[0])
    assert mccl.get_metrics().total_errors == 0


@pytest.mark.parametrize("ws", _world_sizes())
def test_twoshot_push_gather_over_nvlink(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    run_workers(_push_gather_worker, ws, device="cuda", timeout=240,
                env={"MCCL_GATHER": "push", "MCCL_ALGO": "twoshot"})


def _ddp_worker(rank, ws):
    import torch, torch.distributed as dist
    from mccl_b200.parallel import wrap_ddp
    from mccl_b200.optim import FusedAdamW
    def make():
        torch.manual_seed(42)
        return torch.nn.Sequential(torch.nn.Linear(512, 2048), torch.nn.ReLU(), torch.nn.Linear(2048, 2048),
                                   torch.nn.ReLU(), torch.nn.Linear(2048, 10)).to(device)
    # 1. parity with a single process on the union batch (SGD: linear in the gradients, so the
    #    comparison measures the gradient averaging and not an optimizer's amplification)
    ref = make()
    model = wrap_ddp(make(), device_ids=[device.index], bucket_cap_mb=4)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(7)
    for step in range(5):
        xs = torch.randn(8 * ws, 512, generator=g)
        ys = torch.randint(0, 10, (8 * ws,), generator=g)
        opt.zero_grad()   # no host sync between backward and step
        torch.nn.functional.cross_entropy(model(xs[rank * 8:(rank + 1) * 8].to(device)), ys[rank * 8:(rank + 1) * 8].to(device)).backward()
        opt.step()
        ref_opt.zero_grad()
        torch.nn.functional.cross_entropy(ref(xs.to(device)), ys.to(device)).backward()
        ref_opt.step()
    for p, q in zip(model.module.parameters(), ref.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=1e-5), (p - q).abs().max()
    # 2. the fused AdamW path: replicas stay bit-identical
    opt2 = FusedAdamW(model.parameters(), lr=1e-3)
    for step in range(4):
        x = torch.randn(8, 512, generator=g).to(device); y = torch.randint(0, 10, (8,), generator=g).to(device)
        opt2.zero_grad(); torch.nn.functional.cross_entropy(model(x), y).backward(); opt2.step()
    flat = torch.cat([p.detach().reshape(-1) for p in model.module.parameters()])
    outs = [torch.empty_like(flat) for _ in range(ws)]
    dist.all_gather(outs, flat)
    for o in outs:
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("ws", _world_sizes())
def test_ddp_matches_single_process(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    run_workers(_ddp_worker, ws, device="cuda", timeout=240)


def _oib_worker(rank, ws):
    import torch, torch.distributed as dist
    from mccl_b200.parallel import wrap_ddp
    from mccl_b200.optim import FusedAdamW
    def make():
        torch.manual_seed(3)
        return torch.nn.Sequential(torch.nn.Linear(256, 1024), torch.nn.GELU(), torch.nn.Linear(1024, 1024),
                                   torch.nn.GELU(), torch.nn.Linear(1024, 16)).to(device)
    def groups(m):
        # two param groups with different hyper-parameters; buckets hold members of both
        decay = [p for p in m.parameters() if p.ndim > 1]
        rest = [p for p in m.parameters() if p.ndim <= 1]
        return [{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0, "lr": 3e-3}]
    a, b = make(), make()
    opt_a = FusedAdamW(groups(a), lr=1e-3)
    opt_b = FusedAdamW(groups(b), lr=1e-3)
    sched_a = torch.optim.lr_scheduler.StepLR(opt_a, step_size=2, gamma=0.5)
    sched_b = torch.optim.lr_scheduler.StepLR(opt_b, step_size=2, gamma=0.5)
    da = wrap_ddp(a, device_ids=[device.index], bucket_cap_mb=1)                                 # step after backward
    db = wrap_ddp(b, device_ids=[device.index], bucket_cap_mb=1, optimizer_in_backward=opt_b)    # step per bucket
    g = torch.Generator().manual_seed(rank)
    for _ in range(6):
        x = torch.randn(16, 256, generator=g).to(device); y = torch.randint(0, 16, (16,), generator=g).to(device)
        for d, o, s in ((da, opt_a, sched_a), (db, opt_b, sched_b)):
            o.zero_grad(); torch.nn.functional.cross_entropy(d(x), y).backward(); o.step(); s.step()
    for p, q in zip(a.parameters(), b.parameters()):
        assert torch.equal(p, q), (p - q).abs().max()
    assert int(opt_b.state[next(b.parameters())]["step"].item()) == 6
    sd = opt_b.state_dict()   # same layout as torch.optim.AdamW: loads into it
    ref = torch.optim.AdamW(groups(b), lr=1e-3); ref.load_state_dict(sd)
    # and against torch's own AdamW with the same groups and schedule, on the same data
    c = make()
    opt_c = torch.optim.AdamW(groups(c), lr=1e-3)
    sched_c = torch.optim.lr_scheduler.StepLR(opt_c, step_size=2, gamma=0.5)
    dc = wrap_ddp(c, device_ids=[device.index], bucket_cap_mb=1)
    g = torch.Generator().manual_seed(rank)
    for _ in range(6):
        x = torch.randn(16, 256, generator=g).to(device); y = torch.randint(0, 16, (16,), generator=g).to(device)
        opt_c.zero_grad(); torch.nn.functional.cross_entropy(dc(x), y).backward(); opt_c.step(); sched_c.step()
    for p, q in zip(b.parameters(), c.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=2e-5), (p - q).abs().max()


@pytest.mark.parametrize("ws", _world_sizes())
def test_optimizer_in_backward_matches_regular_step(ws):
    if ws > _ngpu():
        pytest.skip("not enough GPUs")
    run_workers(_oib_worker, ws, device="cuda", timeout=240)


def test_optimizer_in_backward_python_hook_matches_too():
    # the Python form of the bucket hook (MCCL_PYTHON_BUCKET_HOOK=1) stays available and equivalent
    run_workers(_oib_worker, 2, device="cuda", timeout=240, env={"MCCL_PYTHON_BUCKET_HOOK": "1"})
