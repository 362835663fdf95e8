"""CPU ranks under a matrix of runtime knobs, and multi-bucket DDP with a conv model.

The same collectives and a small DDP training loop must give the same results whatever the
transport / engine knobs are: CRC on, tiny frames, one collective at a time, overlap off, a
small-message threshold that forces every algorithm branch.  World size 3 keeps an odd rank
count in the matrix (uneven chunking) at little cost; one combination runs with 5 ranks.
Follows the reference's tests/test_ws5_env_matrix.py, tests/test_ddp_multibucket.py and
tests/test_ddp_conv_overlap.py in spirit (CPU tensors here; the CUDA data plane has no such knobs).
"""
import pytest

from mccl_b200.utils.spawn import run_workers

ENVS = [
    {},
    {"MCCL_TRANSPORT_CRC": "1", "MCCL_CHUNK_BYTES": "4096"},
    {"MCCL_COLLECTIVE_CONCURRENCY": "1", "MCCL_OVERLAP_COMM": "0"},
    {"MCCL_SMALL_MSG_THRESHOLD": "64", "MCCL_MAX_QUEUE_DEPTH": "4"},
    {"MCCL_SMALL_MSG_THRESHOLD": "16777216"},
]


def _matrix_worker(rank, ws):
    import torch, torch.distributed as dist
    for n in (1, 7, 1000, 65537):
        t = torch.arange(n, dtype=torch.float32) * (rank + 1)
        dist.all_reduce(t)
        assert torch.equal(t, torch.arange(n, dtype=torch.float32) * sum(range(1, ws + 1))), n
        b = torch.full((n,), float(rank)) if rank == ws - 1 else torch.zeros(n)
        dist.broadcast(b, ws - 1)
        assert b[0].item() == ws - 1
        outs = [torch.empty(n) for _ in range(ws)]
        dist.all_gather(outs, torch.full((n,), float(rank)))
        assert [o[-1].item() for o in outs] == [float(r) for r in range(ws)]
        rs = torch.empty(n)
        dist.reduce_scatter(rs, [torch.full((n,), float(rank + i)) for i in range(ws)])
        assert rs[0].item() == sum(r + rank for r in range(ws))
    works = [dist.all_reduce(torch.ones(257) * i, async_op=True) for i in range(12)]
    for w in works:
        w.wait()
    objs = [None] * ws
    dist.all_gather_object(objs, {"rank": rank})
    assert [o["rank"] for o in objs] == list(range(ws))
    dist.barrier()
    assert mccl.get_metrics().total_errors == 0


@pytest.mark.parametrize("env", ENVS, ids=lambda e: ",".join(f"{k[5:].lower()}={v}" for k, v in e.items()) or "defaults")
def test_collectives_under_env_matrix(env):
    run_workers(_matrix_worker, 3, timeout=180, env=env)


def test_collectives_five_ranks_crc_small_frames():
    run_workers(_matrix_worker, 5, timeout=240, env={"MCCL_TRANSPORT_CRC": "1", "MCCL_CHUNK_BYTES": "65536"})


def _conv_multibucket(rank, ws):
    import torch, torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    def make():
        torch.manual_seed(3)
        return torch.nn.Sequential(
            torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.ReLU(), torch.nn.Conv2d(8, 16, 3, padding=1), torch.nn.ReLU(),
            torch.nn.AdaptiveAvgPool2d(4), torch.nn.Flatten(), torch.nn.Linear(256, 64), torch.nn.ReLU(),
            torch.nn.Linear(64, 10))
    # ~1 KB buckets: every layer gets its own allreduce, several are in flight during backward
    ddp = DDP(make(), bucket_cap_mb=0.001)
    ref = make()
    opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(11)
    for step in range(4):
        xs = torch.randn(4 * ws, 3, 8, 8, generator=g)
        ys = torch.randint(0, 10, (4 * ws,), generator=g)
        opt.zero_grad()
        torch.nn.functional.cross_entropy(ddp(xs[rank * 4:(rank + 1) * 4]), ys[rank * 4:(rank + 1) * 4]).backward()
        opt.step()
        ref_opt.zero_grad()
        torch.nn.functional.cross_entropy(ref(xs), ys).backward()
        ref_opt.step()
    for p, q in zip(ddp.module.parameters(), ref.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=1e-5), (p - q).abs().max()
    flat = torch.cat([p.detach().reshape(-1) for p in ddp.module.parameters()])
    outs = [torch.empty_like(flat) for _ in range(ws)]
    dist.all_gather(outs, flat)
    assert all(torch.equal(o, outs[0]) for o in outs)
    m = mccl.get_metrics()
    assert m.total_ops >= 4 and m.total_errors == 0, (m.total_ops, m.total_errors)


@pytest.mark.parametrize("env", [{}, {"MCCL_COLLECTIVE_CONCURRENCY": "1"}], ids=["defaults", "serial"])
def test_conv_ddp_many_small_buckets_matches_single_process(env):
    run_workers(_conv_multibucket, 2, timeout=180, env=env)
