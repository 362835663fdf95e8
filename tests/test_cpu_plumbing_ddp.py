"""CPU plumbing gate: DDP on CPU tensors, world size 2, gradients bit-identical across ranks.

Model Linear(512,256)-ReLU-Linear(256,10), seed 42, x ~ N(0,1) [8,512], y in [0,10),
CrossEntropyLoss, AdamW lr 1e-3, 10 steps; after every backward the gradients of both ranks
must be bit-identical, and parameters must match a single-process run on the union batch.
"""
from mccl_b200.utils.spawn import run_workers


def _plumbing(rank, ws):
    import torch, torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP
    torch.manual_seed(42)
    model = torch.nn.Sequential(torch.nn.Linear(512, 256), torch.nn.ReLU(), torch.nn.Linear(256, 10))
    ddp = DDP(model)
    opt = torch.optim.AdamW(ddp.parameters(), lr=1e-3)
    loss_fn = torch.nn.CrossEntropyLoss()
    g = torch.Generator().manual_seed(1000 + rank)
    losses = []
    for step in range(10):
        x = torch.randn(8, 512, generator=g)
        y = torch.randint(0, 10, (8,), generator=g)
        opt.zero_grad()
        loss = loss_fn(ddp(x), y)
        loss.backward()
        flat = torch.cat([p.grad.reshape(-1) for p in ddp.parameters()])
        both = [torch.empty_like(flat) for _ in range(ws)]
        dist.all_gather(both, flat)
        assert torch.equal(both[0], both[1]), f"step {step}: gradients differ across ranks"
        opt.step()
        losses.append(loss.item())
    params = torch.cat([p.detach().reshape(-1) for p in ddp.parameters()])
    both = [torch.empty_like(params) for _ in range(ws)]
    dist.all_gather(both, params)
    assert torch.equal(both[0], both[1])
    assert losses[-1] < losses[0] + 0.5
    m = mccl.get_metrics()
    assert m.total_ops > 0 and m.total_bytes_sent > 0


def test_cpu_ddp_gradients_bit_identical():
    run_workers(_plumbing, 2, timeout=120)


def _ddp_state_dict_roundtrip(rank, ws):
    import io, torch, torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    ddp = DDP(model)
    opt = torch.optim.AdamW(ddp.parameters(), lr=1e-2)
    for _ in range(3):
        opt.zero_grad(); ddp(torch.randn(4, 16)).sum().backward(); opt.step()
    # a checkpoint written under DDP+mccl is ordinary PyTorch: "module."-prefixed keys, plain tensors
    buf = io.BytesIO(); torch.save({"model": ddp.state_dict(), "opt": opt.state_dict()}, buf); buf.seek(0)
    ck = torch.load(buf)
    assert all(k.startswith("module.") for k in ck["model"])
    plain = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    plain.load_state_dict({k[len("module."):]: v for k, v in ck["model"].items()})
    for a, b in zip(plain.parameters(), ddp.module.parameters()):
        assert torch.equal(a, b)
    opt2 = torch.optim.AdamW(plain.parameters(), lr=1e-2); opt2.load_state_dict(ck["opt"])
    # and the other way round: a plain checkpoint loads into a DDP-wrapped model
    ddp.module.load_state_dict(plain.state_dict())
    dist.barrier()


def test_checkpoint_compatibility():
    run_workers(_ddp_state_dict_roundtrip, 2, timeout=120)
