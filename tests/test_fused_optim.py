"""Fused AdamW kernel vs torch.optim.AdamW, and per-bucket stepping inside backward (one GPU)."""
import pytest
import torch

from mccl_b200.utils.spawn import run_workers

pytestmark = pytest.mark.gpu


def test_fused_adamw_matches_torch(cuda_device):
    from mccl_b200.optim import FusedAdamW
    torch.manual_seed(0)
    shapes = [(1000, 333), (333,), (7,), (64, 64, 3), (100003,)]
    p1 = [torch.randn(s, device=cuda_device, requires_grad=True) for s in shapes]
    p2 = [p.detach().clone().requires_grad_(True) for p in p1]
    o1 = FusedAdamW(p1, lr=1e-2, weight_decay=0.05)
    o2 = torch.optim.AdamW(p2, lr=1e-2, weight_decay=0.05)
    for step in range(5):
        for a, b in zip(p1, p2):
            g = torch.randn_like(a)
            a.grad = g.clone(); b.grad = g.clone()
        o1.step(); o2.step()
    for a, b in zip(p1, p2):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6), (a - b).abs().max()
    # interchangeable state
    o2.load_state_dict(o1.state_dict())
    o1.load_state_dict(o2.state_dict())


def _oib_single(rank, ws):
    import torch
    from mccl_b200.parallel import wrap_ddp
    from mccl_b200.optim import FusedAdamW
    def make():
        torch.manual_seed(3)
        return torch.nn.Sequential(torch.nn.Linear(128, 512), torch.nn.GELU(), torch.nn.Linear(512, 8)).to(device)
    a, b = make(), make()
    oa, ob = FusedAdamW(a.parameters(), lr=1e-3), FusedAdamW(b.parameters(), lr=1e-3)
    da = wrap_ddp(a, device_ids=[device.index], bucket_cap_mb=1)
    db = wrap_ddp(b, device_ids=[device.index], bucket_cap_mb=1, optimizer_in_backward=ob)
    for i in range(4):
        x = torch.randn(8, 128, device=device); y = torch.randint(0, 8, (8,), device=device)
        for d, o in ((da, oa), (db, ob)):
            o.zero_grad(); torch.nn.functional.cross_entropy(d(x), y).backward(); o.step()
    for p, q in zip(a.parameters(), b.parameters()):
        assert torch.equal(p, q)


def test_optimizer_in_backward_world_size_one():
    run_workers(_oib_single, 1, device="cuda", timeout=180)
