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


def _oib_groups_single(rank, ws):
    import torch
    from mccl_b200.parallel import wrap_ddp
    from mccl_b200.optim import FusedAdamW
    def make():
        torch.manual_seed(5)
        return torch.nn.Sequential(torch.nn.Linear(128, 512), torch.nn.GELU(), torch.nn.Linear(512, 8)).to(device)
    def groups(m):
        return [{"params": [p for p in m.parameters() if p.ndim > 1], "weight_decay": 0.2},
                {"params": [p for p in m.parameters() if p.ndim <= 1], "weight_decay": 0.0, "lr": 5e-3}]
    a, b = make(), make()
    oa, ob = torch.optim.AdamW(groups(a), lr=1e-3), FusedAdamW(groups(b), lr=1e-3)
    sa = torch.optim.lr_scheduler.StepLR(oa, step_size=1, gamma=0.7)
    sb = torch.optim.lr_scheduler.StepLR(ob, step_size=1, gamma=0.7)
    da = wrap_ddp(a, device_ids=[device.index], bucket_cap_mb=25)   # one bucket holding both groups
    db = wrap_ddp(b, device_ids=[device.index], bucket_cap_mb=25, optimizer_in_backward=ob)
    for i in range(5):
        x = torch.randn(8, 128, device=device); y = torch.randint(0, 8, (8,), device=device)
        for d, o, s in ((da, oa, sa), (db, ob, sb)):
            o.zero_grad(); torch.nn.functional.cross_entropy(d(x), y).backward(); o.step(); s.step()
    for p, q in zip(a.parameters(), b.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=2e-5), (p - q).abs().max()
    # a group added later is indexed too
    extra = torch.nn.Parameter(torch.zeros(16, device=device))
    ob.add_param_group({"params": [extra]})
    assert extra.data_ptr() in ob._by_ptr


@pytest.mark.parametrize("python_hook", ["0", "1"])
def test_bucket_spanning_two_param_groups_uses_each_groups_hyperparameters(python_hook):
    run_workers(_oib_groups_single, 1, device="cuda", timeout=180, env={"MCCL_PYTHON_BUCKET_HOOK": python_hook})
