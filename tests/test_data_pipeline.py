"""Input prefetcher and asynchronous loss reader used by the end-to-end training loops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_prefetcher_yields_every_batch_once_in_order(cuda_device):
    from mccl_b200.utils.data import DevicePrefetcher
    host = [(torch.full((64, 8), float(i)).pin_memory(), torch.full((64,), i, dtype=torch.int64).pin_memory())
            for i in range(7)]
    feed = DevicePrefetcher(iter(host), cuda_device)
    seen = []
    for x, y in feed:
        assert x.device == cuda_device and y.device == cuda_device
        # a kernel on the compute stream right after next(): the copy must be complete for it
        seen.append((float((x * 2).sum()) / (2 * 64 * 8), int(y[0])))
    assert seen == [(float(i), i) for i in range(7)]
    with pytest.raises(StopIteration):
        feed.next()


def test_async_scalar_reader_returns_values_in_push_order(cuda_device):
    from mccl_b200.utils.data import AsyncScalarReader
    r = AsyncScalarReader(cuda_device, depth=3)
    vals = [torch.tensor(float(i) + 0.5, device=cuda_device) for i in range(6)]
    out = []
    for i, v in enumerate(vals):
        r.push(v * 2)
        if i > 0:
            out.append(r.pop())
    out += r.drain()
    assert out == [2 * (i + 0.5) for i in range(6)]
    assert len(r) == 0
    with pytest.raises(RuntimeError):
        r.pop()
    for v in vals[:3]:
        r.push(v)
    with pytest.raises(RuntimeError):
        r.push(vals[3])
