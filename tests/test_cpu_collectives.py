"""CPU-tensor collectives over the host transport: local multi-process runs on 127.0.0.1.

Oracles: float64 analytic reduction, bitwise identity across ranks and against gloo
(the styles of the reference's tests/test_process_group_local.py:706-731 and
tests/test_correctness_vs_reference.py:129-150).
"""
import pytest

from mccl_b200.utils.spawn import run_workers


def _allreduce_matrix(rank, ws):
    import torch, torch.distributed as dist
    ops = [dist.ReduceOp.SUM, dist.ReduceOp.AVG, dist.ReduceOp.MIN, dist.ReduceOp.MAX, dist.ReduceOp.PRODUCT]
    for dtype in (torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.uint8):
        for n in (1, 3, 7, 33, 1023, 4097, 70001, 262147):
            for op in ops:
                g = torch.Generator().manual_seed(n)
                base = torch.rand(n, generator=g) + 0.5
                if not dtype.is_floating_point:
                    base = (base * 3).floor()
                xs = [(base * (r + 1) if op != dist.ReduceOp.PRODUCT else base.clamp(0.9, 1.1)).to(dtype) for r in range(ws)]
                if dtype == torch.uint8 or (not dtype.is_floating_point and op == dist.ReduceOp.PRODUCT):
                    xs = [(base % 2 + 1).to(dtype) for _ in range(ws)]
                t = xs[rank].clone()
                dist.all_reduce(t, op=op)
                st = torch.stack([x.double() for x in xs])
                want = {dist.ReduceOp.SUM: st.sum(0), dist.ReduceOp.AVG: st.sum(0) / ws, dist.ReduceOp.MIN: st.min(0).values,
                        dist.ReduceOp.MAX: st.max(0).values, dist.ReduceOp.PRODUCT: st.prod(0)}[op]
                if dtype.is_floating_point:
                    tol = {torch.float32: 1e-5, torch.float64: 1e-12, torch.float16: 5e-3, torch.bfloat16: 4e-2}[dtype]
                    assert torch.allclose(t.double(), want, rtol=tol * ws, atol=tol), (dtype, n, op)
                elif op == dist.ReduceOp.AVG:
                    s = st.sum(0)
                    if dtype == torch.int32:
                        v = s.float() * torch.tensor(1.0 / ws, dtype=torch.float32)
                        w = (torch.sign(v) * torch.floor(v.abs() + 0.5)).to(dtype)
                    elif dtype == torch.int64:
                        w = (s * (1.0 / ws)).to(dtype)
                    else:
                        w = ((s % 256).float() * torch.tensor(1.0 / ws, dtype=torch.float32)).to(dtype)
                    assert torch.equal(t, w), (dtype, n, op, t[:4], w[:4])
                else:
                    assert torch.equal(t.double(), want % 256 if dtype == torch.uint8 else want), (dtype, n, op)
    # bool: SUM/MAX = or, PRODUCT/MIN = and
    b = torch.tensor([rank == 0, True, False, rank == ws - 1])
    t = b.clone(); dist.all_reduce(t, op=dist.ReduceOp.SUM); assert t.tolist() == [True, True, False, True]
    t = b.clone(); dist.all_reduce(t, op=dist.ReduceOp.PRODUCT); assert t.tolist() == [False, True, False, False]


@pytest.mark.parametrize("ws", [2, 3, 4])
def test_allreduce_dtypes_ops_sizes(ws):
    run_workers(_allreduce_matrix, ws, timeout=240)


def _bitwise_vs_gloo(rank, ws):
    import torch, torch.distributed as dist
    gloo = dist.new_group(backend="gloo")
    for n in (5, 1000, 300001):
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(n, generator=g)
        a, b = x.clone(), x.clone()
        dist.all_reduce(a)
        dist.all_reduce(b, group=gloo)
        # identical on every rank, and within rounding of gloo's (different summation order)
        outs = [torch.empty_like(a) for _ in range(ws)]
        dist.all_gather(outs, a)
        for o in outs:
            assert torch.equal(o, outs[0]), "ranks disagree bitwise"
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-5)
    # determinism: same inputs, same bits, run after run
    x = torch.randn(70001, generator=torch.Generator().manual_seed(rank))
    first = x.clone(); dist.all_reduce(first)
    for _ in range(3):
        again = x.clone(); dist.all_reduce(again)
        assert torch.equal(first, again)


@pytest.mark.parametrize("ws", [2, 4])
def test_bitwise_identity_and_gloo_parity(ws):
    run_workers(_bitwise_vs_gloo, ws, timeout=180)


def _other_collectives(rank, ws):
    import torch, torch.distributed as dist
    # broadcast from every root, small (star) and large (scatter + allgather)
    for root in range(ws):
        for n in (1, 4096, 1000003):
            t = torch.arange(n, dtype=torch.float32) + root if rank == root else torch.zeros(n)
            dist.broadcast(t, root)
            assert t[0].item() == root and t[n - 1].item() == n - 1 + root
    u8 = torch.full((512 * 1024,), rank, dtype=torch.uint8)
    dist.broadcast(u8, ws - 1)
    assert int(u8[12345]) == ws - 1
    # allgather: distinct int64 values, f16 payloads
    outs = [torch.zeros(3, dtype=torch.int64) for _ in range(ws)]
    dist.all_gather(outs, torch.tensor([rank, rank * 10, rank * 100]))
    assert [o.tolist() for o in outs] == [[r, r * 10, r * 100] for r in range(ws)]
    outs = [torch.zeros(70001, dtype=torch.float16) for _ in range(ws)]
    dist.all_gather(outs, torch.full((70001,), float(rank), dtype=torch.float16))
    assert all(float(outs[r][-1]) == r for r in range(ws))
    big = torch.empty(ws * 5); dist.all_gather_into_tensor(big, torch.full((5,), float(rank)))
    assert big.view(ws, 5)[:, 0].tolist() == [float(r) for r in range(ws)]
    # reduce_scatter
    ins = [torch.full((1001,), float(rank + i)) for i in range(ws)]
    out = torch.empty(1001)
    dist.reduce_scatter(out, ins)
    assert out[0].item() == sum(r + rank for r in range(ws))
    flat = torch.arange(ws * 7, dtype=torch.float32); o = torch.empty(7)
    dist.reduce_scatter_tensor(o, flat, op=dist.ReduceOp.AVG)
    assert torch.allclose(o, flat[rank * 7:(rank + 1) * 7])
    # reduce to a root
    t = torch.full((100,), float(rank + 1)); dist.reduce(t, dst=0)
    if rank == 0:
        assert t[0].item() == sum(range(1, ws + 1))
    # coalesced
    ts = [torch.full((n,), float(rank)) for n in (3, 50, 7)]
    dist.all_reduce_coalesced(ts)
    assert all(t[0].item() == sum(range(ws)) for t in ts)
    # send / recv with tags, bidirectional, during an in-flight collective
    peer = (rank + 1) % ws
    prev = (rank - 1) % ws
    w_ar = dist.all_reduce(torch.ones(2_000_000), async_op=True)
    s = dist.isend(torch.full((1000,), float(rank)), peer, tag=7)
    r = torch.empty(1000); dist.recv(r, prev, tag=7)
    s.wait(); w_ar.wait()
    assert r[0].item() == prev
    z = torch.empty(0); dist.all_reduce(z)  # zero-size: no-op
    dist.barrier()
    # repeated barrier with skew
    import time
    for i in range(5):
        if rank == i % ws:
            time.sleep(0.05)
        dist.barrier()
    # object collectives (pickle over uint8 broadcast / allgather)
    objs = [{"a": 1, "r": rank}] if rank == 0 else [None]
    dist.broadcast_object_list(objs, src=0)
    assert objs[0] == {"a": 1, "r": 0}


@pytest.mark.parametrize("ws", [2, 3, 5])
def test_broadcast_allgather_reduce_scatter_p2p_barrier(ws):
    run_workers(_other_collectives, ws, timeout=240)


def _edge_cases(rank, ws):
    import torch, torch.distributed as dist
    # rejected calls leave the group usable
    bad = torch.zeros(4, dtype=torch.int8)
    try:
        dist.all_reduce(bad)
        raise SystemExit("int8 must be rejected")
    except RuntimeError as e:
        assert "unsupported dtype" in str(e)
    nc = torch.zeros(8, 8).t()
    try:
        dist.all_reduce(nc)
        raise SystemExit("non-contiguous must be rejected")
    except RuntimeError as e:
        assert "contiguous" in str(e)
    t = torch.ones(10); dist.all_reduce(t); assert t[0].item() == ws
    m = mccl.get_metrics()
    assert m.total_ops >= 1


def test_edge_cases_ws2():
    run_workers(_edge_cases, 2, timeout=120)


def _ws1(rank, ws):
    import torch, torch.distributed as dist
    t = torch.arange(5.0); dist.all_reduce(t); assert t.tolist() == [0, 1, 2, 3, 4]
    outs = [torch.zeros(5)]; dist.all_gather(outs, t); assert torch.equal(outs[0], t)
    dist.broadcast(t, 0); dist.barrier()
    assert mccl.get_backend(device="cpu").data_plane() == "local"


def test_world_size_one():
    run_workers(_ws1, 1, timeout=60)


def _crc_and_small_chunks(rank, ws):
    import torch, torch.distributed as dist
    x = torch.arange(300000, dtype=torch.float32) * (rank + 1)
    dist.all_reduce(x)
    assert x[-1].item() == 299999 * sum(range(1, ws + 1))
    b = torch.arange(100000.) if rank == 0 else torch.zeros(100000)
    dist.broadcast(b, 0); assert b[-1].item() == 99999


def test_crc_and_chunked_frames():
    # 64 KiB frames force multi-chunk messages; CRC on every frame
    run_workers(_crc_and_small_chunks, 3, timeout=120, env={"MCCL_CHUNK_BYTES": "65536", "MCCL_TRANSPORT_CRC": "1"})


def _pair_large(rank, ws):
    import torch, torch.distributed as dist
    # two ranks, >= 4 MiB: segmented exchange with the reduction overlapped (odd length: ragged last segment)
    n = 3_000_001
    g = torch.Generator().manual_seed(7 + rank)
    x = torch.randn(n, generator=g)
    both = [torch.empty_like(x) for _ in range(ws)]
    dist.all_gather(both, x)
    for op, want in ((dist.ReduceOp.SUM, both[0] + both[1]), (dist.ReduceOp.MAX, torch.maximum(both[0], both[1])),
                     (dist.ReduceOp.AVG, (both[0] + both[1]) * 0.5)):
        t = x.clone()
        dist.all_reduce(t, op=op)
        assert torch.equal(t, want), op
    i = torch.arange(n, dtype=torch.int64) * (rank + 1)
    dist.all_reduce(i)
    assert torch.equal(i, torch.arange(n, dtype=torch.int64) * 3)
    works = [dist.all_reduce(torch.full((1_500_000,), float(k)), async_op=True) for k in range(4)]
    for w in works:
        w.wait()
    assert mccl.get_metrics().total_errors == 0


@pytest.mark.parametrize("env", [{}, {"MCCL_CHUNK_BYTES": "65536", "MCCL_TRANSPORT_CRC": "1"}], ids=["defaults", "small-frames-crc"])
def test_two_rank_large_allreduce_segmented(env):
    run_workers(_pair_large, 2, timeout=240, env=env)


def _nan_and_signed_zero(rank, ws):
    import math
    import torch, torch.distributed as dist
    # Rank 0 and rank 1 reduce the same pair in opposite operand orders (each reduces its own buffer
    # in place); MIN / MAX must still give the same bits on both: NaNs propagate, -0 orders below +0.
    nan, inf = float("nan"), float("inf")
    a = [nan, 1.0, 0.0, -0.0, 2.0, -inf, nan]
    b = [1.0, nan, -0.0, 0.0, 2.0, 5.0, nan]
    for op, want in ((dist.ReduceOp.MIN, [nan, nan, -0.0, -0.0, 2.0, -inf, nan]),
                     (dist.ReduceOp.MAX, [nan, nan, 0.0, 0.0, 2.0, 5.0, nan])):
        for dtype in (torch.float32, torch.float64, torch.bfloat16):
            t = torch.tensor(a if rank == 0 else b, dtype=dtype)
            dist.all_reduce(t, op=op)
            outs = [torch.empty_like(t) for _ in range(ws)]
            dist.all_gather(outs, t)
            assert torch.equal(outs[0].view(torch.int16 if dtype == torch.bfloat16 else torch.int32 if dtype == torch.float32 else torch.int64),
                               outs[1].view(torch.int16 if dtype == torch.bfloat16 else torch.int32 if dtype == torch.float32 else torch.int64)), (op, dtype)
            for got, w in zip(t.double().tolist(), want):
                if math.isnan(w):
                    assert math.isnan(got), (op, dtype, got)
                else:
                    assert got == w and math.copysign(1.0, got) == math.copysign(1.0, w), (op, dtype, got, w)
    # large enough for the segmented two-rank path
    n = 3 * (1 << 20)
    t = torch.zeros(n)
    t[::2] = -0.0 if rank == 0 else 0.0
    t[1::2] = nan if rank == 1 else 3.0
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    assert math.copysign(1.0, t[0].item()) == -1.0 and math.isnan(t[1].item()) and math.isnan(t[-1].item())


def test_min_max_nan_and_signed_zero_agree_across_two_ranks():
    run_workers(_nan_and_signed_zero, 2, timeout=120)
