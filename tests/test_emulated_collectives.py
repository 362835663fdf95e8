"""The fused NVLink collective kernels, run on ONE GPU.

``EmuGroup`` places the arenas of all ranks on a single device and launches each
collective once, cooperatively, with grid.y = ranks: the same kernel code that
runs across NVLink (peer stores, epoch flags, slot reuse, fixed-order reduction,
fused scale / wire cast) is exercised without needing several GPUs.  Oracles:
float64 analytic reduction, bitwise identity across ranks, and plain torch ops
(the styles of the reference's tests/test_correctness_vs_reference.py:129-150 and
tests/test_tree_collectives.py:42-57).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = [1, 3, 33, 1023, 4097, 70001, 262147]


def _inputs(ws, n, dtype, dev, seed=0):
    out = []
    for r in range(ws):
        g = torch.Generator().manual_seed(seed * 100 + r)
        if dtype.is_floating_point:
            t = torch.randn(n, generator=g).to(dtype)
        elif dtype == torch.bool:
            t = torch.rand(n, generator=g) > 0.3
        else:
            t = torch.randint(0 if dtype == torch.uint8 else -50, 3 if dtype == torch.uint8 else 50, (n,), generator=g).to(dtype)
        out.append(t.to(dev))
    return out


def _reference(xs, op):
    dtype = xs[0].dtype
    if dtype == torch.bool:
        acc = xs[0].clone()
        for x in xs[1:]:
            acc = (acc | x) if op in ("sum", "max") else (acc & x)
        return acc
    wide = torch.float64 if dtype.is_floating_point else torch.int64
    st = torch.stack([x.to(wide) for x in xs])
    if op in ("sum", "avg"):
        r = st.sum(0)
        if op == "avg":
            r = r / len(xs)
    elif op == "min":
        r = st.min(0).values
    elif op == "max":
        r = st.max(0).values
    else:
        r = st.prod(0)
    return r


def _tol(dtype):
    return {torch.float32: 1e-5, torch.float64: 1e-12, torch.float16: 2e-2, torch.bfloat16: 1e-1}[dtype]


@pytest.mark.parametrize("ws", [2, 4, 8])
@pytest.mark.parametrize("algo", ["oneshot", "twoshot"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_allreduce_sum_matches_f64_and_is_bitwise_identical(native, cuda_device, ws, algo, dtype):
    g = native.EmuGroup(ws, 16 << 20)
    for n in SIZES:
        xs = _inputs(ws, n, dtype, cuda_device, seed=n)
        want = _reference(xs, "sum")
        ts = [x.clone() for x in xs]
        g.allreduce(ts, "sum", algo)
        torch.cuda.synchronize()
        for r in range(1, ws):
            assert torch.equal(ts[0], ts[r]), f"rank {r} differs bitwise (n={n})"
        err = (ts[0].double() - want).abs().max().item()
        scale = max(1.0, want.abs().max().item())
        assert err <= _tol(dtype) * scale * ws, f"n={n} err={err}"


@pytest.mark.parametrize("ws", [2, 3, 5, 8])
@pytest.mark.parametrize("op", ["sum", "avg", "min", "max", "product"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.int32, torch.int64, torch.uint8, torch.bool, torch.float64])
def test_allreduce_ops_and_dtypes(native, cuda_device, ws, op, dtype):
    if dtype == torch.bool and op == "avg":
        pytest.skip("AVG is undefined for bool")
    g = native.EmuGroup(ws, 4 << 20)
    for algo in ("oneshot", "twoshot"):
        for n in (1, 13, 997, 20011):
            xs = _inputs(ws, n, dtype, cuda_device, seed=7)
            if op == "product" and dtype.is_floating_point:
                xs = [x.abs().clamp(0.5, 1.5) for x in xs]
            ts = [x.clone() for x in xs]
            g.allreduce(ts, op, algo)
            torch.cuda.synchronize()
            for r in range(1, ws):
                assert torch.equal(ts[0], ts[r])
            ref = _reference(xs, op)
            if dtype.is_floating_point:
                assert torch.allclose(ts[0].double(), ref, rtol=1e-5, atol=1e-5), (op, algo, n)
            elif dtype == torch.bool:
                assert torch.equal(ts[0], ref)
            elif op == "avg":
                # integer average = accumulate, then scale: i32 rounds, i64/u8 truncate
                s = _reference(xs, "sum")
                if dtype == torch.uint8:
                    s = s % 256
                    want = (s.float() * (1.0 / ws)).to(torch.uint8)
                elif dtype == torch.int32:
                    v = s.float() * torch.tensor(1.0 / ws, dtype=torch.float32)
                    want = (torch.sign(v) * torch.floor(v.abs() + 0.5)).to(torch.int32)  # roundf: halves away from zero
                else:
                    want = (s.double() * float(torch.tensor(1.0 / ws, dtype=torch.float32))).to(torch.int64)
                assert torch.equal(ts[0].cpu(), want.cpu().to(dtype)), (op, algo, n, dtype)
            else:
                want = ref % 256 if dtype == torch.uint8 else ref.to(dtype).to(torch.int64)  # wraps like the dtype
                assert torch.equal(ts[0].to(torch.int64), want), (op, algo, n, dtype)


@pytest.mark.parametrize("ws", [2, 8])
@pytest.mark.parametrize("wire", ["bf16", "fp16"])
def test_allreduce_wire_cast_is_consistent(native, cuda_device, ws, wire):
    g = native.EmuGroup(ws, 8 << 20)
    wdt = torch.bfloat16 if wire == "bf16" else torch.float16
    for algo in ("oneshot", "twoshot"):
        for n in (5, 4099, 100003):
            xs = _inputs(ws, n, torch.float32, cuda_device, seed=3)
            ts = [x.clone() for x in xs]
            g.allreduce(ts, "avg", algo, wire)
            torch.cuda.synchronize()
            for r in range(1, ws):
                assert torch.equal(ts[0], ts[r])
            # contributions are rounded to the wire dtype, summed in fp32 in rank order
            acc = xs[0].to(wdt).float()
            for x in xs[1:]:
                acc = acc + x.to(wdt).float()
            acc = acc * torch.tensor(1.0 / ws, dtype=torch.float32, device=cuda_device)
            if algo == "twoshot":
                acc = acc.to(wdt).float()  # the reduced chunk travels in the wire dtype too
            assert torch.equal(ts[0], acc), (algo, n)


@pytest.mark.parametrize("ws", [2, 4, 7])
def test_fused_scale(native, cuda_device, ws):
    g = native.EmuGroup(ws, 4 << 20)
    xs = _inputs(ws, 50001, torch.float32, cuda_device)
    for algo in ("oneshot", "twoshot"):
        ts = [x.clone() for x in xs]
        g.allreduce(ts, "sum", algo, "none", 0.125)
        acc = xs[0].clone()
        for x in xs[1:]:
            acc = acc + x
        assert torch.equal(ts[0], acc * 0.125)


@pytest.mark.parametrize("ws", [2, 3, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64])
def test_reduce_scatter(native, cuda_device, ws, dtype):
    g = native.EmuGroup(ws, 8 << 20)
    for n in (1, 7, 1001, 70001):
        ins = _inputs(ws, n * ws, dtype, cuda_device, seed=n)
        outs = [torch.empty(n, dtype=dtype, device=cuda_device) for _ in range(ws)]
        g.reduce_scatter(outs, ins, "sum")
        torch.cuda.synchronize()
        full = _reference(ins, "sum")
        for r in range(ws):
            want = full[r * n:(r + 1) * n]
            if dtype.is_floating_point:
                assert torch.allclose(outs[r].double(), want, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-1 if dtype == torch.bfloat16 else 1e-5)
            else:
                assert torch.equal(outs[r].to(torch.int64), want)


@pytest.mark.parametrize("ws", [2, 5, 8])
def test_allgather_distinct_values(native, cuda_device, ws):
    g = native.EmuGroup(ws, 8 << 20)
    for dtype, n in ((torch.int64, 1), (torch.int64, 513), (torch.float32, 70001), (torch.float16, 70001), (torch.uint8, 1_000_003)):
        ins = [(torch.arange(n, device=cuda_device) % 251 + r).to(dtype) for r in range(ws)]
        outs = [torch.empty(n * ws, dtype=dtype, device=cuda_device) for _ in range(ws)]
        g.allgather(outs, ins)
        torch.cuda.synchronize()
        want = torch.cat(ins)
        for r in range(ws):
            assert torch.equal(outs[r], want), (dtype, n, r)


@pytest.mark.parametrize("ws", [2, 4, 8])
def test_broadcast_every_root(native, cuda_device, ws):
    g = native.EmuGroup(ws, 16 << 20)
    for n in (1, 4096, 1_000_003, 3_000_001):
        for root in range(ws):
            ts = [torch.full((n,), float(r), device=cuda_device) for r in range(ws)]
            ts[root] = torch.arange(n, device=cuda_device, dtype=torch.float32) + root
            want = ts[root].clone()
            g.broadcast(ts, root)
            torch.cuda.synchronize()
            for r in range(ws):
                assert torch.equal(ts[r], want), (n, root, r)


def test_epoch_reuse_many_collectives(native, cuda_device):
    # Alternating sizes and variants through the same two parity buffers: stale
    # data from epoch e-2 must never be observed.
    ws = 4
    g = native.EmuGroup(ws, 8 << 20)
    for it in range(60):
        n = [17, 50000, 4097, 300000][it % 4]
        algo = "oneshot" if it % 3 else "twoshot"
        xs = [torch.full((n,), float(it + r), device=cuda_device) for r in range(ws)]
        g.allreduce(xs, "sum", algo)
        if it % 5 == 0:
            g.barrier()
    torch.cuda.synchronize()
    assert xs[0][0].item() == sum(59 + r for r in range(ws))


def test_bounded_wait_reports_instead_of_hanging(native, cuda_device):
    # One rank never shows up: the others' waits expire (0.2 s), the kernel
    # returns normally with a status the host can read, and the context is usable.
    ws = 4
    g = native.EmuGroup(ws, 1 << 20, 200_000)
    xs = [torch.ones(8, device=cuda_device) for _ in range(ws)]
    g.allreduce(xs, "sum", "oneshot")
    st = g.barrier_with_absent_rank(2)
    assert st[0] == 1, st            # ERR_WAIT_TIMEOUT
    assert st[3] == 2, st            # the rank that was waited for
    g.clear_status()
    y = torch.ones(4, device=cuda_device) * 2
    assert y.sum().item() == 8.0     # context still healthy
    xs = [torch.ones(8, device=cuda_device) for _ in range(ws)]
    g.allreduce(xs, "sum", "oneshot")
    torch.cuda.synchronize()
    assert xs[0][0].item() == ws


@pytest.mark.parametrize("ws", [2, 4, 8])
@pytest.mark.parametrize("tiles", [2, 3, 8])
def test_twoshot_tile_pipeline_matches_bulk(native, cuda_device, ws, tiles):
    # the software-pipelined form (push tile i, reduce i-1, pull i-2) must give the same bits as bulk phases
    g = native.EmuGroup(ws, 16 << 20)
    for n in (1000, 70001, 1_000_003):
        xs = _inputs(ws, n, torch.float32, cuda_device, seed=n)
        a = [x.clone() for x in xs]; b = [x.clone() for x in xs]
        g.allreduce(a, "sum", "twoshot", "none", 1.0, 4, 1)
        g.allreduce(b, "sum", "twoshot", "none", 1.0, 4, tiles)
        torch.cuda.synchronize()
        for r in range(ws):
            assert torch.equal(a[r], b[r]) and torch.equal(b[r], b[0])


@pytest.mark.parametrize("ws", [2, 3, 4, 8])
@pytest.mark.parametrize("tiles", [1, 3])
@pytest.mark.parametrize("dtype,wire", [(torch.float32, "none"), (torch.bfloat16, "none"), (torch.float32, "bf16")])
def test_twoshot_push_gather_matches_pull(native, cuda_device, ws, tiles, dtype, wire):
    # owners pushing the reduced chunks (second arena half + local copy) must give the same bits as
    # peers pulling them; repeated so that buffer reuse across epochs is covered
    g = native.EmuGroup(ws, 16 << 20)
    for n in (1, 1000, 70001, 1_000_003):
        for rep in range(3):
            xs = _inputs(ws, n, dtype, cuda_device, seed=n + rep)
            a = [x.clone() for x in xs]; b = [x.clone() for x in xs]
            g.allreduce(a, "avg", "twoshot", wire, 1.0, 4, tiles, False)
            g.allreduce(b, "avg", "twoshot", wire, 1.0, 4, tiles, True)
            torch.cuda.synchronize()
            for r in range(ws):
                assert torch.equal(a[r], b[r]) and torch.equal(b[r], b[0])


def test_twoshot_push_gather_needs_twice_the_arena(native, cuda_device):
    g = native.EmuGroup(2, 1 << 20)
    xs = _inputs(2, 200_000, torch.float32, cuda_device)  # 800 KB: fits once, not twice
    g.allreduce([x.clone() for x in xs], "sum", "twoshot", "none", 1.0, 4, 1, False)
    with pytest.raises(Exception, match="arena bytes"):
        g.allreduce(xs, "sum", "twoshot", "none", 1.0, 4, 1, True)
    torch.cuda.synchronize()


@pytest.mark.parametrize("ws", [2, 3, 8])
def test_reduce_scatter_reads_slices_in_place(native, cuda_device, ws):
    # a chunk pitch larger than the count: each launch reduces one slice of every chunk of a larger
    # input without packing it first (how inputs beyond one arena buffer are handled)
    g = native.EmuGroup(ws, 16 << 20)
    n, cnt = 5 * 256 + 77, 512          # per-rank chunk length, slice length
    ins = [torch.randn(ws * n, generator=torch.Generator().manual_seed(r)).to(cuda_device) for r in range(ws)]
    want = torch.stack([x.double() for x in ins]).sum(0)
    outs = [torch.zeros(n, device=cuda_device) for _ in range(ws)]
    for off in range(0, n, cnt):
        c = min(cnt, n - off)
        g.reduce_scatter([o[off:off + c] for o in outs], [x[off:] for x in ins], "sum", 4, n)
    torch.cuda.synchronize()
    for r in range(ws):
        assert torch.allclose(outs[r].double(), want[r * n:(r + 1) * n], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("ws", [2, 3, 8])
@pytest.mark.parametrize("tile_bytes", [0, 8192, 65536])
def test_allgather_tile_pipeline_and_slices(native, cuda_device, ws, tile_bytes):
    # push + per-tile flags + copy-out; small tiles force many pipeline iterations per CTA.
    # Also gathers a block in two slices that land at their final (strided) place.
    g = native.EmuGroup(ws, 16 << 20)
    for n in (1, 4099, 600_001):
        ins = [((torch.arange(n, device=cuda_device) * 7 + r * 13) % 255).to(torch.uint8) for r in range(ws)]
        want = torch.cat(ins)
        outs = [torch.zeros(n * ws, dtype=torch.uint8, device=cuda_device) for _ in range(ws)]
        g.allgather(outs, ins, 4, tile_bytes)
        torch.cuda.synchronize()
        for r in range(ws):
            assert torch.equal(outs[r], want), (n, r)
        if n > 1024:
            cut = (n // 2) // 256 * 256
            outs = [torch.zeros(n * ws, dtype=torch.uint8, device=cuda_device) for _ in range(ws)]
            g.allgather(outs, ins, 4, tile_bytes, n, cut, 0)
            g.allgather(outs, ins, 4, tile_bytes, n, n - cut, cut)
            torch.cuda.synchronize()
            for r in range(ws):
                assert torch.equal(outs[r], want), ("sliced", n, r)


@pytest.mark.parametrize("ws", [2, 5])
def test_allgather_in_place(native, cuda_device, ws):
    # torch's all_gather_into_tensor allows input == own slice of the output
    g = native.EmuGroup(ws, 8 << 20)
    n = 70001
    outs = [torch.zeros(n * ws, device=cuda_device) for _ in range(ws)]
    ins = []
    for r in range(ws):
        outs[r][r * n:(r + 1) * n] = torch.arange(n, device=cuda_device, dtype=torch.float32) + 1000 * r
        ins.append(outs[r][r * n:(r + 1) * n])
    want = torch.cat([i.clone() for i in ins])
    g.allgather(outs, ins)
    torch.cuda.synchronize()
    for r in range(ws):
        assert torch.equal(outs[r], want)


@pytest.mark.parametrize("ws", [3, 4, 8])
@pytest.mark.parametrize("tile_bytes", [8192, 0])
def test_broadcast_two_hop_tiles_and_odd_sizes(native, cuda_device, ws, tile_bytes):
    # above 256 KiB the root sends each slice to one owner, which forwards it; every size here has a
    # ragged last slice, and small tiles make every CTA run several pipeline iterations
    g = native.EmuGroup(ws, 16 << 20)
    for nbytes in (262_145, 1_000_003, 4_194_304 + 16):
        for root in (0, ws - 1, 1):
            ts = [torch.full((nbytes,), r + 1, dtype=torch.uint8, device=cuda_device) for r in range(ws)]
            ts[root] = ((torch.arange(nbytes, device=cuda_device) * 31 + root) % 251).to(torch.uint8)
            want = ts[root].clone()
            g.broadcast(ts, root, 4, tile_bytes)
            torch.cuda.synchronize()
            for r in range(ws):
                assert torch.equal(ts[r], want), (nbytes, root, r)


def test_broadcast_unaligned_views(native, cuda_device):
    # tensors that start at odd byte offsets take the guarded (element-wise) load/store path
    ws = 4
    g = native.EmuGroup(ws, 8 << 20)
    for n in (5, 70001, 400_003):
        base = [torch.zeros(n + 3, dtype=torch.uint8, device=cuda_device) for _ in range(ws)]
        ts = [b[1 + (r % 2):1 + (r % 2) + n] for r, b in enumerate(base)]
        ts[2].copy_((torch.arange(n, device=cuda_device) % 199).to(torch.uint8))
        want = ts[2].clone()
        g.broadcast(ts, 2)
        torch.cuda.synchronize()
        for r in range(ws):
            assert torch.equal(ts[r], want)
            assert base[r][0].item() == 0 and base[r][-1].item() == 0  # nothing written outside the view


def test_poisoned_buffers_between_epochs(native, cuda_device):
    # All data buffers are filled with 0xFF (NaNs) before every collective: a kernel that consumed a
    # slot nobody wrote in the current epoch would produce NaNs or wrong bytes.
    ws = 4
    g = native.EmuGroup(ws, 8 << 20)
    for it in range(24):
        g.poison_buffers(0xFF)
        n = [17, 50_000, 4097, 300_000][it % 4]
        xs = [torch.full((n,), float(it + r), device=cuda_device) for r in range(ws)]
        g.allreduce(xs, "sum", "oneshot" if it % 3 else "twoshot", "none", 1.0, 0, 1, it % 2 == 1)
        want = float(sum(it + r for r in range(ws)))
        torch.cuda.synchronize()
        for r in range(ws):
            assert torch.all(xs[r] == want), (it, r)
        g.poison_buffers(0xFF)
        ins = [torch.full((n,), float(r + it), device=cuda_device) for r in range(ws)]
        outs = [torch.empty(n * ws, device=cuda_device) for _ in range(ws)]
        g.allgather(outs, ins)
        g.poison_buffers(0xFF)
        ts = [torch.full((n,), float(r), device=cuda_device) for r in range(ws)]
        g.broadcast(ts, it % ws)
        rs_in = [torch.full((n * ws,), float(r + 1), device=cuda_device) for r in range(ws)]
        rs_out = [torch.empty(n, device=cuda_device) for _ in range(ws)]
        g.poison_buffers(0xFF)
        g.reduce_scatter(rs_out, rs_in, "sum")
        torch.cuda.synchronize()
        for r in range(ws):
            assert torch.equal(outs[r], torch.cat(ins)) and torch.all(ts[r] == float(it % ws))
            assert torch.all(rs_out[r] == float(sum(range(1, ws + 1))))


def test_debug_checks_pass_on_the_small_case_matrix_and_catch_a_short_buffer(native, cuda_device):
    # MCCL_DEBUG_CHECKS: kernels verify the ranges they are about to use.  The whole small-case
    # matrix must run clean under it; a buffer that is claimed to be smaller than the payload needs
    # is reported as ERR_BOUNDS (code 2) without any access outside it.
    ws = 4
    g = native.EmuGroup(ws, 4 << 20, 500_000)
    g.set_debug_checks(True)
    for n in (1, 33, 4097, 70001):
        for algo in ("oneshot", "twoshot"):
            xs = _inputs(ws, n, torch.float32, cuda_device, seed=n)
            want = _reference(xs, "sum")
            g.allreduce(xs, "sum", algo)
            torch.cuda.synchronize()
            assert torch.allclose(xs[0].double(), want, rtol=1e-5, atol=1e-5)
        ins = _inputs(ws, n, torch.float32, cuda_device, seed=1)
        outs = [torch.empty(n * ws, device=cuda_device) for _ in range(ws)]
        g.allgather(outs, ins)
        ts = [torch.full((n,), float(r), device=cuda_device) for r in range(ws)]
        g.broadcast(ts, 1)
        torch.cuda.synchronize()
        assert torch.equal(outs[2], torch.cat(ins)) and torch.all(ts[3] == 1.0)
    assert g.status(0)[0] == 0
    g.set_claimed_capacity(1024)          # the kernels are told the buffer holds 1 KiB
    ins = _inputs(ws, 4096, torch.float32, cuda_device, seed=2)
    outs = [torch.full((4096 * ws,), -1.0, device=cuda_device) for _ in range(ws)]
    g.allgather(outs, ins)
    torch.cuda.synchronize()
    st = g.status(0)
    assert st[0] == 2 and st[2] == 10, st  # ERR_BOUNDS at the allgather's range check
    assert torch.all(outs[0] == -1.0)      # nothing was written
    g.clear_status()
    g.set_claimed_capacity(0)
    g.allgather(outs, ins)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], torch.cat(ins))
