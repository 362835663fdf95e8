"""Single-GPU microbenchmarks of the native kernels with roofline fractions.

    python -m mccl_b200.bench.kernels --kernel adamw --elements 94000000
    python -m mccl_b200.bench.kernels --kernel all

Each kernel is timed with CUDA events after warm-up on inputs larger than the 126 MB L2 (or
with rotating buffers), and the achieved algorithmic bandwidth is reported against the
measured copy bandwidth in MEASURED_PEAKS.json (fallback 6650 GB/s).  The collective kernels
run through the single-device emulation (all ranks' arenas on one GPU), so their traffic is
HBM traffic; across real GPUs the same kernels are bounded by NVLink instead.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch


def peak_gbs() -> tuple[float, str]:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def timeit(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def bench_adamw(native, n, iters):
    sizes = [n // 10] * 10
    ps = [torch.randn(s, device="cuda") for s in sizes]
    gs = [torch.randn(s, device="cuda") for s in sizes]
    ms_ = [torch.zeros(s, device="cuda") for s in sizes]
    vs = [torch.zeros(s, device="cuda") for s in sizes]
    plan = native.AdamWPlan(ps, ms_, vs)
    step = [0]

    def run():
        step[0] += 1
        plan.step(gs, 1e-3, 0.9, 0.999, 1e-8, 0.01, step[0], 1.0)
    ms = timeit(run, iters)
    return ms, sum(sizes) * 28, "p,g,m,v read + p,m,v written (28 B per fp32 parameter)"


def bench_ew(native, n, iters):
    a = [torch.randn(n, device="cuda") for _ in range(2)]
    b = torch.randn(n, device="cuda")
    i = [0]

    def run():
        i[0] ^= 1
        native._ew_accumulate_chunk(a[i[0]], b)
    return timeit(run, iters), n * 12, "dst,src read + dst written (12 B per fp32 element)"


def bench_twoshot(native, n, iters, ws=4):
    grp = native.EmuGroup(ws, max(2 * n * 4 // ws * 2, 8 << 20))
    ts = [torch.randn(n, device="cuda") for _ in range(ws)]

    def run():
        grp.allreduce(ts, "sum", "twoshot", "none", 1.0, 16)
    ms = timeit(run, iters)
    # per rank: push reads N(ws-1)/ws + writes the same; reduce reads N + writes 2N/ws; pull reads and writes N(ws-1)/ws
    per_rank = n * 4 * (4 * (ws - 1) / ws + 1 + 2 / ws)
    return ms, per_rank * ws, f"emulated {ws} ranks on one GPU: all push/reduce/pull traffic is local HBM"


def bench_oneshot(native, n, iters, ws=4):
    n = min(n, 1 << 20)  # the one-shot kernel is the small-message variant
    grp = native.EmuGroup(ws, max(n * 4 * ws * 2, 8 << 20))
    ts = [torch.randn(n, device="cuda") for _ in range(ws)]

    def run():
        grp.allreduce(ts, "sum", "oneshot", "none", 1.0, 16)
    ms = timeit(run, iters)
    # per rank: reads N, writes (ws-1) N into the peers' slots, reads ws N back, writes N
    return ms, n * 4 * (1 + (ws - 1) + ws + 1) * ws, f"emulated {ws} ranks on one GPU (one-shot: push to every peer, reduce ws slots)"


def bench_allgather(native, n, iters, ws=4):
    per = n // ws
    grp = native.EmuGroup(ws, max(per * 4 * ws * 2, 8 << 20))
    ins = [torch.randn(per, device="cuda") for _ in range(ws)]
    outs = [torch.empty(per * ws, device="cuda") for _ in range(ws)]

    def run():
        grp.allgather(outs, ins, 16)
    ms = timeit(run, iters)
    # per rank: reads its block, stores it ws-1 times remotely + once locally, copies ws-1 blocks out (read + write)
    return ms, per * 4 * (1 + ws + 2 * (ws - 1)) * ws, f"emulated {ws} ranks on one GPU (push + per-tile flags + copy-out)"


def bench_broadcast(native, n, iters, ws=4):
    grp = native.EmuGroup(ws, max(n * 4 * 2, 8 << 20))
    ts = [torch.randn(n, device="cuda") for _ in range(ws)]

    def run():
        grp.broadcast(ts, 0, 16)
    ms = timeit(run, iters)
    # two hops: root reads N and stores N; each owner re-reads its slice, stores it ws-2 times and once to its tensor;
    # every non-root copies the other slices out (read + write)
    nr = ws - 1
    total = n * 4 * (2 + nr * (1.0 / nr) * (1 + (ws - 2) + 1) + nr * 2.0 * (nr - 1) / nr)
    return ms, total, f"emulated {ws} ranks on one GPU (two-hop push broadcast)"


def bench_reduce_scatter(native, n, iters, ws=4):
    per = n // ws
    grp = native.EmuGroup(ws, max(per * 4 * ws * 2 + 4096, 8 << 20))
    ins = [torch.randn(per * ws, device="cuda") for _ in range(ws)]
    outs = [torch.empty(per, device="cuda") for _ in range(ws)]

    def run():
        grp.reduce_scatter(outs, ins, "sum", 16, 0)
    ms = timeit(run, iters)
    # per rank: reads (ws-1) chunks and stores them remotely, then reads ws-1 slots + own chunk and writes one chunk
    return ms, per * 4 * (2 * (ws - 1) + ws + 1) * ws, f"emulated {ws} ranks on one GPU (push + rank-ordered reduction)"


def bench_topk_exchange(native, n, iters, ws=4):
    n = min(n, 16 << 20)
    grp = native.EmuGroup(ws, 32 << 20)
    gs = [torch.randn(n, device="cuda") for _ in range(ws)]
    rs = [torch.zeros(n, device="cuda") for _ in range(ws)]

    def run():
        grp.topk_allreduce(gs, rs, 0.01, 1.0 / ws, 16)
    ms = timeit(run, iters)
    k = max(1, int(n * 0.01))
    # select (20 B/elem) + pairs pushed to ws ranks + dense zero-fill and sparse adds
    return ms, (n * 20 + k * 8 * (1 + ws) + n * 4 + k * 8 * ws) * ws, f"emulated {ws} ranks: select + sparse exchange + scatter"


def bench_topk(native, n, iters):
    g = torch.randn(n, device="cuda")
    r = torch.zeros(n, device="cuda")

    def run():
        native._topk_select(g, r, 0.01)
    return timeit(run, iters), n * 20, "adjust + histogram (12 B) + collect (4 B) + ordered compaction (4 B) per element"


def bench_stft(native, n, iters, n_fft=2048):
    from mccl_b200.transforms import stft
    x = torch.randn(16, n // 16, device="cuda")
    w = torch.hann_window(n_fft, device="cuda")
    hop = n_fft // 4

    def run():
        stft(x, n_fft=n_fft, hop_length=hop, win_length=n_fft, window=w)
    frames = 1 + (n // 16) // hop
    return timeit(run, iters), 16 * frames * (n_fft * 4 + (n_fft // 2 + 1) * 8), "frame loads (L2-resident overlap) + spectrum written"


def stft_vs_torch(native, n, iters):
    """Forward and forward+backward of STFT / iSTFT against torch.stft / torch.istft (cuFFT), same box."""
    from mccl_b200.transforms import istft, stft
    rows = []
    for n_fft in (512, 2048, 4096):
        hop = n_fft // 4
        w = torch.hann_window(n_fft, device="cuda")
        x = torch.randn(16, n // 16, device="cuda", requires_grad=True)

        def ours_f():
            return stft(x, n_fft=n_fft, hop_length=hop, win_length=n_fft, window=w)

        def torch_f():
            return torch.stft(x, n_fft, hop_length=hop, win_length=n_fft, window=w, center=True, pad_mode="reflect",
                              return_complex=True)

        def fb(fn):
            def run():
                x.grad = None
                y = fn()
                torch.view_as_real(y).square().sum().backward()
            return run
        spec = ours_f().detach()

        def ours_i():
            return istft(spec, n_fft=n_fft, hop_length=hop, win_length=n_fft, window=w, length=n // 16)

        def torch_i():
            return torch.istft(spec, n_fft, hop_length=hop, win_length=n_fft, window=w, center=True, length=n // 16)
        with torch.no_grad():
            t = {"stft_fwd_ms": timeit(ours_f, iters), "torch_stft_fwd_ms": timeit(torch_f, iters),
                 "istft_fwd_ms": timeit(ours_i, iters), "torch_istft_fwd_ms": timeit(torch_i, iters)}
        t["stft_fwd_bwd_ms"] = timeit(fb(ours_f), iters)
        t["torch_stft_fwd_bwd_ms"] = timeit(fb(torch_f), iters)
        rows.append({"kernel": "stft_vs_torch", "n_fft": n_fft, "hop": hop, "batch": 16, "samples": n // 16,
                     **{k: round(v, 4) for k, v in t.items()}})
    return rows


BENCHES = {"adamw": bench_adamw, "ew": bench_ew, "twoshot": bench_twoshot, "oneshot": bench_oneshot,
           "allgather": bench_allgather, "broadcast": bench_broadcast, "reduce_scatter": bench_reduce_scatter,
           "topk": bench_topk, "topk_exchange": bench_topk_exchange, "stft": bench_stft}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all", choices=["all", "stft_vs_torch"] + list(BENCHES))
    ap.add_argument("--elements", type=int, default=64 << 20)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    import mccl_b200 as mccl
    native = mccl.require_native()
    torch.cuda.set_device(0)
    peak, src = peak_gbs()
    if args.kernel == "stft_vs_torch":
        for row in stft_vs_torch(native, args.elements, args.iters):
            print(json.dumps(row), flush=True)
        return
    for name in (BENCHES if args.kernel == "all" else [args.kernel]):
        ms, nbytes, what = BENCHES[name](native, args.elements, args.iters)
        gbs = nbytes / (ms * 1e-3) / 1e9
        print(json.dumps({"kernel": name, "elements": args.elements, "ms": round(ms, 4), "algorithmic_GBps": round(gbs, 1),
                          f"fraction_of_{src}_hbm": round(gbs / peak, 3), "peak_GBps": peak, "bytes_model": what}), flush=True)


if __name__ == "__main__":
    main()
