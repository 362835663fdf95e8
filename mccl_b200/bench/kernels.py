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


def bench_topk(native, n, iters):
    g = torch.randn(n, device="cuda")
    r = torch.zeros(n, device="cuda")

    def run():
        native._topk_select(g, r, 0.01)
    return timeit(run, iters), n * 28, "adjust (12 B) + 2 histogram passes + count + compact (4 B each) per element"


def bench_stft(native, n, iters):
    from mccl_b200.transforms import stft
    x = torch.randn(16, n // 16, device="cuda")
    w = torch.hann_window(2048, device="cuda")

    def run():
        stft(x, n_fft=2048, hop_length=512, win_length=2048, window=w)
    frames = 1 + (n // 16) // 512
    return timeit(run, iters), 16 * frames * (2048 * 4 + 1025 * 8), "frame loads (L2-resident overlap) + spectrum written"


BENCHES = {"adamw": bench_adamw, "ew": bench_ew, "twoshot": bench_twoshot, "topk": bench_topk, "stft": bench_stft}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all", choices=["all"] + list(BENCHES))
    ap.add_argument("--elements", type=int, default=64 << 20)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    import mccl_b200 as mccl
    native = mccl.require_native()
    torch.cuda.set_device(0)
    peak, src = peak_gbs()
    for name in (BENCHES if args.kernel == "all" else [args.kernel]):
        ms, nbytes, what = BENCHES[name](native, args.elements, args.iters)
        gbs = nbytes / (ms * 1e-3) / 1e9
        print(json.dumps({"kernel": name, "elements": args.elements, "ms": round(ms, 4), "algorithmic_GBps": round(gbs, 1),
                          f"fraction_of_{src}_hbm": round(gbs / peak, 3), "peak_GBps": peak, "bytes_model": what}), flush=True)


if __name__ == "__main__":
    main()
