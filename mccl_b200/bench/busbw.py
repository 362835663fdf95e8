"""Collective bus-bandwidth sweep: mccl vs torch's NCCL backend on the same GPUs.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29520 \
        -m mccl_b200.bench.busbw --ops allreduce,reduce_scatter,allgather,broadcast \
        --dtypes fp32,bf16 --min-bytes 1024 --max-bytes 1073741824 --compare-nccl --out busbw.jsonl

Method (as in NCCL-tests and the reference's tests/bench_busbw.py:57-137):
``algbw = bytes / t`` and ``busbw = algbw * f`` with f = 2(n-1)/n for allreduce, (n-1)/n
for reduce_scatter/allgather (bytes = the full gathered size) and 1 for broadcast.
Timing: CUDA events around `iters` back-to-back calls after warm-up, max over ranks.
Buffers rotate through a pool larger than the 126 MB L2, so no iteration finds its input
in cache.  Run it with ``MCCL_ALGO=oneshot`` and ``MCCL_ALGO=twoshot`` to find the crossover
that goes into a tuner file, or let ``--tune FILE`` measure it (one-shot and two-shot pinned through
``MCCLOptions`` on two extra groups) and write the file for ``MCCL_TUNE_FILE``; ``MCCL_COMM_CTAS`` sizes the grid.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}
L2_BYTES = 126 << 20


def bus_factor(op: str, n: int) -> float:
    if op == "allreduce":
        return 2.0 * (n - 1) / n
    if op in ("reduce_scatter", "allgather"):
        return (n - 1) / n
    return 1.0


def make_call(op, group, ws, rank, numel_total, dtype, dev, pool):
    """Returns (list of zero-arg callables, payload bytes); one callable per pooled buffer."""
    esz = torch.empty(0, dtype=dtype).element_size()
    calls = []
    if op == "allreduce":
        for _ in range(pool):
            t = torch.randn(numel_total, device=dev).to(dtype)
            calls.append(lambda t=t: dist.all_reduce(t, group=group))
        nbytes = numel_total * esz
    elif op == "broadcast":
        for _ in range(pool):
            t = torch.randn(numel_total, device=dev).to(dtype)
            calls.append(lambda t=t: dist.broadcast(t, 0, group=group))
        nbytes = numel_total * esz
    elif op == "allgather":
        per = max(numel_total // ws, 1)
        for _ in range(pool):
            i = torch.randn(per, device=dev).to(dtype)
            o = torch.empty(per * ws, device=dev, dtype=dtype)
            calls.append(lambda i=i, o=o: dist.all_gather_into_tensor(o, i, group=group))
        nbytes = per * ws * esz
    elif op == "reduce_scatter":
        per = max(numel_total // ws, 1)
        for _ in range(pool):
            i = torch.randn(per * ws, device=dev).to(dtype)
            o = torch.empty(per, device=dev, dtype=dtype)
            calls.append(lambda i=i, o=o: dist.reduce_scatter_tensor(o, i, group=group))
        nbytes = per * ws * esz
    else:
        raise ValueError(op)
    return calls, nbytes


def time_calls(calls, iters, warmup, dev, sync_group):
    for i in range(warmup):
        calls[i % len(calls)]()
    torch.cuda.synchronize()
    dist.barrier(group=sync_group)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(iters):
        calls[i % len(calls)]()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / iters
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=sync_group)
    return float(t.item())


def tune(path, rank, ws, dev):
    """Finds the one-shot / two-shot crossover for this world size and writes a tuner file.

    Two extra process groups are created with the variant pinned through ``MCCLOptions``
    (``pg_options`` are honoured by the backend); fp32 allreduce is timed from 16 KiB to
    64 MiB and the largest size at which one-shot is at least as fast becomes
    ``ws<N>_oneshot_max_bytes``.  The two forms of the two-shot second half (peers pull the
    reduced chunks / owners push them) are then timed at 32 and 64 MiB; ``ws<N>_push_gather``
    is 1 when pushing wins at both.  Load the result with ``MCCL_TUNE_FILE`` on every rank.
    """
    import datetime

    from mccl_b200 import _C
    groups = {}
    for algo in ("oneshot", "twoshot"):
        o = _C.MCCLOptions(datetime.timedelta(seconds=120))
        o.algo = algo
        groups[algo] = dist.new_group(backend="mccl", pg_options=o)
    best, rows, size = 0, [], 16 << 10
    while size <= (64 << 20):
        numel = size // 4
        t = {}
        for algo, g in groups.items():
            calls, _ = make_call("allreduce", g, ws, rank, numel, torch.float32, dev, pool=8)
            t[algo] = time_calls(calls, 40, 5, dev, None)
        rows.append({"bytes": size, "oneshot_us": round(t["oneshot"] * 1e3, 2), "twoshot_us": round(t["twoshot"] * 1e3, 2)})
        if t["oneshot"] <= t["twoshot"]:
            best = size
        if rank == 0:
            print(json.dumps(rows[-1]), flush=True)
        size *= 2
    gather_groups = {}
    for mode in ("pull", "push"):
        o = _C.MCCLOptions(datetime.timedelta(seconds=120))
        o.algo = "twoshot"
        o.gather = mode
        gather_groups[mode] = dist.new_group(backend="mccl", pg_options=o)
    push_wins, gather_rows = 0, []
    for size in (32 << 20, 64 << 20):
        t = {}
        for mode, g in gather_groups.items():
            calls, _ = make_call("allreduce", g, ws, rank, size // 4, torch.float32, dev, pool=4)
            t[mode] = time_calls(calls, 20, 5, dev, None)
        gather_rows.append({"bytes": size, "pull_us": round(t["pull"] * 1e3, 2), "push_us": round(t["push"] * 1e3, 2)})
        push_wins += t["push"] < t["pull"]
        if rank == 0:
            print(json.dumps(gather_rows[-1]), flush=True)
    push = int(push_wins == 2)
    if rank == 0:
        with open(path, "w") as f:
            json.dump({f"ws{ws}_oneshot_max_bytes": best, f"ws{ws}_push_gather": push, "measured": rows,
                       "measured_gather": gather_rows}, f, indent=1)
        print(f"wrote {path}: ws{ws}_oneshot_max_bytes = {best}, ws{ws}_push_gather = {push}", flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="allreduce")
    ap.add_argument("--dtypes", default="fp32")
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--compare-nccl", action="store_true")
    ap.add_argument("--out", default="")
    ap.add_argument("--quick", action="store_true", help="every other size, fewer iterations")
    ap.add_argument("--tune", default="", help="measure one-shot vs two-shot allreduce and write a tuner file here")
    args = ap.parse_args(argv)

    import mccl_b200 as mccl  # noqa: F401  (registers the backend)

    rank = int(os.environ.get("RANK", "0"))
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("mccl", rank=rank, world_size=ws, device_id=dev)
    if args.tune:
        tune(args.tune, rank, ws, dev)
        dist.destroy_process_group()
        return 0
    groups = {"mccl": None}
    if args.compare_nccl:
        groups["nccl"] = dist.new_group(backend="nccl")
    sizes = []
    b = args.min_bytes
    while b <= args.max_bytes:
        sizes.append(b)
        b *= 4 if args.quick else 2
    rows = []
    for op in args.ops.split(","):
        for dname in args.dtypes.split(","):
            dtype = DTYPES[dname]
            esz = torch.empty(0, dtype=dtype).element_size()
            for nbytes_req in sizes:
                numel = max(nbytes_req // esz, 1)
                pool = max(1, min(16, (2 * L2_BYTES) // max(nbytes_req, 1)))
                if nbytes_req >= L2_BYTES:
                    pool = 2 if nbytes_req <= (256 << 20) else 1
                iters = 200 if nbytes_req <= (1 << 20) else 50 if nbytes_req <= (64 << 20) else 10
                if args.quick:
                    iters = max(iters // 4, 5)
                for gname, group in groups.items():
                    calls, nbytes = make_call(op, group, ws, rank, numel, dtype, dev, pool)
                    ms = time_calls(calls, iters, max(3, iters // 10), dev, groups["mccl"])
                    algbw = nbytes / (ms * 1e-3) / 1e9
                    row = {"op": op, "dtype": dname, "bytes": nbytes, "backend": gname, "n_gpus": ws,
                           "us": round(ms * 1e3, 2), "algbw_gbs": round(algbw, 2),
                           "busbw_gbs": round(algbw * bus_factor(op, ws), 2), "iters": iters}
                    rows.append(row)
                    if rank == 0:
                        print(json.dumps(row), flush=True)
                    del calls
                torch.cuda.empty_cache()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
