"""Collective bus-bandwidth sweep: mccl vs torch's NCCL backend on the same GPUs.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29520 \
        -m mccl_b200.bench.busbw --ops allreduce,reduce_scatter,allgather,broadcast \
        --dtypes fp32,bf16 --min-bytes 1024 --max-bytes 1073741824 --compare-nccl --out busbw.jsonl

Method (as in NCCL-tests and the reference's tests/bench_busbw.py:57-137):
``algbw = bytes / t`` and ``busbw = algbw * f`` with f = 2(n-1)/n for allreduce, (n-1)/n
for reduce_scatter/allgather (bytes = the full gathered size) and 1 for broadcast.
Timing: CUDA events around `iters` back-to-back calls after warm-up, max over ranks.
Buffers rotate through a pool larger than the 126 MB L2, so no iteration finds its input
in cache.

``--variants oneshot,twoshot,nvls`` adds one extra mccl process group per name with the kernel
variant pinned through ``MCCLOptions`` (the default group keeps the tuner's choice), so one run
shows every variant next to NCCL.  ``--tune FILE`` measures the crossovers for every op and both
element classes on this world size and writes the file ``MCCL_TUNE_FILE`` loads.  ``--overlap``
measures communication / compute overlap at a 25 MB bucket (reference tests/bench_busbw.py:69-137).
"""
from __future__ import annotations

import argparse
import datetime
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


def make_call(op, group, ws, rank, numel_total, dtype, dev, pool, mem_pool=None):
    """Returns (list of zero-arg callables, payload bytes); one callable per pooled buffer.

    ``mem_pool``: allocate the allreduce buffers from this ``torch.cuda.MemPool`` (multicast-bound
    memory: the in-place NVLS kernel then runs instead of the staged ones).
    """
    esz = torch.empty(0, dtype=dtype).element_size()
    calls = []
    if op == "allreduce":
        for _ in range(pool):
            src = torch.randn(numel_total, device=dev).to(dtype)
            if mem_pool is not None:
                with torch.cuda.use_mem_pool(mem_pool):
                    t = torch.empty_like(src)
                t.copy_(src)
            else:
                t = src
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
    for i in range(max(warmup, len(calls))):  # every buffer once: first use of a buffer may do one-time setup
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


def pinned_group(algo=None, gather=None, nvls=None):
    """An extra mccl process group whose kernel variant is pinned through ``MCCLOptions``."""
    from mccl_b200 import _C
    o = _C.MCCLOptions(datetime.timedelta(seconds=120))
    if algo is not None:
        o.algo = algo
    if gather is not None:
        o.gather = gather
    if nvls is not None:
        o.nvls = nvls
    return dist.new_group(backend="mccl", pg_options=o)


def has_nvls(group, dev):
    import mccl_b200 as mccl
    dist.all_reduce(torch.ones(8, device=dev), group=group)
    return mccl.get_backend(group=group, device=dev).data_plane().endswith("+nvls")


def pool_and_iters(nbytes, quick=False):
    pool = max(1, min(16, (2 * L2_BYTES) // max(nbytes, 1)))
    if nbytes >= L2_BYTES:
        pool = 2 if nbytes <= (256 << 20) else 1
    iters = 200 if nbytes <= (1 << 20) else 50 if nbytes <= (64 << 20) else 10
    if quick:
        iters = max(iters // 4, 5)
    return pool, iters


def oneshot_ceiling(sizes, t_all):
    """The largest size at which one-shot is not beaten by any other variant (0: never).

    A single noisy row below it must not move the threshold: one-shot's advantage only grows downwards.
    """
    best = 0
    for size in sizes:
        t = t_all[size]
        others = [v for k, v in t.items() if k != "oneshot"]
        if "oneshot" in t and others and t["oneshot"] <= min(others):
            best = size
    return best


def nvls_floor(sizes, t_all, above):
    """The smallest size > ``above`` from which NVLS beats two-shot in all rows but at most one (-1: never).

    One lost row inside a range that NVLS otherwise wins (a noisy measurement) does not push the floor
    above that range; two lost rows do.
    """
    cand = [s for s in sizes if s > above and "nvls" in t_all[s] and "twoshot" in t_all[s]]
    for i, s in enumerate(cand):
        rest = cand[i:]
        lost = sum(1 for r in rest if t_all[r]["nvls"] > t_all[r]["twoshot"])
        if t_all[s]["nvls"] <= t_all[s]["twoshot"] and lost <= (1 if len(rest) >= 4 else 0):
            return s
    return -1


def tune(path, rank, ws, dev, max_bytes):
    """Measures, for this world size, every choice the tuner table holds and writes a tuner file.

    allreduce (fp32 and bf16): one-shot, two-shot and, where the box has it, NVLS kernels pinned on
    three groups and timed from 16 KiB to ``max_bytes``; ``oneshot_max_bytes`` is the largest size
    up to which one-shot is never beaten, ``nvls_min_bytes`` the smallest size from which NVLS is
    never beaten by two-shot.  allgather / broadcast: plain peer stores vs ``multimem.st``.
    The two forms of the two-shot second half (peers pull / owners push) are timed at 32 and
    64 MiB.  Load the result with ``MCCL_TUNE_FILE`` on every rank.
    """
    groups = {"oneshot": pinned_group("oneshot", nvls="0"), "twoshot": pinned_group("twoshot", nvls="0")}
    nv = pinned_group("nvls", nvls="1")
    nvls = has_nvls(nv, dev)
    if nvls:
        groups["nvls"] = nv
    table, measured = {}, []
    sizes = []
    b = 16 << 10
    while b <= max_bytes:
        sizes.append(b)
        b *= 2
    for dname, key in (("fp32", ""), ("bf16", "_16bit")):
        dtype = DTYPES[dname]
        esz = 4 if dname == "fp32" else 2
        t_all = {}
        for g in groups.values():  # first use of a group pays its one-time setup: keep it out of the table
            calls, _ = make_call("allreduce", g, ws, rank, sizes[0] // esz, dtype, dev, 1)
            time_calls(calls, 5, 3, dev, None)
        for size in sizes:
            pool, iters = pool_and_iters(size, quick=True)
            t = {}
            for algo, g in groups.items():
                if algo == "oneshot" and size * ws > (128 << 20):
                    continue  # needs ws slots of the whole vector in one arena buffer
                calls, _ = make_call("allreduce", g, ws, rank, size // esz, dtype, dev, pool)
                t[algo] = time_calls(calls, iters, 3, dev, None)
                del calls
            t_all[size] = t
            row = {"op": "allreduce", "dtype": dname, "bytes": size, **{k + "_us": round(v * 1e3, 2) for k, v in t.items()}}
            measured.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
            torch.cuda.empty_cache()
        best_one = oneshot_ceiling(sizes, t_all)
        table[f"ws{ws}_oneshot_max_bytes{key}"] = best_one
        nvls_min = -1
        if nvls:
            nvls_min = nvls_floor(sizes, t_all, best_one)
            if nvls_min >= 0:
                nvls_min = max(nvls_min, best_one + 1)
        table[f"ws{ws}_nvls_min_bytes{key}"] = nvls_min
    if nvls:
        for op, field in (("allgather", "allgather_nvls_min_bytes"), ("broadcast", "broadcast_nvls_min_bytes")):
            t_all = {}
            for size in sizes:
                pool, iters = pool_and_iters(size, quick=True)
                t = {}
                for name, g in (("unicast", groups["twoshot"]), ("nvls", nv)):
                    calls, _ = make_call(op, g, ws, rank, size // 4, torch.float32, dev, pool)
                    t[name] = time_calls(calls, iters, 3, dev, None)
                    del calls
                t_all[size] = t
                row = {"op": op, "bytes": size, **{k + "_us": round(v * 1e3, 2) for k, v in t.items()}}
                measured.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
                torch.cuda.empty_cache()
            if op == "broadcast":
                # one sender: multimem.st can win at small sizes and lose at large ones, so the table
                # holds a floor and a ceiling (the smallest and the largest size at which it won)
                wins = [size for size in sizes if t_all[size]["nvls"] <= t_all[size]["unicast"]]
                table[f"ws{ws}_{field}"] = wins[0] if wins else -1
                table[f"ws{ws}_broadcast_nvls_max_bytes"] = -1 if (not wins or wins[-1] == sizes[-1]) else wins[-1]
                continue
            m = -1
            for size in reversed(sizes):
                if t_all[size]["nvls"] <= t_all[size]["unicast"]:
                    m = size // ws  # allgather's threshold is per-rank bytes
                else:
                    break
            table[f"ws{ws}_{field}"] = m
    gather_groups = {"pull": pinned_group("twoshot", "pull", "0"), "push": pinned_group("twoshot", "push", "0")}
    push_wins = 0
    for size in (32 << 20, 64 << 20):
        t = {}
        for mode, g in gather_groups.items():
            calls, _ = make_call("allreduce", g, ws, rank, size // 4, torch.float32, dev, pool=4)
            t[mode] = time_calls(calls, 20, 5, dev, None)
            del calls
        row = {"op": "allreduce-twoshot-gather", "bytes": size, "pull_us": round(t["pull"] * 1e3, 2), "push_us": round(t["push"] * 1e3, 2)}
        measured.append(row)
        push_wins += t["push"] < t["pull"]
        if rank == 0:
            print(json.dumps(row), flush=True)
    table[f"ws{ws}_push_gather"] = int(push_wins == 2)
    if rank == 0:
        with open(path, "w") as f:
            json.dump({**table, "measured": measured}, f, indent=1)
        print(f"wrote {path}: {json.dumps(table)}", flush=True)


def overlap(rank, ws, dev, bucket_bytes=25 << 20, iters=30):
    """Communication / compute overlap at one DDP-bucket size.

    Times `iters` allreduces alone, `iters` matmul chains alone and both together (async allreduce
    issued first, then the chain, then wait), on the device, max over ranks.  Efficiency is
    (serial - together) / (serial - max(comm, compute)): 1.0 = the shorter one is hidden completely.
    """
    t = torch.randn(bucket_bytes // 4, device=dev)
    a = torch.randn(4096, 4096, device=dev)

    def chain():
        b = a
        for _ in range(8):
            b = b @ a
        return b

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        v = torch.tensor([s.elapsed_time(e) / iters], dtype=torch.float64, device=dev)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v.item())

    def both():
        w = dist.all_reduce(t, async_op=True)
        chain()
        w.wait()

    comm = timed(lambda: dist.all_reduce(t))
    comp = timed(chain)
    tog = timed(both)
    serial, ideal = comm + comp, max(comm, comp)
    row = {"op": "overlap", "bucket_bytes": bucket_bytes, "n_gpus": ws, "comm_ms": round(comm, 4), "compute_ms": round(comp, 4),
           "together_ms": round(tog, 4), "overlap_efficiency": round((serial - tog) / max(serial - ideal, 1e-9), 3)}
    if rank == 0:
        print(json.dumps(row), flush=True)
    return row


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="allreduce")
    ap.add_argument("--dtypes", default="fp32")
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--compare-nccl", action="store_true")
    ap.add_argument("--variants", default="",
                    help="comma list of oneshot,twoshot,nvls (extra groups with the variant pinned) and pool "
                         "(allreduce buffers allocated in multicast-bound memory on the default group: in-place NVLS)")
    ap.add_argument("--out", default="")
    ap.add_argument("--quick", action="store_true", help="every other size, fewer iterations")
    ap.add_argument("--tune", default="", help="measure every tuner crossover on this world size and write a tuner file here")
    ap.add_argument("--tune-max-bytes", type=int, default=256 << 20)
    ap.add_argument("--overlap", action="store_true", help="also measure comm/compute overlap at a 25 MB bucket")
    args = ap.parse_args(argv)

    import mccl_b200 as mccl  # noqa: F401  (registers the backend)

    rank = int(os.environ.get("RANK", "0"))
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("mccl", rank=rank, world_size=ws, device_id=dev)
    if args.tune:
        tune(args.tune, rank, ws, dev, args.tune_max_bytes)
        dist.destroy_process_group()
        return 0
    groups = {"mccl": None}
    mem_pool = None
    for v in [x for x in args.variants.split(",") if x]:
        if v == "pool":
            from mccl_b200.parallel import nvls_tensor_pool
            mem_pool = nvls_tensor_pool(min(3 << 30, 2 * args.max_bytes + (256 << 20)), device=dev)
            if mem_pool is None and rank == 0:
                print(json.dumps({"note": "no NVLS on this box: pool variant skipped"}), flush=True)
            if mem_pool is not None:
                groups["mccl-pool"] = None
            continue
        g = pinned_group(v, nvls="1" if v == "nvls" else "0")
        if v == "nvls" and not has_nvls(g, dev):
            if rank == 0:
                print(json.dumps({"note": "no NVLS on this box: variant skipped"}), flush=True)
            continue
        groups["mccl-" + v] = g
    if args.compare_nccl:
        groups["nccl"] = dist.new_group(backend="nccl")
    sizes = []
    b = args.min_bytes
    while b <= args.max_bytes:
        sizes.append(b)
        b *= 4 if args.quick else 2
    rows = []
    if rank == 0:
        print(json.dumps({"data_plane": mccl.get_backend(device=dev).data_plane() if ws > 1 else "local", "n_gpus": ws}), flush=True)
    for op in [o for o in args.ops.split(",") if o]:
        for dname in args.dtypes.split(","):
            dtype = DTYPES[dname]
            esz = torch.empty(0, dtype=dtype).element_size()
            for nbytes_req in sizes:
                numel = max(nbytes_req // esz, 1)
                pool, iters = pool_and_iters(nbytes_req, args.quick)
                for gname, group in groups.items():
                    if gname == "mccl-oneshot" and (op != "allreduce" or nbytes_req * ws > (128 << 20)):
                        continue
                    if gname == "mccl-twoshot" and op == "reduce_scatter":
                        continue  # reduce_scatter has one kernel: same as the default group
                    if gname == "mccl-pool" and op != "allreduce":
                        continue
                    calls, nbytes = make_call(op, group, ws, rank, numel, dtype, dev, pool,
                                              mem_pool if gname == "mccl-pool" else None)
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
    if args.overlap:
        rows.append(overlap(rank, ws, dev))
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
