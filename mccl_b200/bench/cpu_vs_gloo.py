"""CPU-tensor collectives: the mccl host path (framed TCP mesh + C++ reductions) vs gloo.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29570 \
        -m mccl_b200.bench.cpu_vs_gloo --ops allreduce,broadcast --min-bytes 1024 --max-bytes 67108864

GPU tensors never take this path (their data plane is NVLink peer memory); it serves CPU tensors,
object collectives and control traffic.  Timing is wall clock around back-to-back blocking calls after
warm-up, max over ranks.  One JSON line per (op, bytes, backend) on rank 0.  Counterpart of the
reference's tests/bench_mccl_vs_gloo.py:41-188, which compared its GPU path with gloo on CPU.
"""
import argparse
import json
import os
import time

import torch
import torch.distributed as dist


def _calls(op, group, ws, numel):
    if op == "allreduce":
        t = torch.randn(numel)
        return (lambda: dist.all_reduce(t, group=group)), numel * 4
    if op == "broadcast":
        t = torch.randn(numel)
        return (lambda: dist.broadcast(t, 0, group=group)), numel * 4
    if op == "allgather":
        per = max(numel // ws, 1)
        i, o = torch.randn(per), torch.empty(per * ws)
        return (lambda: dist.all_gather_into_tensor(o, i, group=group)), per * ws * 4
    if op == "reduce_scatter":
        per = max(numel // ws, 1)
        i, o = torch.randn(per * ws), torch.empty(per)
        return (lambda: dist.reduce_scatter_tensor(o, i, group=group)), per * ws * 4
    raise ValueError(op)


def _time(fn, iters, warmup, sync_group):
    for _ in range(warmup):
        fn()
    dist.barrier(group=sync_group)
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    dt = (time.perf_counter() - t0) / iters
    t = torch.tensor([dt], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=sync_group)
    return float(t.item())


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="allreduce")
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=64 << 20)
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)

    import mccl_b200  # noqa: F401  (registers the backend)

    rank = int(os.environ.get("RANK", "0"))
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    dist.init_process_group("mccl", rank=rank, world_size=ws)
    groups = {"mccl": None, "gloo": dist.new_group(backend="gloo")}
    rows = []
    for op in args.ops.split(","):
        nbytes = args.min_bytes
        while nbytes <= args.max_bytes:
            numel = max(nbytes // 4, 1)
            for name, g in groups.items():
                if op == "reduce_scatter" and name == "gloo":
                    continue  # gloo has no reduce_scatter
                fn, payload = _calls(op, g, ws, numel)
                iters = 200 if nbytes <= (64 << 10) else 40 if nbytes <= (4 << 20) else 8
                sec = _time(fn, iters, 3, None)
                row = {"op": op, "bytes": payload, "backend": name, "n_ranks": ws, "us": round(sec * 1e6, 1),
                       "algbw_gbs": round(payload / sec / 1e9, 3), "device": "cpu"}
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
            nbytes *= 4
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
