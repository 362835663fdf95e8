#!/usr/bin/env python
"""DDP training on synthetic data: the reference's benchmark/"train()" entry, for B200.

    python examples/ddp_dummy_train.py --baseline --steps 100                    # one GPU, no DDP
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/ddp_dummy_train.py --backend mccl

Flags follow reference examples/ddp_dummy_train.py:45-70 (``--backend``, ``--baseline``,
``--steps``, ``--batch-size`` per rank, ``--bucket-mb``, ``--stress-model``, ``--fp16``,
``--save-stats``, ``--warmup``) plus ``--model`` (heavy | mlp | resnet50 | gpt2-medium | gpt2-tiny),
``--compression`` (none | fp16 | topk) and ``--fused-optim``.  AdamW lr 1e-4 wd 0.01 by
default; after the run the first weights are broadcast from rank 0 and compared on every
rank (replicas must be identical).
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="mccl", choices=["mccl", "nccl", "gloo"])
    ap.add_argument("--baseline", action="store_true", help="single process, no DDP")
    ap.add_argument("--model", default="heavy", choices=["heavy", "mlp", "resnet50", "gpt2-medium", "gpt2-tiny"])
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch-size", type=int, default=128, help="per rank")
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--depth", type=int, default=4)
    ap.add_argument("--bucket-mb", type=int, default=int(os.environ.get("DDP_BUCKET_MB", "25")))
    ap.add_argument("--stress-model", action="store_true", help="double the hidden size")
    ap.add_argument("--fp16", action="store_true", help="bf16 autocast for forward/backward")
    ap.add_argument("--compression", default=None, choices=[None, "none", "fp16", "topk"])
    ap.add_argument("--topk-ratio", type=float, default=0.01)
    ap.add_argument("--fused-optim", action="store_true", help="use the fused AdamW kernel")
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--save-stats", default="")
    ap.add_argument("--cpu", action="store_true", help="CPU tensors (host transport)")
    return ap.parse_args()


def build(args, device):
    from mccl_b200 import models
    hidden = args.hidden * (2 if args.stress_model else 1)
    if args.model == "heavy":
        return models.HeavyDummyModel(512, 10, hidden, args.depth).to(device), "vector"
    if args.model == "mlp":
        return models.MLP94M().to(device), "mlp"
    if args.model == "resnet50":
        return models.ResNet50().to(device), "image"
    if args.model == "gpt2-medium":
        return models.gpt2_medium().to(device), "tokens"
    return models.gpt2_tiny().to(device), "tokens-tiny"


def make_batch(kind, n, ds, device):
    if kind == "vector":
        return ds.batch(n, device)
    if kind == "mlp":
        return torch.randn(n, 2048, device=device), torch.randint(0, 1000, (n,), device=device)
    if kind == "image":
        return torch.randn(n, 3, 224, 224, device=device), torch.randint(0, 1000, (n,), device=device)
    vocab, seq = (50257, 1024) if kind == "tokens" else (1024, 64)
    ids = torch.randint(0, vocab, (n, seq + 1), device=device)
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = 1 if args.baseline else int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and not args.cpu
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    import mccl_b200 as mccl
    if args.compression:
        mccl.init(compression=args.compression, topk_ratio=args.topk_ratio)
    if not args.baseline:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(args.backend, rank=rank, world_size=world,
                                **({"device_id": device} if use_cuda else {}))
    torch.manual_seed(42)
    model, kind = build(args, device)
    n_params = sum(p.numel() for p in model.parameters())
    mccl.params.ensure_contiguous_parameters(model)
    if not args.baseline:
        if args.backend == "mccl":
            from mccl_b200.parallel import wrap_ddp
            model = wrap_ddp(model, device_ids=[local] if use_cuda else None, bucket_cap_mb=args.bucket_mb)
        else:
            from torch.nn.parallel import DistributedDataParallel
            model = DistributedDataParallel(model, device_ids=[local] if use_cuda else None,
                                            bucket_cap_mb=args.bucket_mb)
    if args.fused_optim and use_cuda:
        from mccl_b200.optim import FusedAdamW
        opt = FusedAdamW(model.parameters(), lr=args.lr, weight_decay=0.01)
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=args.lr, weight_decay=0.01)
    from mccl_b200.utils import SyntheticDataset, write_training_stats
    ds = SyntheticDataset(512, 10, seed=0, rank=rank)
    step_times, losses = [], []
    for step in range(args.warmup + args.steps):
        x, y = make_batch(kind, args.batch_size, ds, device)
        if use_cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=args.fp16 and use_cuda):
            loss = model(x, y) if kind.startswith("tokens") else torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        if use_cuda:
            torch.cuda.synchronize()
        if step >= args.warmup:
            step_times.append(time.perf_counter() - t0)
            losses.append(float(loss))
        if rank == 0 and (step % 50 == 0 or step == args.warmup + args.steps - 1):
            print(f"step {step:5d} loss {float(loss):.4f}", flush=True)
    avg = sum(step_times) / max(len(step_times), 1)
    if rank == 0:
        print(f"[{('baseline' if args.baseline else args.backend)}] params={n_params/1e6:.1f}M world={world} "
              f"avg_step={avg*1e3:.2f} ms throughput={args.batch_size*world/avg:.1f} samples/s")
        m = mccl.get_metrics() if (not args.baseline and args.backend == "mccl") else None
        if m is not None:
            print(f"  mccl metrics: ops={m.total_ops} sent={m.total_bytes_sent/1e9:.2f} GB p50={m.p50_latency_ms:.3f} ms "
                  f"p99={m.p99_latency_ms:.3f} ms peak={m.peak_throughput_gbps:.1f} Gbps sync/net/reduce="
                  f"{m.avg_sync_ms:.3f}/{m.avg_network_ms:.3f}/{m.avg_reduce_ms:.3f} ms errors={m.total_errors}")
        if args.save_stats:
            write_training_stats(args.save_stats, "baseline" if args.baseline else f"ddp-{args.backend}", step_times,
                                 losses, args.batch_size, world, n_params)
    if not args.baseline:
        first = next(model.parameters()).detach().reshape(-1)[:8].clone()
        ref = first.clone()
        dist.broadcast(ref, 0)
        dist.barrier()
        assert torch.allclose(first, ref), f"rank {rank}: replica diverged from rank 0"
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
