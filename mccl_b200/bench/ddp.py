"""DDP throughput: this backend vs torch's NCCL backend on the same GPUs, device-timed.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29530 \
        -m mccl_b200.bench.ddp --model resnet50 --impl mccl --steps 20
    ... --model gpt2-medium --compression topk        # top-k 1 % + error feedback vs the dense path

Configs: ``mlp`` (94 M fp32 MLP, global batch 256, AdamW), ``resnet50`` (bf16 autocast,
256 images per GPU, SGD momentum 0.9 lr 0.1), ``gpt2-medium`` (bf16 autocast, seq 1024,
micro-batch 8 per GPU, AdamW).  Synthetic data, random-init weights.  Prints one JSON line
from rank 0 (samples/s aggregated over all ranks, ms/step = max over ranks, and the loss
curve so compressed and dense runs can be compared).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mlp", choices=["mlp", "resnet50", "gpt2-medium", "gpt2-tiny"])
    ap.add_argument("--impl", default="mccl", choices=["mccl", "nccl"])
    ap.add_argument("--compression", default="none", choices=["none", "topk"])
    ap.add_argument("--topk-ratio", type=float, default=0.01)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--bucket-mb", type=int, default=25)
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (0: the config's default)")
    ap.add_argument("--curve-points", type=int, default=10, help="how many points of the loss curve to print")
    ap.add_argument("--optim-in-backward", action="store_true", help="AdamW per bucket behind its allreduce (native hook)")
    args = ap.parse_args(argv)

    rank, ws, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import mccl_b200 as mccl
    from mccl_b200 import models
    from mccl_b200.optim import FusedAdamW
    from mccl_b200.parallel import wrap_ddp
    dist.init_process_group(args.impl, rank=rank, world_size=ws, device_id=dev)
    torch.manual_seed(42)
    if args.model == "mlp":
        model, bs, autocast = models.MLP94M().to(dev), args.batch or 256 // ws, False
        batch = lambda: (torch.randn(bs, 2048, device=dev), torch.randint(0, 1000, (bs,), device=dev))
    elif args.model == "resnet50":
        model, bs, autocast = models.ResNet50().to(dev).to(memory_format=torch.channels_last), args.batch or 256, True
        batch = lambda: (torch.randn(bs, 3, 224, 224, device=dev).contiguous(memory_format=torch.channels_last),
                         torch.randint(0, 1000, (bs,), device=dev))
    else:
        big = args.model == "gpt2-medium"
        model, bs, autocast = (models.gpt2_medium() if big else models.gpt2_tiny()).to(dev), args.batch or 8, True
        vocab, seq = (50257, 1024) if big else (1024, 64)

        def batch():
            ids = torch.randint(0, vocab, (bs, seq + 1), device=dev)
            return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    n_params = sum(p.numel() for p in model.parameters())
    pre_opt = None
    if args.impl == "mccl":
        if args.optim_in_backward and args.model != "resnet50" and args.compression == "none":
            pre_opt = FusedAdamW(model.parameters(), lr=1e-3 if args.model == "mlp" else 3e-4)
        ddp = wrap_ddp(model, device_ids=[local], bucket_cap_mb=args.bucket_mb, compression=args.compression,
                       optimizer_in_backward=pre_opt)
        if args.compression == "topk":
            ddp._mccl_topk_state.ratio = args.topk_ratio
    else:
        from torch.nn.parallel import DistributedDataParallel
        ddp = DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=args.bucket_mb,
                                      gradient_as_bucket_view=True)
    if args.model == "resnet50":
        opt = torch.optim.SGD(ddp.parameters(), lr=0.1, momentum=0.9)
    elif pre_opt is not None:
        opt = pre_opt
    elif args.impl == "mccl":
        opt = FusedAdamW(ddp.parameters(), lr=1e-3 if args.model == "mlp" else 3e-4)
    else:
        opt = torch.optim.AdamW(ddp.parameters(), lr=1e-3 if args.model == "mlp" else 3e-4, fused=True)
    data = [batch() for _ in range(4)]
    losses = []

    def step(i):
        x, y = data[i % len(data)]
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
            loss = ddp(x, y) if args.model.startswith("gpt2") else torch.nn.functional.cross_entropy(ddp(x), y)
        loss.backward()
        opt.step()
        return loss

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(args.steps):
        losses.append(step(i).detach())
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / args.steps
    if rank == 0:
        print(json.dumps({"bench": "ddp", "model": args.model, "impl": args.impl, "compression": args.compression,
                          "n_gpus": ws, "params": n_params, "per_gpu_batch": bs, "ms_per_step": round(ms, 3),
                          "samples_per_s": round(bs * ws / (ms / 1e3), 1), "dtype": "bf16 autocast" if autocast else "fp32",
                          "losses": [round(float(l), 4) for l in losses[:: max(1, len(losses) // max(1, args.curve_points))]],
                          "data": "synthetic"}), flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
