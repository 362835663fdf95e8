"""Benchmarks: ``python -m mccl_b200.bench.busbw`` (collective bus bandwidth vs NCCL) and
``python -m mccl_b200.bench.ddp`` (DDP throughput vs NCCL, dense and top-k compressed)."""
