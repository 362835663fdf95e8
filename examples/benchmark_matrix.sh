#!/usr/bin/env bash
# Runs the headline DDP benchmark and the allreduce bus-bandwidth sweep for every
# GPU count up to the number given, for this backend and for NCCL, and collects
# one JSON line per run under the output folder.
# usage: benchmark_matrix.sh [max_gpus] [out_dir]
set -euo pipefail
cd "$(dirname "$0")/.."
MAXN=${1:-8}
OUT=${2:-bench_out}
STEPS=${STEPS:-60}
WARMUP=${WARMUP:-5}
mkdir -p "$OUT"
port=29600
run() {  # run <n> <args...>
  local n=$1; shift
  port=$((port + 1))
  if [ "$n" -eq 1 ]; then python "$@"; else
    python -m torch.distributed.run --nnodes=1 --nproc-per-node "$n" --master-addr 127.0.0.1 --master-port "$port" "$@"
  fi
}
for n in 1 2 4 8; do
  [ "$n" -le "$MAXN" ] || break
  for impl in mccl nccl; do
    run "$n" bench.py --impl "$impl" --gpus "$n" --steps "$STEPS" --warmup "$WARMUP" | grep '"metric"' > "$OUT/ddp_${impl}_n${n}.json" || true
  done
  if [ "$n" -ge 2 ]; then
    run "$n" -m mccl_b200.bench.busbw --compare-nccl --ops allreduce,allgather,reduce_scatter,broadcast \
        --dtypes fp32,bf16 --out "$OUT/busbw_n${n}.jsonl" > "$OUT/busbw_n${n}.log" 2>&1 || true
  fi
done
ls -l "$OUT"
