#!/usr/bin/env bash
# usage: launch_single_node.sh <num_gpus> <script.py> [script args...]
set -euo pipefail
N=${1:?number of GPUs}; shift
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 \
     --master-port "${MASTER_PORT:-29500}" "$@"
