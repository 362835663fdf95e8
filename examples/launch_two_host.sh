#!/usr/bin/env bash
# usage (run once on EACH host): launch_two_host.sh <node_rank 0|1> <master_ip> <gpus_per_host> <script.py> [args...]
#
# Two hosts are not one NVLink domain: the peer arena cannot be mapped across them, so every rank
# agrees through the Store to stage CUDA collectives through host memory and the framed TCP mesh
# (slow path, for functional runs).  MCCL_LISTEN_ADDR must be an address the other host can reach.
set -euo pipefail
NODE_RANK=${1:?node rank (0 or 1)}; MASTER=${2:?address of host 0}; N=${3:?GPUs per host}; shift 3
export MCCL_LISTEN_ADDR=${MCCL_LISTEN_ADDR:-$(hostname -I | awk '{print $1}')}
export MCCL_PORT_BASE=${MCCL_PORT_BASE:-29600}
export MCCL_NVLS=0
exec python -m torch.distributed.run --nnodes=2 --node-rank "$NODE_RANK" --nproc-per-node "$N" \
     --master-addr "$MASTER" --master-port "${MASTER_PORT:-29500}" "$@"
