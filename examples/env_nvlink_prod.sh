#!/usr/bin/env bash
# Environment preset for an 8x B200 NVSwitch node: source before torchrun.
export MCCL_OVERLAP_COMM=${MCCL_OVERLAP_COMM:-1}     # collectives on the side streams
export MCCL_ALGO=${MCCL_ALGO:-auto}                  # one-shot / two-shot / NVLS from the tuner table
export MCCL_NVLS=${MCCL_NVLS:-auto}                  # multimem kernels and in-place DDP buckets where the switch supports them
export MCCL_LOG_LEVEL=${MCCL_LOG_LEVEL:-WARN}
export MCCL_WATCHDOG_TIMEOUT_MS=${MCCL_WATCHDOG_TIMEOUT_MS:-300000}
export DDP_BUCKET_MB=${DDP_BUCKET_MB:-25}
# export MCCL_WIRE_DTYPE=bf16                        # fp32 gradients travel as bf16 (fused cast)
# export MCCL_COMPRESSION=topk MCCL_TOPK_RATIO=0.01  # top-k gradients with error feedback
# export MCCL_TUNE_FILE=/path/to/tune.json           # written by: python -m mccl_b200.bench.busbw --tune FILE
# export MCCL_GATHER=pull                            # two-shot second half: peers pull (owners push is the measured default)
# export MCCL_NVLS_BUCKETS=0                         # keep DDP's buckets out of the multicast-bound pool
# export MCCL_DEVICE_TIMING=0                        # no device-timed samples for the metrics (saves ~3 us per call)
