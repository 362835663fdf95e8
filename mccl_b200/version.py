"""Version and capability matrix (reference ``mccl/version.py:1-16``, re-targeted at B200)."""

__version__ = "0.5.0"

COMPATIBILITY_MATRIX = {
    "os": ["linux-x86_64"],
    "python": ["3.10", "3.11", "3.12"],
    "pytorch": ["2.11.x"],
    "cuda": ["12.8", "12.9"],
    "hardware": "NVIDIA B200 (sm_100a), up to 8 GPUs per NVLink 5 / NVSwitch domain",
    "backend_name": "mccl",
    "supported_devices": ["cuda", "cpu"],
    "supported_collectives": [
        "allreduce", "broadcast", "barrier",
        "allgather", "reduce_scatter",
        "send", "recv",
    ],
    "extra_collectives": [
        "allreduce_coalesced", "reduce", "_allgather_base", "_reduce_scatter_base",
        "allgather_into_tensor_coalesced", "reduce_scatter_tensor_coalesced",
    ],
    "compression_modes": ["none", "fp16", "topk"],
    "wire_dtypes": ["none", "bf16", "fp16"],
}
