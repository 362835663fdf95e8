"""Optional presets applied to ``os.environ`` before ``init_process_group``.

``apply_thunderbolt_production_defaults`` keeps the reference's name and
contract (``mccl/tuning.py:9-28``): it opts the *host* transport into its
high-bandwidth-link profile (larger socket buffers, frames of at least 16 MiB).
``apply_nvlink_production_defaults`` is the B200 counterpart for the CUDA data
plane.  Both only set variables that are not set already.
"""
from __future__ import annotations

import os


def apply_thunderbolt_production_defaults(*, training_defaults: bool = False) -> None:
    """Host-transport preset; with ``training_defaults`` also overlap + large DDP buckets."""
    os.environ.setdefault("MCCL_LINK_PROFILE", "thunderbolt")
    if training_defaults:
        os.environ.setdefault("MCCL_OVERLAP_COMM", "1")
        os.environ.setdefault("DDP_BUCKET_MB", "512")


def apply_nvlink_production_defaults(*, training_defaults: bool = False) -> None:
    """CUDA data-plane preset for an 8x B200 NVSwitch node.

    Collectives run on the side streams (overlap on) with the tuner's size table and the NVLS
    kernels where the switch offers multicast; with ``training_defaults`` DDP buckets are sized
    so that one bucket is one segment (launch latency amortised, still several buckets in
    flight for a ~100 M parameter model).
    """
    os.environ.setdefault("MCCL_OVERLAP_COMM", "1")
    os.environ.setdefault("MCCL_ALGO", "auto")
    os.environ.setdefault("MCCL_NVLS", "auto")
    if training_defaults:
        os.environ.setdefault("DDP_BUCKET_MB", "64")


__all__ = ["apply_thunderbolt_production_defaults", "apply_nvlink_production_defaults"]
