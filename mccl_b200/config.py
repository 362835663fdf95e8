"""MCCLConfig: every tunable of the backend, mirrored to ``MCCL_*`` environment variables.

The native layer reads its knobs from the environment when a process group is
constructed, so the Python side's job is to validate values and export them.
Field names, defaults, validation ranges and the env-var mapping follow the
reference (``mccl/config.py:22-284``) so existing launch scripts keep working;
fields that only meant something for Apple GPUs / TCP rings are still accepted
and exported but are documented as having no effect on the CUDA data plane.
B200-specific knobs (``algo``, ``oneshot_max_bytes``, ``comm_ctas``,
``wire_dtype``, ``tune_file``, ``device_wait_us``, ``arena_bytes``,
``blocking_wait``) are additions.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Any, Callable, Dict, Optional

_LOG_LEVELS = ("TRACE", "DEBUG", "INFO", "WARN", "ERROR", "FATAL", "OFF")


def _one_of(*allowed: str) -> Callable[[str, Any], None]:
    def check(name: str, value: Any) -> None:
        if value not in allowed:
            raise ValueError(f"{name} must be one of {sorted(allowed)}, got {value!r}")
    return check


def _in_range(lo: Optional[float], hi: Optional[float], *, lo_open: bool = False) -> Callable[[str, Any], None]:
    def check(name: str, value: Any) -> None:
        too_low = lo is not None and (value <= lo if lo_open else value < lo)
        too_high = hi is not None and value > hi
        if too_low or too_high:
            left = "(" if lo_open else "["
            raise ValueError(f"{name} must be in {left}{lo}, {hi}], got {value}" if hi is not None
                             else f"{name} must be >= {lo}, got {value}")
    return check


def _log_level(name: str, value: Any) -> None:
    if str(value).upper() not in _LOG_LEVELS:
        raise ValueError(f"{name} must be one of {sorted(_LOG_LEVELS)}, got {value!r}")


# field -> (env var or None, validator or None, "cuda" | "host" | "both" | "compat")
# "compat": accepted for API compatibility, no effect on the CUDA data plane.
_FIELD_SPEC: Dict[str, tuple] = {
    # transport (host control/data plane)
    "transport": ("MCCL_TRANSPORT", _one_of("auto", "tcp", "rdma"), "host"),
    "listen_addr": ("MCCL_LISTEN_ADDR", None, "host"),
    "port_base": ("MCCL_PORT_BASE", _in_range(1, 65535), "host"),
    "ifname": ("MCCL_IFNAME", None, "host"),
    "chunk_bytes": ("MCCL_CHUNK_BYTES", _in_range(1, None), "host"),
    "small_msg_threshold": ("MCCL_SMALL_MSG_THRESHOLD", None, "host"),
    "connect_timeout_ms": ("MCCL_CONNECT_TIMEOUT_MS", None, "host"),
    "transport_crc": ("MCCL_TRANSPORT_CRC", None, "host"),
    # compute
    "fast_math": ("MCCL_FAST_MATH", None, "compat"),
    "gpu_threshold": ("MCCL_GPU_THRESHOLD", _in_range(0, None), "compat"),
    "shader_path": ("MCCL_SHADER_PATH", None, "compat"),
    "overlap_comm": ("MCCL_OVERLAP_COMM", None, "cuda"),
    "ring_algo": ("MCCL_RING_ALGO", _one_of("auto", "chunked", "basic", "ring", "plain"), "compat"),
    "ring_pipeline": ("MCCL_RING_PIPELINE", None, "compat"),
    "pipeline_depth": ("MCCL_PIPELINE_DEPTH", _in_range(1, 8), "compat"),
    "collective_concurrency": ("MCCL_COLLECTIVE_CONCURRENCY", _in_range(1, 8), "both"),
    "max_collective_concurrency": ("MCCL_MAX_COLLECTIVE_CONCURRENCY", _in_range(1, 16), "both"),
    "demux_park_bytes": ("MCCL_DEMUX_PARK_BYTES", None, "host"),
    "demux_inflight_budget_bytes": ("MCCL_DEMUX_INFLIGHT_BUDGET_BYTES", None, "both"),
    "credit_min_chunk": ("MCCL_CREDIT_MIN_CHUNK", None, "compat"),
    "fp32_cpu_reduce": ("MCCL_FP32_CPU_REDUCE", None, "compat"),
    "cpu_write_sync": ("MCCL_CPU_WRITE_SYNC", _one_of("auto", "none", "full"), "compat"),
    "event_sync": ("MCCL_EVENT_SYNC", None, "compat"),
    "link_profile": ("MCCL_LINK_PROFILE", None, "host"),
    "unified_collective": ("MCCL_UNIFIED_COLLECTIVE", None, "compat"),
    # compression
    "compression": ("MCCL_COMPRESSION", _one_of("none", "fp16", "topk"), "both"),
    "topk_ratio": ("MCCL_TOPK_RATIO", _in_range(0.0, 1.0, lo_open=True), "both"),
    # runtime
    "watchdog_timeout_ms": ("MCCL_WATCHDOG_TIMEOUT_MS", _in_range(1, None), "both"),
    "heartbeat_interval_ms": ("MCCL_HEARTBEAT_INTERVAL_MS", None, "both"),
    "max_queue_depth": ("MCCL_MAX_QUEUE_DEPTH", _in_range(1, None), "host"),
    "log_level": ("MCCL_LOG_LEVEL", _log_level, "both"),
    # B200 data plane
    "algo": ("MCCL_ALGO", _one_of("auto", "oneshot", "twoshot", "nvls", "staged"), "cuda"),
    "oneshot_max_bytes": ("MCCL_ONESHOT_MAX_BYTES", _in_range(-1, None), "cuda"),
    "comm_ctas": ("MCCL_COMM_CTAS", _in_range(0, 64), "cuda"),
    "wire_dtype": ("MCCL_WIRE_DTYPE", _one_of("none", "bf16", "fp16"), "cuda"),
    "tune_file": ("MCCL_TUNE_FILE", None, "cuda"),
    "device_wait_us": ("MCCL_DEVICE_WAIT_US", _in_range(1, None), "cuda"),
    "arena_bytes": ("MCCL_ARENA_BYTES", _in_range(1 << 20, None), "cuda"),
    "blocking_wait": ("MCCL_BLOCKING_WAIT", None, "cuda"),
    "gather": ("MCCL_GATHER", _one_of("auto", "pull", "push"), "cuda"),
    "tiles": ("MCCL_TILES", _in_range(1, 64), "cuda"),
    "segment_bytes": ("MCCL_SEGMENT_BYTES", _in_range(1 << 20, None), "cuda"),
    "device_timing": ("MCCL_DEVICE_TIMING", _in_range(0, None), "cuda"),
    "nvls": ("MCCL_NVLS", _one_of("auto", "0", "1", "on", "off"), "cuda"),
    "nvls_bytes": ("MCCL_NVLS_BYTES", _in_range(1 << 20, None), "cuda"),
    "nvls_min_bytes": ("MCCL_NVLS_MIN_BYTES", _in_range(-2, None), "cuda"),
    "nvls_split_min_bytes": ("MCCL_NVLS_SPLIT_MIN_BYTES", _in_range(-2, None), "cuda"),
    "tile_bytes": ("MCCL_TILE_BYTES", _in_range(0, None), "cuda"),
    "debug_checks": ("MCCL_DEBUG_CHECKS", None, "cuda"),
    # integration hint only (never exported)
    "ddp_bucket_mb": (None, _in_range(1, None), "both"),
}


@dataclasses.dataclass
class MCCLConfig:
    """All tunables in one place; see the module docstring for the contract."""

    # transport
    transport: str = "auto"
    listen_addr: str = "auto"
    port_base: int = 20100
    ifname: str = ""
    chunk_bytes: int = 16 * 1024 * 1024
    small_msg_threshold: int = 262144
    connect_timeout_ms: int = 30000
    transport_crc: bool = False
    # compute
    fast_math: bool = True
    gpu_threshold: int = 4096
    shader_path: str = ""
    overlap_comm: bool = True
    ring_algo: str = "auto"
    ring_pipeline: bool = True
    pipeline_depth: int = 1
    collective_concurrency: int = 1
    max_collective_concurrency: int = 8
    demux_park_bytes: int = 512 * 1024 * 1024
    demux_inflight_budget_bytes: int = 1024 * 1024 * 1024
    credit_min_chunk: int = 1024 * 1024
    fp32_cpu_reduce: bool = False
    cpu_write_sync: str = "auto"
    event_sync: bool = True
    link_profile: str = ""
    unified_collective: bool = True
    # compression
    compression: str = "none"
    topk_ratio: float = 0.01
    # runtime
    watchdog_timeout_ms: int = 300000
    heartbeat_interval_ms: int = 5000
    max_queue_depth: int = 1024
    log_level: str = "WARN"
    # B200 data plane
    algo: str = "auto"
    oneshot_max_bytes: int = -1
    comm_ctas: int = 0
    wire_dtype: str = "none"
    tune_file: str = ""
    device_wait_us: int = 60_000_000
    arena_bytes: int = 128 * 1024 * 1024
    blocking_wait: bool = False
    gather: str = "auto"            # second half of the two-shot allreduce: tuner table | peers pull | owners push
    tiles: int = 1                  # two-shot pipeline tiles per CTA
    segment_bytes: int = 64 * 1024 * 1024   # large allreduces run as segments of this size on alternating lanes
    device_timing: int = 8          # every Nth CUDA collective is device-timed for the metrics (0: never)
    nvls: str = "auto"              # NVLink multicast (in-switch reduction): auto | 0 | 1
    nvls_bytes: int = 64 * 1024 * 1024      # one of the four NVLS buffers per rank
    nvls_min_bytes: int = -2        # allreduce: smallest payload for the NVLS kernel (-2: tuner table, -1: never)
    nvls_split_min_bytes: int = -2  # NVLS allreduce: staging passes as separate kernels from this size (-2: tuner, -1: never)
    tile_bytes: int = 0             # pipeline tile of the byte movers and NVLS kernels (0: tuner table)
    debug_checks: bool = False      # kernels verify their buffer ranges and report violations instead of accessing
    # integration hint (not exported to the native layer)
    ddp_bucket_mb: int = 25

    _ENV_MAP: Dict[str, str] = dataclasses.field(default_factory=dict, repr=False, init=False)

    # Fields whose default must not be exported unless the user set them: the
    # native default differs (ephemeral ports) or derives from other knobs.
    _EXPORT_ONLY_IF_CHANGED = ("port_base", "device_wait_us", "oneshot_max_bytes", "comm_ctas",
                               "arena_bytes", "blocking_wait", "algo", "wire_dtype", "gather", "tiles", "segment_bytes",
                               "device_timing", "nvls", "nvls_bytes", "nvls_min_bytes", "nvls_split_min_bytes", "tile_bytes", "debug_checks")

    def __post_init__(self) -> None:
        self._ENV_MAP = {env: name for name, (env, _v, _s) in _FIELD_SPEC.items() if env}
        self._validate()

    def __setattr__(self, name: str, value: Any) -> None:
        object.__setattr__(self, name, value)

    def _validate(self) -> None:
        for name, (_env, validator, _scope) in _FIELD_SPEC.items():
            if validator is not None:
                validator(name, getattr(self, name))

    # ---- construction ------------------------------------------------------
    @classmethod
    def from_env(cls) -> "MCCLConfig":
        """Defaults overridden by whatever ``MCCL_*`` variables are set."""
        cfg = cls()
        for env_key, name in cfg._ENV_MAP.items():
            raw = os.environ.get(env_key)
            if raw is not None:
                setattr(cfg, name, _coerce(raw, type(getattr(cfg, name))))
        cfg._validate()
        return cfg

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MCCLConfig":
        """Build from a plain mapping (parsed YAML/JSON); unknown keys are ignored."""
        known = {f.name for f in dataclasses.fields(cls) if f.init}
        return cls(**{k: v for k, v in d.items() if k in known})

    @classmethod
    def for_world_size(cls, world_size: int, *, mode: str = "lab", link_profile: str = "") -> "MCCLConfig":
        """Defaults do not depend on the world size; ``mode="perf"`` raises concurrency knobs."""
        del world_size
        cfg = cls()
        if link_profile:
            cfg.link_profile = link_profile
        if mode == "perf":
            cfg.ring_algo = "chunked"
            cfg.collective_concurrency = 3
            cfg.pipeline_depth = 3
        return cfg

    # ---- export --------------------------------------------------------------
    def _env_items(self):
        defaults = {f.name: f.default for f in dataclasses.fields(self) if f.init}
        for env_key, name in self._ENV_MAP.items():
            value = getattr(self, name)
            if name in self._EXPORT_ONLY_IF_CHANGED and value == defaults[name]:
                continue
            text = ("1" if value else "0") if isinstance(value, bool) else str(value)
            # "" and "auto" mean "use the built-in default": leave the environment alone.
            if text and text != "auto":
                yield env_key, text

    def to_env(self) -> Dict[str, str]:
        """Write the values into ``os.environ`` and return what was written."""
        self._validate()
        out = dict(self._env_items())
        os.environ.update(out)
        return out

    def apply_to_env(self, only_if_unset: bool = True) -> Dict[str, str]:
        """Like :meth:`to_env`, but keeps variables the user already set."""
        self._validate()
        out = {}
        for key, text in self._env_items():
            if only_if_unset and os.environ.get(key) is not None:
                continue
            os.environ[key] = text
            out[key] = text
        return out

    def to_dict(self) -> Dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in dataclasses.fields(self) if f.init}

    @staticmethod
    def scope(field_name: str) -> str:
        """"cuda", "host", "both" or "compat" (accepted, no effect on CUDA)."""
        return _FIELD_SPEC[field_name][2]

    def __str__(self) -> str:
        body = "".join(f"  {k}={v!r},\n" for k, v in self.to_dict().items())
        return f"MCCLConfig(\n{body})"


def _coerce(raw: str, target: type) -> Any:
    if target is bool:
        return raw not in ("0", "false", "FALSE", "no", "NO", "")
    if target is int:
        return int(raw)
    if target is float:
        return float(raw)
    return raw
