"""mccl_b200: a Blackwell-native ``torch.distributed`` backend named ``"mccl"``.

Importing the package registers the backend for CUDA and CPU tensors::

    import mccl_b200 as mccl          # or simply:  import mccl
    mccl.init(compression="none")     # optional: validates and exports MCCL_* knobs
    torch.distributed.init_process_group(backend="mccl", ...)
    model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank])

CUDA collectives are single fused sm_100a kernels that read and write the
peers' memory over NVLink 5 / NVSwitch (see ``csrc/kernels/reduce_kernels.cuh`` and ``csrc/kernels/collectives.cu``);
CPU collectives run over a framed TCP mesh.  The public names mirror the
reference package (``mccl/__init__.py:167-179``): ``init``, ``get_config``,
``get_metrics``, ``log_metrics``, ``reset_metrics``, ``trim_staging_pool``,
``staging_pool_bytes``, ``MCCLConfig``, ``apply_thunderbolt_production_defaults``,
``__version__`` and ``COMPATIBILITY_MATRIX``.
"""
from __future__ import annotations

import os
import sys
import warnings
from typing import Any, Dict, Optional

from .version import __version__, COMPATIBILITY_MATRIX
from .config import MCCLConfig
from .tuning import apply_thunderbolt_production_defaults, apply_nvlink_production_defaults
from . import config, params, tuning, version  # noqa: F401  (submodules reachable as attributes)

_active_config: Optional[MCCLConfig] = None
_backend_registered: bool = False
_native_error: Optional[BaseException] = None


def _load_native():
    """Imports ``_C``; builds it first when the library is missing (source checkout)."""
    global _native_error
    import torch.distributed  # noqa: F401  (registers the c10d pybind base classes)
    alt = os.environ.get("MCCL_NATIVE_LIB", "")
    if alt:
        # An explicitly named build of the extension (the sanitizer-instrumented one, for instance).
        import importlib.machinery
        import importlib.util
        try:
            loader = importlib.machinery.ExtensionFileLoader(__name__ + "._C", alt)
            spec = importlib.util.spec_from_file_location(__name__ + "._C", alt, loader=loader)
            mod = importlib.util.module_from_spec(spec)
            loader.exec_module(mod)
            sys.modules[__name__ + "._C"] = mod
            return mod
        except Exception as e:
            _native_error = e
            return None
    import importlib
    try:
        # import_module, not `from . import _C`: on a reload of this package the old module-level
        # name `_C` (None after a failed first import) would be found and returned instead
        return importlib.import_module(__name__ + "._C")
    except ImportError as first:
        building_now = "mccl_b200._build" in getattr(sys, "orig_argv", [])
        if os.environ.get("MCCL_NO_AUTOBUILD") == "1" or building_now:
            _native_error = first
            return None
        from . import _build
        if _build.TARGET.exists():
            # The library exists but does not load: rebuilding silently would hide the cause.
            _native_error = first
            return None
        try:
            _build.build()
            return importlib.import_module(__name__ + "._C")
        except Exception as e:  # pragma: no cover - depends on the toolchain
            _native_error = e
            return None


_C = _load_native()
if _C is not None:
    try:
        _C._register_backend()
        _backend_registered = True
    except Exception as e:  # pragma: no cover
        _native_error = e
        warnings.warn(f"mccl_b200: backend registration failed: {e}", RuntimeWarning, stacklevel=2)
elif "mccl_b200._build" not in getattr(sys, "orig_argv", []):
    warnings.warn(
        f"mccl_b200: native extension unavailable ({_native_error}). "
        "Build it with: python -m mccl_b200._build",
        RuntimeWarning,
        stacklevel=2,
    )


def require_native():
    """Returns the native module or raises: GPU code paths never fall back silently."""
    if _C is None:
        raise RuntimeError(f"mccl_b200 native extension is not loaded: {_native_error}")
    return _C


def init(config: "MCCLConfig | Dict[str, Any] | None" = None, **kwargs: Any) -> MCCLConfig:
    """Resolve the configuration and export it to ``MCCL_*`` variables.

    Accepts an :class:`MCCLConfig`, a mapping, keyword arguments, or nothing
    (then the current environment is read).  Call before
    ``init_process_group(backend="mccl")``; returns the active config.
    """
    global _active_config
    if isinstance(config, MCCLConfig):
        for k, v in kwargs.items():
            setattr(config, k, v)
        cfg = config
    elif isinstance(config, dict):
        cfg = MCCLConfig.from_dict({**config, **kwargs})
    elif kwargs:
        cfg = MCCLConfig(**kwargs)
    else:
        cfg = MCCLConfig.from_env()
    cfg.to_env()
    _active_config = cfg
    return cfg


def get_config() -> Optional[MCCLConfig]:
    """The config passed to / produced by :func:`init`, or ``None``."""
    return _active_config


def get_metrics():
    """Snapshot of the active process group's metrics (``None`` without a group)."""
    if _C is None:
        return None
    try:
        return _C._get_metrics_summary()
    except RuntimeError:
        return None


def log_metrics() -> None:
    """Print the metrics summary of the active process group to stderr."""
    if _C is not None:
        try:
            _C._log_metrics()
        except RuntimeError:
            pass


def reset_metrics() -> None:
    """Zero all metric counters of the active process group."""
    if _C is not None:
        try:
            _C._reset_metrics()
        except RuntimeError:
            pass


def trim_staging_pool() -> None:
    """Free idle buffers of the host staging pool."""
    if _C is not None:
        _C._trim_staging_pool()


def staging_pool_bytes() -> int:
    """Bytes currently held by the host staging pool (0 when unavailable)."""
    return int(_C._staging_pool_bytes()) if _C is not None else 0


def get_backend(group=None, device=None):
    """The native ``ProcessGroupMCCL`` behind ``group`` (default group if omitted)."""
    import torch
    import torch.distributed as dist

    pg = group if group is not None else dist.distributed_c10d._get_default_group()
    if device is None:
        device = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
    return pg._get_backend(torch.device(device))


__all__ = [
    "__version__",
    "COMPATIBILITY_MATRIX",
    "MCCLConfig",
    "init",
    "get_config",
    "get_metrics",
    "log_metrics",
    "reset_metrics",
    "trim_staging_pool",
    "staging_pool_bytes",
    "apply_thunderbolt_production_defaults",
    "apply_nvlink_production_defaults",
    "get_backend",
    "require_native",
]
