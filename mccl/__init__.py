"""``import mccl``: drop-in name of the reference package, served by :mod:`mccl_b200`."""
import sys as _sys

import mccl_b200 as _impl
from mccl_b200 import *  # noqa: F401,F403
from mccl_b200 import __version__, COMPATIBILITY_MATRIX, _C, config, tuning, params, version  # noqa: F401

__all__ = _impl.__all__

# `mccl.config`, `mccl.params`, `mccl._C`, `mccl.transforms` ... resolve to the implementation modules.
for _name in ("config", "tuning", "params", "version"):
    _sys.modules[__name__ + "." + _name] = getattr(_impl, _name)
if _C is not None:
    _sys.modules[__name__ + "._C"] = _C


def __getattr__(name):
    import importlib

    if name in ("transforms", "ddp", "bench", "ops", "models", "parallel", "utils", "optim"):
        mod = importlib.import_module("mccl_b200." + name)
        _sys.modules[__name__ + "." + name] = mod
        return mod
    raise AttributeError(f"module 'mccl' has no attribute {name!r}")
