"""Packaging: the native extension loads, versions agree, the backend is registered."""
import torch.distributed as dist


def test_versions(native):
    import mccl_b200
    assert mccl_b200.__version__ == "0.5.0"
    assert native.__version__ == mccl_b200.__version__
    assert native.__protocol_version__ == 5
    assert mccl_b200.COMPATIBILITY_MATRIX["backend_name"] == "mccl"
    assert set(mccl_b200.COMPATIBILITY_MATRIX["supported_devices"]) == {"cuda", "cpu"}
    for c in ("allreduce", "broadcast", "barrier", "allgather", "reduce_scatter", "send", "recv"):
        assert c in mccl_b200.COMPATIBILITY_MATRIX["supported_collectives"]


def test_backend_registered(native):
    assert "mccl" in dist.Backend.backend_list
    caps = dist.Backend.backend_capability["mccl"]
    assert "cpu" in caps and "cuda" in caps


def test_library_is_in_tree():
    from pathlib import Path
    import mccl_b200
    so = Path(mccl_b200._C.__file__)
    assert so.parent == Path(mccl_b200.__file__).parent, "the extension must live inside the package"


def test_import_mccl_alias():
    import mccl
    import mccl_b200
    assert mccl.MCCLConfig is mccl_b200.MCCLConfig
    from mccl.config import MCCLConfig  # noqa: F401
    from mccl.params import ensure_contiguous_parameters  # noqa: F401
    assert mccl.get_metrics() is None  # no process group yet
    assert mccl.staging_pool_bytes() >= 0
    mccl.log_metrics(); mccl.reset_metrics(); mccl.trim_staging_pool()


def test_nvls_tensor_pool_is_none_without_a_group_or_when_switched_off(monkeypatch):
    # the public helper never raises where NVLS cannot exist: no process group, or MCCL_NVLS=0
    from mccl_b200.parallel import nvls_tensor_pool
    assert nvls_tensor_pool(1 << 20) is None
    monkeypatch.setenv("MCCL_NVLS", "0")
    assert nvls_tensor_pool(1 << 20) is None


def test_package_reload_imports_the_library_again(native):
    # `from . import _C` would return the stale module-level name on a reload; the loader has to
    # import the submodule itself (the build entry point reloads the package after compiling)
    import importlib
    import mccl_b200
    saved = mccl_b200._C
    try:
        mccl_b200._C = None          # what a first import without the library leaves behind
        importlib.reload(mccl_b200)
        assert mccl_b200._C is not None and mccl_b200.require_native().__protocol_version__ == 5
    finally:
        if mccl_b200._C is None:
            mccl_b200._C = saved
