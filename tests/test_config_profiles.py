"""MCCLConfig: defaults, validation, env round-trip, profiles (reference tests/test_config_profiles.py)."""
import os

import pytest

from mccl_b200 import MCCLConfig
import mccl_b200 as mccl


@pytest.fixture(autouse=True)
def clean_env(monkeypatch):
    for k in list(os.environ):
        if k.startswith("MCCL_") or k == "DDP_BUCKET_MB":
            monkeypatch.delenv(k)
    yield


def test_defaults_match_reference_contract():
    c = MCCLConfig()
    assert c.transport == "auto" and c.port_base == 20100 and c.chunk_bytes == 16 * 1024 * 1024
    assert c.small_msg_threshold == 262144 and c.compression == "none" and c.topk_ratio == 0.01
    assert c.watchdog_timeout_ms == 300000 and c.heartbeat_interval_ms == 5000 and c.max_queue_depth == 1024
    assert c.overlap_comm is True and c.ring_algo == "auto" and c.log_level == "WARN" and c.ddp_bucket_mb == 25
    assert len(c._ENV_MAP) >= 31 and c._ENV_MAP["MCCL_TOPK_RATIO"] == "topk_ratio"


@pytest.mark.parametrize("kw", [
    dict(transport="udp"), dict(compression="zip"), dict(ring_algo="tree"), dict(pipeline_depth=0),
    dict(pipeline_depth=9), dict(collective_concurrency=9), dict(max_collective_concurrency=17),
    dict(cpu_write_sync="maybe"), dict(log_level="LOUD"), dict(port_base=0), dict(port_base=70000),
    dict(gpu_threshold=-1), dict(topk_ratio=0.0), dict(topk_ratio=1.5), dict(max_queue_depth=0),
    dict(chunk_bytes=0), dict(watchdog_timeout_ms=0), dict(algo="ring"), dict(wire_dtype="fp8"),
])
def test_validation_rejects(kw):
    with pytest.raises(ValueError):
        MCCLConfig(**kw)


def test_aliases_accepted():
    for a in ("auto", "chunked", "basic", "ring", "plain"):
        MCCLConfig(ring_algo=a)
    MCCLConfig(log_level="debug")


def test_to_env_skips_auto_and_empty():
    out = MCCLConfig().to_env()
    assert "MCCL_TRANSPORT" not in out and "MCCL_LISTEN_ADDR" not in out and "MCCL_IFNAME" not in out
    assert out["MCCL_COMPRESSION"] == "none" and out["MCCL_OVERLAP_COMM"] == "1"
    assert os.environ["MCCL_TOPK_RATIO"] == "0.01"


def test_env_roundtrip():
    os.environ["MCCL_COMPRESSION"] = "topk"
    os.environ["MCCL_TOPK_RATIO"] = "0.05"
    os.environ["MCCL_TRANSPORT_CRC"] = "1"
    os.environ["MCCL_PIPELINE_DEPTH"] = "4"
    os.environ["MCCL_ALGO"] = "twoshot"
    c = MCCLConfig.from_env()
    assert c.compression == "topk" and c.topk_ratio == 0.05 and c.transport_crc is True
    assert c.pipeline_depth == 4 and c.algo == "twoshot"
    os.environ["MCCL_PIPELINE_DEPTH"] = "40"
    with pytest.raises(ValueError):
        MCCLConfig.from_env()


def test_apply_to_env_respects_user_settings():
    os.environ["MCCL_COMPRESSION"] = "fp16"
    out = MCCLConfig(compression="topk").apply_to_env(only_if_unset=True)
    assert "MCCL_COMPRESSION" not in out and os.environ["MCCL_COMPRESSION"] == "fp16"
    out = MCCLConfig(compression="topk").apply_to_env(only_if_unset=False)
    assert os.environ["MCCL_COMPRESSION"] == "topk"


def test_from_dict_ignores_unknown_keys():
    c = MCCLConfig.from_dict({"compression": "fp16", "nonsense": 1})
    assert c.compression == "fp16"
    assert c.to_dict()["compression"] == "fp16" and "_ENV_MAP" not in c.to_dict()


def test_for_world_size_profiles():
    lab, perf = MCCLConfig.for_world_size(8), MCCLConfig.for_world_size(8, mode="perf", link_profile="thunderbolt")
    assert lab.collective_concurrency == 1
    assert perf.collective_concurrency == 3 and perf.pipeline_depth == 3 and perf.ring_algo == "chunked"
    assert perf.link_profile == "thunderbolt"


def test_init_variants():
    c = mccl.init(compression="fp16")
    assert mccl.get_config() is c and os.environ["MCCL_COMPRESSION"] == "fp16"
    c = mccl.init({"compression": "topk", "topk_ratio": 0.05})
    assert c.topk_ratio == 0.05 and os.environ["MCCL_TOPK_RATIO"] == "0.05"
    cfg = MCCLConfig(gpu_threshold=8192)
    assert mccl.init(cfg, log_level="INFO").log_level == "INFO"
    os.environ["MCCL_COMPRESSION"] = "none"
    assert mccl.init().compression == "none"


def test_presets():
    mccl.apply_thunderbolt_production_defaults(training_defaults=True)
    assert os.environ["MCCL_LINK_PROFILE"] == "thunderbolt" and os.environ["DDP_BUCKET_MB"] == "512"
    os.environ.pop("DDP_BUCKET_MB")
    mccl.apply_nvlink_production_defaults(training_defaults=True)
    assert os.environ["DDP_BUCKET_MB"] == "64"


def test_scope_annotations():
    assert MCCLConfig.scope("fast_math") == "compat" and MCCLConfig.scope("algo") == "cuda"
    assert MCCLConfig.scope("chunk_bytes") == "host"


def test_data_plane_knobs_validate_and_export(monkeypatch):
    import os
    import mccl_b200 as mccl
    for k in ("MCCL_GATHER", "MCCL_TILES", "MCCL_SEGMENT_BYTES", "MCCL_DEVICE_TIMING"):
        monkeypatch.delenv(k, raising=False)
    cfg = mccl.MCCLConfig()
    cfg.to_env()
    assert "MCCL_GATHER" not in os.environ and "MCCL_DEVICE_TIMING" not in os.environ   # defaults stay unexported
    cfg = mccl.MCCLConfig(gather="push", tiles=2, segment_bytes=32 << 20, device_timing=0)
    cfg.to_env()
    assert os.environ["MCCL_GATHER"] == "push" and os.environ["MCCL_TILES"] == "2"
    assert os.environ["MCCL_SEGMENT_BYTES"] == str(32 << 20) and os.environ["MCCL_DEVICE_TIMING"] == "0"
    import pytest
    for bad in (dict(gather="shove"), dict(tiles=0), dict(segment_bytes=1000), dict(device_timing=-1)):
        with pytest.raises(ValueError):
            mccl.MCCLConfig(**bad)
    for k in ("MCCL_GATHER", "MCCL_TILES", "MCCL_SEGMENT_BYTES", "MCCL_DEVICE_TIMING"):
        os.environ.pop(k, None)
