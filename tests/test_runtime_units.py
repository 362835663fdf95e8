"""Host runtime pieces in isolation: watchdog, engine, memory pool, metrics, options."""
import datetime

import torch.distributed as dist


def test_watchdog_unarmed_entries_never_expire(native):
    assert native._test_watchdog(50, False, 300) == 0   # watched but never touched: queued work is safe
    assert native._test_watchdog(50, True, 300) == 1    # armed: fires exactly once


def test_engine_runs_everything_and_reports_errors(native):
    order, done, errs = native._test_engine(1, 4, 50, 5)
    assert order == list(range(50)), "one worker = submission order"
    assert done == 40 and errs == 10
    order, done, errs = native._test_engine(3, 2, 40, 0)  # tiny queue: submitter blocks, nothing is lost
    assert sorted(order) == list(range(40)) and done == 40 and errs == 0


def test_memory_pool_reuse_and_trim(native):
    first, second, reused, total, after_trim = native._test_mempool()
    assert first >= 1_250_000 and first % 4096 == 0      # 25 % head-room, page aligned
    assert reused and second == first                     # best fit reuses the freed buffer
    assert total == first and after_trim == 0


def test_options_object_is_honoured(native):
    o = native.MCCLOptions(datetime.timedelta(seconds=30))
    o.small_msg_threshold = 1234
    o.algo = "twoshot"
    pg = native.ProcessGroupMCCL(dist.HashStore(), 0, 1, o)
    d = pg.describe()
    assert "small_msg_threshold=1234" in d and "algo=twoshot" in d
    assert pg.data_plane() == "local" and not pg.poisoned
    m = pg.get_metrics()
    assert m.total_ops == 0 and m.total_errors == 0
    pg.shutdown()


def test_metrics_summary_fields(native):
    fields = ["total_ops", "total_bytes_sent", "total_bytes_recv", "total_errors", "avg_latency_ms",
              "p50_latency_ms", "p99_latency_ms", "peak_throughput_gbps", "avg_sync_ms", "avg_network_ms",
              "avg_reduce_ms", "avg_queue_wait_ms", "avg_execution_ms"]
    pg = native._create_process_group(dist.HashStore(), 0, 1, datetime.timedelta(seconds=10))
    m = pg.get_metrics()
    for f in fields:
        assert hasattr(m, f), f
    pg.shutdown()


def test_tuner_file_overrides(native, tmp_path, monkeypatch):
    import json
    f = tmp_path / "tune.json"
    f.write_text(json.dumps({"ws8_oneshot_max_bytes": 524288, "ws8_ctas_large": 48, "segment_bytes": 33554432,
                             "ws8_push_gather": 1, "ws2_push_gather": 0, "ws8_ctas_overlap": 40,
                             "ws8_broadcast_nvls_min_bytes": 65536, "ws8_broadcast_nvls_max_bytes": 4194304,
                             "measured": [{"bytes": 1, "oneshot_us": 2.0}]}))
    monkeypatch.setenv("MCCL_TUNE_FILE", str(f))
    pg = native._create_process_group(dist.HashStore(), 0, 1, datetime.timedelta(seconds=10))
    t = json.loads(pg.tuner_dump())
    assert t["ws8_oneshot_max_bytes"] == 524288 and t["ws8_ctas_large"] == 48 and t["segment_bytes"] == 33554432
    assert t["ws2_oneshot_max_bytes"] == 32 << 20   # untouched default
    assert t["ws8_push_gather"] == 1 and t["ws2_push_gather"] == 0
    assert t["ws4_push_gather"] == 1 and t["ws6_push_gather"] == 1   # untouched defaults (measured: owners push)
    assert t["ws8_ctas_overlap"] == 40 and t["ws2_ctas_overlap"] == 48 and t["ws4_ctas_overlap"] == 0
    # broadcast through multimem.st has a floor and a ceiling (no ceiling at 3-4 ranks by default)
    assert t["ws8_broadcast_nvls_min_bytes"] == 65536 and t["ws8_broadcast_nvls_max_bytes"] == 4194304
    assert t["ws6_broadcast_nvls_max_bytes"] == 8 << 20 and t["ws4_broadcast_nvls_max_bytes"] == -1
    pg.shutdown()


def test_collective_concurrency_caps_lanes(native, monkeypatch):
    monkeypatch.setenv("MCCL_COLLECTIVE_CONCURRENCY", "1")
    pg = native._create_process_group(dist.HashStore(), 0, 1, datetime.timedelta(seconds=10))
    assert "lanes=1" in pg.describe()
    pg.shutdown()
    monkeypatch.delenv("MCCL_COLLECTIVE_CONCURRENCY")
    pg = native._create_process_group(dist.HashStore(), 0, 1, datetime.timedelta(seconds=10))
    assert "lanes=2" in pg.describe()
    pg.shutdown()


def test_tile_plan_is_a_partition_owned_by_cta_index(native):
    # Every unit belongs to exactly one tile, tile g to CTA g % nctas, and the plan depends only on
    # (units, grid, tile size): writer and reader of a tile are the same CTA index on every rank.
    for units in (1, 2047, 2048, 2049, 62_500, 1_000_000, 8_388_608):
        for nctas in (1, 4, 62, 64):
            for tile_bytes in (0, 8192, 1 << 20):
                tu, nt = native._tile_plan(units, nctas, 512, tile_bytes)
                assert tu % (512 * 4) == 0 and tu > 0
                assert (nt - 1) * tu < units <= nt * tu
                per_cta = -(-nt // nctas)
                assert per_cta <= 1024, "12-bit tile counters"


def test_pool_range_allocator_first_fit_and_coalescing(native):
    # steps: +n allocates n bytes, -i releases the block of step i (1-based); 512-byte granules
    offs, used, free_blocks = native._test_range_allocator(1 << 20, [1000, 512, 4096, -2, 300, -1, -3, -5, 1 << 20])
    assert offs[0] == 0 and offs[1] == 1024 and offs[2] == 1536          # 1000 B takes two granules
    assert offs[3] == 0                                                    # release of step 2's block
    assert offs[4] == 1024                                                 # first fit: reuses the hole
    assert offs[5:8] == [0, 0, 0] and used == 1 << 20 and free_blocks == 0  # all released, coalesced, whole range taken
    assert offs[8] == 0
    offs, used, _ = native._test_range_allocator(4096, [4096, 1, -1, -1])
    assert offs == [0, -1, 0, -2] and used == 0                            # full -> -1; double release is refused


def test_mover_tile_rule_keeps_small_world_sizes_and_cuts_small_shares(native):
    MiB, KiB = 1 << 20, 1 << 10
    # up to four ranks: the configured tile, whatever the share per CTA
    for ws in (2, 3, 4):
        for units in (1, 10_000, 2_000_000):
            assert native._mover_tile_bytes(units, 64, MiB, ws) == MiB
            assert native._mover_tile_bytes(units, 64, 0, ws) == 128 * KiB
    # more ranks: a share below two tiles per CTA is cut into about four tiles of at least 64 KiB
    units = (32 * MiB) // 16                     # 32 MiB block on 64 CTAs = 512 KiB per CTA
    assert native._mover_tile_bytes(units, 64, MiB, 8) == 128 * KiB
    assert native._mover_tile_bytes(units // 16, 64, MiB, 8) == 64 * KiB      # small share: the floor
    assert native._mover_tile_bytes(units * 8, 64, MiB, 8) == MiB             # 4 MiB per CTA: the configured tile
    # whatever the tile, the plan stays a partition with tile g owned by CTA g % nctas
    for ws in (5, 8):
        for u in (4097, 300_000, 2_400_000):
            tb = native._mover_tile_bytes(u, 64, MiB, ws)
            tu, nt = native._tile_plan(u, 64, 512, tb)
            assert tu > 0 and (nt - 1) * tu < u <= nt * tu
