"""The tuning tool's threshold rules on rows measured on 8 and 4 B200 (microseconds per call)."""
from mccl_b200.bench.busbw import nvls_floor, oneshot_ceiling

# (bytes, one-shot, two-shot, NVLS); None = not measured at that size
WS8_FP32 = [
    (16384, 20.1, 45.08, 30.7),
    (32768, 21.47, 45.2, 31.01),
    (65536, 21.14, 46.75, 31.39),
    (131072, 24.6, 50.12, 33.58),
    (262144, 23.05, 58.64, 37.22),
    (524288, 29.47, 60.04, 40.09),
    (1048576, 31.91, 63.96, 43.21),
    (2097152, 49.78, 71.54, 48.86),
    (4194304, 71.92, 71.21, 53.22),
    (8388608, 125.47, 77.55, 63.38),
    (16777216, 236.28, 89.5, 88.77),
    (33554432, None, 143.57, 134.83),
    (67108864, None, 253.6, 224.55),
    (134217728, None, 441.23, 412.94),
]
WS8_BF16 = [
    (16384, 23.1, 45.23, 33.63),
    (32768, 21.14, 45.52, 30.86),
    (65536, 20.71, 47.23, 31.46),
    (131072, 21.55, 50.73, 33.33),
    (262144, 22.95, 60.63, 36.74),
    (524288, 26.37, 61.72, 38.82),
    (1048576, 31.87, 65.93, 41.87),
    (2097152, 46.86, 71.39, 48.84),
    (4194304, 75.48, 72.87, 52.22),
    (8388608, 126.91, 78.59, 82.29),
    (16777216, 238.06, 91.31, 88.94),
    (33554432, None, 147.52, 134.61),
    (67108864, None, 262.68, 222.73),
    (134217728, None, 441.59, 412.35),
]
WS4_FP32 = [
    (16384, 20.12, 31.44, 25.15),
    (32768, 24.66, 32.04, 26.24),
    (65536, 20.35, 34.25, 27.27),
    (131072, 19.56, 37.69, 29.7),
    (262144, 19.76, 39.94, 32.06),
    (524288, 19.97, 42.98, 34.42),
    (1048576, 23.49, 45.19, 36.19),
    (2097152, 30.76, 49.39, 40.72),
    (4194304, 42.23, 51.35, 46.46),
    (8388608, 64.22, 55.65, 59.37),
    (16777216, 108.66, 80.94, 82.93),
    (33554432, 206.66, 132.08, 129.83),
    (67108864, None, 237.02, 220.22),
    (134217728, None, 390.91, 408.29),
    (268435456, None, 775.87, 795.9),
]


def _table(rows):
    sizes, t_all = [], {}
    for size, one, two, nvls in rows:
        sizes.append(size)
        t_all[size] = {k: v for k, v in (("oneshot", one), ("twoshot", two), ("nvls", nvls)) if v is not None}
    return sizes, t_all


def test_eight_ranks_fp32_one_shot_to_1_mib_then_nvls():
    sizes, t = _table(WS8_FP32)
    one = oneshot_ceiling(sizes, t)
    assert one == 1 << 20
    assert nvls_floor(sizes, t, one) == 2 << 20


def test_one_noisy_row_does_not_move_the_nvls_floor():
    # bf16 at 8 ranks: NVLS wins from 4 MiB up except for one row (8 MiB: 82.3 against 78.6 us)
    sizes, t = _table(WS8_BF16)
    one = oneshot_ceiling(sizes, t)
    assert one == 2 << 20
    assert nvls_floor(sizes, t, one) == 4 << 20
    # two lost rows do move it
    t[16 << 20]["nvls"] = t[16 << 20]["twoshot"] + 5.0
    assert nvls_floor(sizes, t, one) == 32 << 20


def test_four_ranks_fp32_nvls_never_pays_consistently():
    sizes, t = _table(WS4_FP32)
    one = oneshot_ceiling(sizes, t)
    assert one == 4 << 20
    floor = nvls_floor(sizes, t, one)
    # NVLS and two-shot trade places above 8 MiB at 4 ranks: whatever floor comes out, it is not below 32 MiB
    assert floor == -1 or floor >= 32 << 20


def test_cold_first_row_does_not_zero_the_one_shot_ceiling():
    sizes, t = _table(WS8_FP32)
    t[sizes[0]]["oneshot"] = 99.0     # a first row that still contains one-time setup
    assert oneshot_ceiling(sizes, t) == 1 << 20
