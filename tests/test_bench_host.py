"""The benchmark's host arithmetic without a GPU: the algorithmic byte count the roofline is computed
from, the synthetic lengths, the bf16 rounding of the synthetic inputs, and what the clock sampler
reports for timed regions longer and shorter than its sampling period."""
import numpy as np

import bench
from oracle import oracle


def test_algorithmic_bytes_per_sequence_layer_and_step():
    # K and V of every visible key (2 x 64 x 2 bytes per key and KV head, 8 heads), q in and out
    # (64 heads x 64 x 2 bytes each), the new k and v read and written (2 x 8 x 64 x 2 bytes, twice)
    one = bench.algorithmic_bytes(np.array([4608]), 0)
    assert one == 2048 * 4608 + 8192 + 8192 + 4096
    assert bench.algorithmic_bytes(np.array([4608]), 128) == 2048 * 128 + 20480
    assert bench.algorithmic_bytes(np.array([100]), 128) == 2048 * 100 + 20480        # shorter than the window
    assert bench.algorithmic_bytes(np.array([4608]), 0, kv_heads=1) == one // 8       # one of the 8 KV heads
    lens = np.array([1024, 8192, 3000])
    assert bench.algorithmic_bytes(lens, 0) == sum(bench.algorithmic_bytes(np.array([l]), 0) for l in lens)


def test_synthetic_lengths_are_the_stated_draw():
    lens = bench.draw_lengths(32)
    assert np.array_equal(lens, np.random.default_rng(0).integers(1024, 8193, 32))
    assert lens.min() >= 1024 and lens.max() <= 8192
    assert np.array_equal(bench.draw_lengths(64)[:32], np.random.default_rng(0).integers(1024, 8193, 64)[:32])


def test_the_gpu_arm_rounds_its_inputs_as_the_oracle_does():
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(100000).astype(np.float32) * 3,
                        np.array([0.9567871, 1 + 2.0 ** -8, 1 + 3 * 2.0 ** -8, -0.0, 0.0, 65504.0, 1e-30], np.float32)])
    assert np.array_equal(bench.bf16_bits(x), oracle.f32_to_bf16_bits(x))
    assert np.array_equal(bench.bf16_to_f32(bench.bf16_bits(x)), oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(x)))


def _sampler(rows, t0, t1):
    s = bench.ClockSampler(0)
    s.rows, s.t0, s.t1 = rows, t0, t1
    return s.summary()


def test_clock_summary_uses_the_lines_inside_the_timed_region():
    idle = ["1200", "1965", "Not Active", "Not Active", "Not Active", "Not Active"]
    busy = ["1965", "1965", "Not Active", "Not Active", "Not Active", "Active"]
    rows = [(0.0, idle), (0.1, busy), (0.2, ["1950", "1965", "Not Active", "Not Active", "Not Active", "Not Active"]),
            (0.3, busy), (0.5, idle)]
    got = _sampler(rows, 0.05, 0.35)
    assert got["samples"] == 3 and got["sm_mhz"] == 1965.0 and got["sm_max_mhz"] == 1965.0
    assert got["reasons"] == ["sw_power_cap"] and got["sampled"] == "inside the timed region"


def test_clock_summary_of_a_region_shorter_than_the_sampling_period():
    a = ["1965", "1965", "Not Active", "Not Active", "Not Active", "Not Active"]
    b = ["1905", "1965", "Active", "Not Active", "Not Active", "Not Active"]
    got = _sampler([(0.00, a), (0.02, a), (0.04, b), (0.06, a)], 0.025, 0.035)
    assert got["samples"] == 2 and got["sm_mhz"] == 1935.0 and got["reasons"] == ["hw_slowdown"]
    assert "nearest" in got["sampled"]


def test_clock_summary_without_nvidia_smi_or_with_garbage_lines():
    assert _sampler([], 0.0, 1.0) == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    got = _sampler([(0.1, ["[N/A]", "1965", "x"]), (0.2, ["1800", "1965", "Not Active", "Not Active", "Not Active", "Not Active"])],
                   0.0, 1.0)
    assert got["samples"] == 1 and got["sm_mhz"] == 1800.0
