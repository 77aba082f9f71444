"""Host-side pieces of bench.py that need no GPU."""
import datetime
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402


SAMPLES = """\
2026/11/25 10:00:00.100, 1965, 1965, 300.5, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active
2026/11/25 10:00:00.150, 1920, 1965, 910.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active
2026/11/25 10:00:00.200, 1905, 1965, 990.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active
garbage line
2026/11/25 10:00:00.250, 1500, 1965, 990.0, 0x0000000000000040, Not Active, Active, Not Active, Not Active
"""


def test_clock_samples_inside_the_timed_region():
    s = bench.ClockSampler(0)
    rows = s.parse(SAMPLES)
    assert len(rows) == 4 and rows[1][3] == ["sw_power_cap"]
    s.started = datetime.datetime(2026, 11, 25, 10, 0, 0, 0)
    s.begin = datetime.datetime(2026, 11, 25, 10, 0, 0, 140000)
    s.end = datetime.datetime(2026, 11, 25, 10, 0, 0, 210000)
    out = s.summarise(rows)
    assert out["samples"] == 2 and out["sm_mhz"] == 1912.5 and out["reasons"] == ["sw_power_cap"]
    assert out["window"] == "timed region" and out["sm_max_mhz"] == 1965


def test_clock_samples_fall_back_to_the_warm_up_window():
    s = bench.ClockSampler(0)
    rows = s.parse(SAMPLES)
    s.started = datetime.datetime(2026, 11, 25, 10, 0, 0, 120000)
    s.begin = datetime.datetime(2026, 11, 25, 10, 0, 0, 160000)      # a region between two samples
    s.end = datetime.datetime(2026, 11, 25, 10, 0, 0, 190000)
    out = s.summarise(rows)
    assert out["samples"] == 3 and out["window"].startswith("warm-up")
    assert "hw_thermal_slowdown" in out["reasons"]
