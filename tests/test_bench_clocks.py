"""Host logic of bench.py's clock record: nvidia-smi's csv lines are parsed with their own timestamps and only the
samples inside the timed region count (those of the second before it when the region caught none)."""
import datetime
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import bench  # noqa: E402


def _line(t, sm, cap="Not Active", hw="Not Active"):
    ts = datetime.datetime.fromtimestamp(t).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    return f"{ts}, 0, {sm}, 1965, 412.30, 0x0000000000000004, {hw}, Not Active, Not Active, {cap}"


def test_samples_inside_the_timed_region_are_kept():
    t0 = 1_800_000_000.0
    text = "\n".join([_line(t0 - 0.9, 1200), _line(t0 - 0.1, 1500), _line(t0 + 0.05, 1950, cap="Active"),
                      _line(t0 + 0.15, 1965), _line(t0 + 0.25, 1965), _line(t0 + 0.9, 300)])
    rows = bench.ClockSampler.parse(text)
    assert len(rows) == 6
    out = bench.ClockSampler.summarise(rows, t0, t0 + 0.3)
    assert out["samples"] == 3 and out["sm_mhz"] == 1965 and out["sm_max_mhz"] == 1965
    assert out["reasons"] == ["sw_power_cap"] and out["window"] == "timed region"


def test_short_region_falls_back_to_the_preceding_second_and_says_so():
    t0 = 1_800_000_000.0
    text = "\n".join([_line(t0 - 5.0, 300), _line(t0 - 0.6, 1900, hw="Active"), _line(t0 - 0.2, 1960)])
    out = bench.ClockSampler.summarise(bench.ClockSampler.parse(text), t0, t0 + 0.01)
    assert out["samples"] == 2 and out["sm_mhz"] == 1930 and out["reasons"] == ["hw_slowdown"]
    assert out["window"].startswith("timed region held no sample")


def test_no_output_gives_an_empty_record():
    out = bench.ClockSampler.summarise(bench.ClockSampler.parse("garbage\n"), 0.0, 1.0)
    assert out == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
