"""The clock sampler of bench.py keeps only the nvidia-smi samples taken inside the measured load window."""
import datetime
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import bench  # noqa: E402


class _Done:
    def terminate(self):
        pass

    def wait(self, timeout=None):
        return 0

    def kill(self):
        pass


def _stamp(t):
    return datetime.datetime.fromtimestamp(t).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]


def test_timestamps_parse_and_window_selects_the_samples_under_load():
    t0 = 1_700_000_000.0
    assert abs(bench.ClockSampler._when(_stamp(t0 + 0.25)) - (t0 + 0.25)) < 2e-3
    assert bench.ClockSampler._when("not a time") is None
    s = bench.ClockSampler(0)
    s.proc = _Done()
    rows = [
        (t0 + 0.00, 1965, 1965, 180.0, "Not Active", "Not Active"),   # idle, before the window
        (t0 + 0.10, 1800, 1965, 900.0, "Not Active", "Active"),       # under load
        (t0 + 0.12, 1600, 1965, 1001.0, "Not Active", "Active"),
        (t0 + 0.14, 1700, 1965, 950.0, "Not Active", "Active"),
        (t0 + 0.50, 1965, 1965, 200.0, "Not Active", "Not Active"),   # after the window
    ]
    for t, sm, mx, pw, thermal, cap in rows:
        s.file.write(f"{_stamp(t)}, {sm}, {mx}, {pw}, 0x4, Not Active, {thermal}, Not Active, {cap}\n")
    s.file.flush()
    out = s.stop(window=(t0 + 0.05, t0 + 0.20))
    assert out["samples"] == 3 and out["sm_mhz"] == 1700.0 and out["sm_max_mhz"] == 1965.0
    assert out["power_w_max"] == 1001.0 and out["reasons"] == ["sw_power_cap"]


def test_no_window_keeps_every_sample_and_short_rows_are_skipped():
    s = bench.ClockSampler(0)
    s.proc = _Done()
    s.file.write("garbage line\n")
    s.file.write(f"{_stamp(1_700_000_000.0)}, 1500, 1965, 500.0, 0x0, Not Active, Active, Not Active, Not Active\n")
    s.file.flush()
    out = s.stop()
    assert out["samples"] == 1 and out["reasons"] == ["hw_thermal_slowdown"]
