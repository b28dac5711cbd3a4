"""Host-side pieces of bench.py that need no GPU: the clock-sample parser and the launch counts."""
import datetime
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bench  # noqa: E402


class _Done:
    """Stands in for a finished nvidia-smi process."""

    def terminate(self):
        pass

    def wait(self, timeout=None):
        return 0

    def kill(self):
        pass


class _Joined:
    def join(self, timeout=None):
        pass


def _line(ts, sm, reasons=("Not Active",) * 4):
    stamp = datetime.datetime.fromtimestamp(ts).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    return ", ".join([stamp, str(sm), "1965", "700.0", "0x0000000000000004", *reasons]) + "\n"


def _sampler(lines):
    s = bench.ClockSampler(0)
    s.proc, s.reader, s.lines = _Done(), _Joined(), list(lines)
    return s


def test_clock_samples_outside_the_window_are_dropped():
    now = time.time()
    lines = [_line(now - 5.0, 300), _line(now + 0.10, 1500), _line(now + 0.20, 1600), _line(now + 0.30, 1700),
             _line(now + 9.0, 200), "garbage line\n"]
    out = _sampler(lines).stop((now, now + 0.5))
    assert out["samples"] == 3
    assert out["sm_mhz"] == 1600 and out["sm_max_mhz"] == 1965
    assert out["reasons"] == []


def test_clock_sample_reasons_are_collected():
    now = time.time()
    lines = [_line(now + 0.1, 1400, ("Not Active", "Not Active", "Not Active", "Active")),
             _line(now + 0.2, 1300, ("Not Active", "Active", "Not Active", "Active"))]
    out = _sampler(lines).stop((now, now + 1.0))
    assert out["reasons"] == ["hw_thermal_slowdown", "sw_power_cap"]
    assert out["samples"] == 2


def test_no_samples_is_reported_as_such():
    out = _sampler([]).stop((0.0, 1.0))
    assert out["sm_mhz"] is None and out["reasons"] == ["no samples"]
    s = bench.ClockSampler(0)          # nvidia-smi never started
    assert s.stop()["reasons"] == ["nvidia-smi unavailable"]


def test_launch_counts_cover_every_mode():
    for key in ("fwd", "fwd_fp32", "bwd", "train", "decode", "ep_fwd", "ep_bwd"):
        assert bench.LAUNCHES[key] > 0
    assert bench.LAUNCHES["train"] == bench.LAUNCHES["fwd"] + bench.LAUNCHES["bwd"]
    for name, w in bench.WORKLOADS.items():
        assert w["mode"] in ("fwd", "bwd", "train"), name
