"""Host-side pieces of the benchmark harness that need no GPU: the clock sampler's window logic and the roofline
denominators."""
import importlib.util
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


class _Done:
    def terminate(self):
        pass

    def wait(self, timeout=None):
        pass


LINE_IDLE = "1200, 1965, 310.5, Not Active, Not Active, Not Active, Not Active\n"
LINE_LOAD = "1890, 1965, 960.1, Not Active, Not Active, Not Active, Active\n"
LINE_HOT = "1500, 1965, 900.0, Not Active, Active, Not Active, Active\n"


def test_clock_sampler_summarises_only_the_marked_window():
    bench = _load("bench_under_test", os.path.join(ROOT, "bench.py"))
    s = bench.ClockSampler(0)
    s.proc = _Done()
    with open(s.path, "w") as f:
        f.write(LINE_IDLE * 4 + LINE_LOAD * 3)
    s.first_line = 4                                  # what mark() records: lines written before the timed region
    out = s.stop()
    assert out["samples"] == 3 and out["sm_mhz"] == 1890.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"]
    assert not os.path.exists(s.path)


def test_clock_sampler_falls_back_to_the_last_lines_before_a_too_short_window():
    bench = _load("bench_under_test2", os.path.join(ROOT, "bench.py"))
    s = bench.ClockSampler(0)
    s.proc = _Done()
    with open(s.path, "w") as f:
        f.write(LINE_IDLE * 2 + LINE_HOT * 3)
    s.first_line = 5                                  # nothing was written inside the window
    out = s.stop()
    assert out["samples"] == 3 and out["sm_mhz"] == 1500.0
    assert out["reasons"] == ["hw_thermal_slowdown", "sw_power_cap"]


def test_clock_sampler_without_nvidia_smi_says_so():
    bench = _load("bench_under_test3", os.path.join(ROOT, "bench.py"))
    s = bench.ClockSampler(0)
    out = s.stop()                                    # never started
    assert out["sm_mhz"] is None and "unavailable" in out["reasons"][0]


def test_roofline_denominators_come_from_the_measured_peaks_file():
    fp = _load("fused_paths_under_test", os.path.join(ROOT, "benchmarks", "fused_paths_bench.py"))
    tf, link = fp.peaks()
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        want = float(json.load(open(path)).get("bf16_tflops_sustained", 1393.0)) * 1e12
        assert abs(tf - want) < 1e6
    else:
        assert tf == 1393e12
    assert link == 770e9
