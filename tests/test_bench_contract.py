"""Host-side pieces of ``bench.py``: the workload table and the clock-sample parser (no GPU needed)."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_workload_table_has_the_four_benchmark_configs():
    want = {"131k-s32": (131072, 32, 256), "131k-s128": (131072, 128, 128), "1.3m": (1310720, 32, 512),
            "100m": (100_000_000, 32, 1024)}
    for name, (labels, seq, batch) in want.items():
        c = bench.CONFIGS[name]
        assert (c["labels"], c["seq"], c["batch"]) == (labels, seq, batch)
        assert c["batch"] % 8 == 0                      # divisible over 1, 2, 4 and 8 GPUs
    base = json.load(open(os.path.join(ROOT, "BASELINE.json")))
    assert "samples" in json.dumps(base).lower()        # the metric the JSON line reports


class _FakeProc:
    def __init__(self, text):
        self.text = text

    def terminate(self):
        pass

    def communicate(self, timeout=None):
        return self.text, ""


def test_clock_sampler_reports_median_clock_and_active_reasons():
    s = bench.ClockSampler(0)
    rows = ["0, 1965, 1965, 512.1, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active",
            "0, 1845, 1965, 998.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
            "0, 1800, 1965, 1001.3, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
            "garbage line"]
    s.proc = _FakeProc("\n".join(rows) + "\n")
    out = s.stop()
    assert out == {"sm_mhz": 1845.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    s2 = bench.ClockSampler(0)
    assert s2.stop()["reasons"] == ["nvidia-smi unavailable"]
