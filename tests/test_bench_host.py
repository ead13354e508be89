"""Host-side pieces of bench.py that need no GPU: the byte accounting, the CPU arm on a bounded sample, the clock
sampler's summary, and the reference arm's JSON line."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_algorithmic_bytes_of_the_step():
    assert bench.q4_weight_bytes(12288, 4096) == 28_311_552
    assert bench.q4_weight_bytes(4096, 4096) == 9_437_184
    assert bench.q4_weight_bytes(6144, 4096) == 14_155_776
    assert bench.STEP_WEIGHT_BYTES == 14_155_776 + 9_437_184 + 2 * 28_311_552 + 28_311_552 == 108_527_616


def test_the_cpu_step_runs_on_a_bounded_sample_and_counts_its_bytes(monkeypatch):
    # a small layer with the real generator and the real oracle: shrink the dimensions, keep the code path
    monkeypatch.setattr(bench, "HIDDEN", 256)
    monkeypatch.setattr(bench, "QKV", 384)
    monkeypatch.setattr(bench, "INTER", 512)
    banks, xs = bench.cpu_step_inputs(0x1234)
    y_full, done_full = bench.cpu_step(banks, xs, 2, 1.0)
    assert y_full.shape == (256,) and np.all(np.isfinite(y_full))
    want = (bench.q4_weight_bytes(384, 256) + bench.q4_weight_bytes(256, 256) + 2 * bench.q4_weight_bytes(512, 256)
            + bench.q4_weight_bytes(256, 512))
    assert done_full == want
    _, done_part = bench.cpu_step(banks, xs, 2, 0.25)
    assert 0 < done_part < done_full
    # thread count does not change the result (rows are independent)
    y1, _ = bench.cpu_step(banks, xs, 1, 1.0)
    assert np.array_equal(y1, y_full)


def test_clock_summary_reports_unavailable_without_samples():
    class FakeTorch:
        class cuda:
            @staticmethod
            def get_device_properties(i):
                raise RuntimeError("no device")

    cs = bench.ClockSampler(FakeTorch, 0, enabled=False)
    s = cs.summary()
    assert s["samples"] == 0 and "unavailable" in s
    cs.rows = [["0", "1965", "1965", "400", "0x0", "Not Active", "Not Active", "Not Active", "Active"],
               ["0", "1905", "1965", "900", "0x4", "Not Active", "Not Active", "Not Active", "Not Active"], ["garbage"]]
    s = cs.summary()
    assert s["samples"] == 2 and s["sm_mhz"] == 1935.0 and s["sm_max_mhz"] == 1965.0 and s["reasons"] == ["sw_power_cap"]


def test_host_threads_is_explicit_and_positive(monkeypatch):
    monkeypatch.setenv("OMP_NUM_THREADS", "1")
    assert bench.host_threads() >= 1
