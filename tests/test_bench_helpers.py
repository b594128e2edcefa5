"""Host-side arithmetic of bench.py (CPU only): the byte counts its rooflines divide by."""
import importlib.util
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_masked_softmax_byte_counts():
    """Row g keeps g % cols + 1 columns: the necessary bytes are the kept columns read plus
    every output written; a row offset shifts the saw-tooth; the algorithmic count is the whole
    tensor read and written."""
    bench = _bench()
    rows, cols = bench.ROWS, bench.COLS
    assert bench.SOFTMAX_BYTES == 2 * rows * cols * 2 == 262_144_000
    kept = sum(g % cols + 1 for g in range(rows))
    assert bench.softmax_necessary_bytes() == kept * 2 + rows * cols * 2 == 195_235_840
    shifted = sum((g + 12345) % cols + 1 for g in range(64))
    assert bench.softmax_necessary_bytes(64, cols, 12345) == shifted * 2 + 64 * cols * 2
    assert bench.softmax_necessary_bytes(3, 8) == (1 + 2 + 3) * 2 + 3 * 8 * 2


def test_roofline_fractions():
    bench = _bench()
    peaks = {"hbm_gbs": 6535.1, "bf16_tflops": 1646.2, "bf16_tflops_sustained": 1375.0}
    line = bench.roofline("hbm", 262_144_000, 0.04, peaks, "measured", 197_000_000)
    assert np.isclose(line["achieved"], 6553.6) and np.isclose(line["frac"], 6553.6 / 6535.1, atol=1e-4)
    assert line["peak_source"] == "of measured" and line["traffic"] == 197_000_000
    burst = bench.roofline("tensor", 2 * 8192 ** 3, 0.75, peaks, "measured", None)
    held = bench.roofline("tensor", 2 * 8192 ** 3, 0.75, peaks, "measured", None, sustained=True)
    assert burst["peak_kind"] == "burst" and held["peak_kind"] == "sustained"
    assert np.isclose(burst["achieved"], 2 * 8192 ** 3 / 0.75e-3 / 1e12, atol=0.01)
    assert held["frac"] > burst["frac"]


def test_headline_config_is_shared_by_both_arms():
    """The reference arm and the GPU arm print the same config (the driver compares them)."""
    bench = _bench()
    first, second = bench.headline_config(), bench.headline_config()
    assert first == second and "workload" in first and "model" not in first
