"""The benchmark lane: workload entries, size rules and the measuring protocol (CPU), and one
entry per family through the protocol on the GPU."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest

import golden_cases
from compiler_b200 import lane
from compiler_b200.registry import default_registry

FIXTURE = json.loads((Path(__file__).parent / "golden" / "lane_fixture.json").read_text())
WORKLOAD = lane.load_workload()
ENTRIES = {entry["id"]: entry for entry in WORKLOAD["entries"]}


def test_workload_entries_have_the_fields_the_runner_reads():
    assert set(ENTRIES) == set(FIXTURE)
    for entry in WORKLOAD["entries"]:
        for key in ("id", "operator", "class", "family", "pattern", "dtype", "declared_shape",
                    "scale", "bytes_model"):
            assert key in entry, (entry["id"], key)
        assert entry["class"] in ("memory", "reduction", "compute")
        assert entry["operator"] == f"suite/perf/{entry['id']}.py"
        # the operator file declares this dtype (recorded from the reference's module)
        assert entry["dtype"] in FIXTURE[entry["id"]]["declared_dtypes"]


@pytest.mark.parametrize("entry_id", sorted(ENTRIES))
def test_size_rules_agree_with_the_reference(entry_id):
    """``resolve_shape`` against the shapes the reference's size.py gave for the same entry."""
    for llc, shape in FIXTURE[entry_id]["shapes"].items():
        assert lane.resolve_shape(ENTRIES[entry_id], int(llc), 8, WORKLOAD["dtype"]) == shape


@pytest.mark.parametrize("entry_id", sorted(ENTRIES))
def test_every_lane_kernel_has_a_native_operator(entry_id):
    info = FIXTURE[entry_id]
    handle = golden_cases.make_handle(info["kernel_name"], info["parameters"], info["autotuned"])
    assert default_registry().supports(handle)


def test_stop_rule_and_summary():
    # fixed count
    assert not lane.enough([1.0] * 4, samples=5)
    assert lane.enough([1.0] * 5, samples=5)
    # slow kernel: the time budget is reached at once, the floor still holds
    assert not lane.enough([0.5] * 9, min_time_s=0.2)
    assert lane.enough([0.5] * 10, min_time_s=0.2)
    # fast kernel: runs to min_samples, never past max_samples
    assert not lane.enough([1e-6] * 49)
    assert lane.enough([1e-6] * 50)
    assert lane.enough([1e-9] * 20, min_samples=100, max_samples=20)
    summary = lane.summarize([1.0, 2.0, 3.0, 10.0])
    assert summary["kernel_s"] == 2.5 and summary["mean_s"] == 4.0
    assert summary["n_samples"] == 4 and not summary["steady"]
    assert lane.summarize([2.0, 2.0], "mean")["steady"]
    assert summary["p10_s"] == 1.0 and summary["p90_s"] == 10.0


class _FakeDevice:
    """Runs a python stand-in for the kernel on the host arrays; counts launches."""

    def __init__(self, body):
        self.body, self.launches, self.released = body, 0, 0

    def upload(self, array, dtype=None):
        return np.array(array, copy=True)

    def download(self, buffer):
        return np.asarray(buffer)

    def synchronize(self):
        pass

    def launch(self, kernel, grid, positional, keywords):
        self.launches += 1
        self.body(*positional)

    def release(self, buffers):
        self.released += 1


def _copy_case(scale=1.0):
    x = np.arange(8, dtype=np.float32)
    kernel = golden_cases.make_handle("copy_kernel", ["x_ptr", "y_ptr", "n"])
    return {"kernel": kernel, "args": {"x_ptr": x, "y_ptr": np.full(8, 7.0, np.float32), "n": 8},
            "grid": (1,), "inputs": ("x_ptr",), "outputs": ("y_ptr",),
            "expected": {"y_ptr": x * scale},
            "comparison": {"y_ptr": {"rtol": 1e-6, "atol": 1e-6}}}


def test_run_entry_records_pass_mismatch_and_launch_failure():
    def copy(x, y, n):
        y[:n] = x[:n]

    device = _FakeDevice(copy)
    record = lane.run_entry({"id": "copy"}, _copy_case(), device, samples=12)
    assert record["status"] == "PASS" and record["verified"] and record["n_samples"] == 12
    assert record["timer"] == "host" and record["max_abs_error"] == 0.0
    assert device.launches == 1 + 3 + 12 and device.released == 1   # first + warm-ups + samples

    # a kernel that does not write fails verification: the output buffer was zeroed first
    idle = _FakeDevice(lambda x, y, n: None)
    record = lane.run_entry({"id": "copy"}, _copy_case(), idle, samples=12)
    assert record["status"] == "MISMATCH" and "n_samples" not in record

    wrong = lane.run_entry({"id": "copy"}, _copy_case(scale=2.0), _FakeDevice(copy), samples=12)
    assert wrong["status"] == "MISMATCH"

    def broken(x, y, n):
        raise RuntimeError("no such operator")

    record = lane.run_entry({"id": "copy"}, _copy_case(), _FakeDevice(broken), samples=12)
    assert record["status"] == "LAUNCH_FAIL" and "no such operator" in record["error"]

    unverified = lane.run_entry({"id": "copy"}, _copy_case(scale=2.0), _FakeDevice(copy),
                                do_verify=False, samples=10)
    assert unverified["status"] == "PASS" and unverified["verified"] is False


def test_cli_lists_shapes_without_a_corpus(capsys):
    assert lane.main(["--list", "--llc-bytes", str(126 << 20), "--only", "softmax"]) == 0
    out = capsys.readouterr().out
    assert "softmax" in out and "[66060, 4000]" in out


# --------------------------------------------------------------------------- GPU
def _grown(tag, arrays, scalars, meta, grid, expected):
    """A golden case of the operator, with its arrays and scalars swapped for larger ones:
    kernel handle, outputs, pointer dtypes and comparison policy stay the reference's."""
    case, _ = golden_cases.load(tag)
    case = dict(case)
    case["args"] = {**{k: v for k, v in case["args"].items() if not isinstance(v, np.ndarray)},
                    **scalars, **arrays}
    case["meta"] = {**case.get("meta", {}), **meta}
    case["grid"] = grid
    case["expected"] = expected
    case["inputs"] = tuple(name for name in arrays if name not in case["outputs"])
    return case


def _lane_cases():
    from oracle import oracle
    rng = np.random.default_rng(2026)

    def bf16(a):
        return oracle.bf16_round(a.astype(np.float32))

    rows, cols = 4096, 4096
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    w = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    y_ref, r_ref = oracle.rmsnorm_ref(x, w, 1e-5)
    yield "fast_rms_layernorm", _grown(
        "fast_rms_layernorm__4x64__float32",
        {"X": x, "W": w, "Y": np.empty_like(x), "r": np.empty(rows, np.float32)},
        {"X_row_stride": cols, "Y_row_stride": cols, "n_cols": cols, "eps": 1e-5},
        {"BLOCK_SIZE": cols}, (rows,),
        {"Y": y_ref.astype(np.float32), "r": r_ref.astype(np.float32)}), 2 * x.nbytes

    rows, cols = 8192, 4000
    x = (rng.standard_normal((rows, cols), dtype=np.float32) * 2).astype(np.float16)
    yield "softmax", _grown(
        "softmax__4x16__float16", {"x_ptr": x, "y_ptr": np.empty_like(x)}, {"n_cols": cols},
        {"BLOCK_N": 4096}, (rows,),
        {"y_ptr": oracle.softmax_ref(x.astype(np.float64)).astype(np.float32)}), 2 * x.nbytes

    n = 1024
    a = bf16(rng.standard_normal((n, n)) / 32)
    b = bf16(rng.standard_normal((n, n)) / 32)
    yield "matmul", _grown(
        "matmul__16x16x16__bfloat16", {"a_ptr": a, "b_ptr": b, "y_ptr": np.empty_like(a)},
        {"M": n, "N": n, "K": n}, {}, (n // 16, n // 16),
        {"y_ptr": oracle.matmul_ref(a, b).astype(np.float32)}), 2 * n ** 3

    z, h, n, d = 1, 4, 1024, 128
    q, k, v = (bf16(rng.standard_normal((z, h, n, d))) for _ in range(3))
    scale = 1.0 / np.sqrt(d)
    strides = {}
    for t, (sz, sh, sm, sk) in {"q": "zhmk", "k": "zhnk", "v": "zhkn", "o": "zhmn"}.items():
        strides.update({f"stride_{t}{sz}": h * n * d, f"stride_{t}{sh}": n * d,
                        f"stride_{t}{sm}": d, f"stride_{t}{sk}": 1})
    out_ref = oracle.attention_ref(q, k, v, scale, causal=True)
    out_ref = out_ref[0] if isinstance(out_ref, tuple) else out_ref
    yield "attn_fwd_causal", _grown(
        "attn_fwd_causal__2x2x16x32__bfloat16",
        {"q_ptr": q, "k_ptr": k, "v_ptr": v, "out_ptr": np.empty_like(q)},
        {"Z": z, "H": h, "N_CTX": n, "scale": float(scale), **strides},
        {"HEAD_DIM": d, "BLOCK_N": 64, "CAUSAL": True}, (n, z * h),
        {"out_ptr": np.asarray(out_ref, dtype=np.float32)}), 4 * z * h * d * n * (n + 1) // 2

    rows, cols = 2048, 11008
    x = bf16(rng.standard_normal((rows, cols)))
    y = bf16(rng.standard_normal((rows, cols)))
    yield "swiglu_fwd", _grown(
        "swiglu_fwd__4x64__bfloat16", {"X": x, "Y": y, "OUT": np.empty_like(x)},
        {"stride_x_row": cols, "stride_y_row": cols, "stride_out_row": cols, "ncols": cols}, {},
        (rows, cols // 32), {"OUT": oracle.swiglu_ref(x, y).astype(np.float32)}), 3 * rows * cols * 2


@pytest.mark.gpu
def test_lane_protocol_on_the_device(device):
    """One entry per family at a shape the oracle finishes in seconds: verified against the
    oracle under the reference's policy, then timed by the lane's sampler on device events."""
    print()
    for entry_id, case, work in _lane_cases():
        entry = ENTRIES[entry_id]
        record = lane.run_entry({"id": entry_id, "class": entry["class"]}, case, device,
                                min_samples=30, min_time_s=0.05)
        assert record["status"] == "PASS", (entry_id, record.get("error"))
        assert record["verified"] and record["timer"] == "device"
        assert record["n_samples"] >= lane.MIN_SAMPLES_FLOOR and record["kernel_s"] > 0
        rate = work / record["kernel_s"]
        unit = "TFLOP/s" if entry["class"] == "compute" else "GB/s"
        print(f"lane {entry['class']:9s} {entry_id:20s} kernel={record['kernel_s'] * 1e6:9.1f} us "
              f"n={record['n_samples']:3d} cov={record['cov']:.3f} "
              f"{rate / (1e12 if unit == 'TFLOP/s' else 1e9):8.1f} {unit} "
              f"max_abs_error={record['max_abs_error']:.2e}")
