"""The launch surface driven by the reference's REAL objects (CPU only).

When the reference tree is present (``REFERENCE_ROOT``, or next to this repository) every
operator file the golden fixtures come from is loaded with the reference's own
``opslib.runner.load_operator``; its ``make_case`` builds the case with the real
``triton.JITFunction`` / ``Autotuner`` as ``case["kernel"]``; and the reference's own
``opslib.device.stage_case`` + ``StagedCase.launch``
(ops/harness/opslib/device.py:323-415, with ``_device_upload``'s signature probe and
``patch_pointer_tables``) drive ``B200Device``.  The C library is replaced by a recording fake
whose "device memory" is host memory, so no GPU is needed and nothing is computed: the test
asserts that the registry resolves the real kernel objects, which entry point each launch
reaches, and that the descriptors (shapes, strides, dtype codes, scalars) are the ones the
signature-only stand-in handles of ``tests/golden_cases.py`` produce through this
repository's own ``harness.stage_case``.
"""
import ctypes
import os
import sys
from pathlib import Path

import numpy as np
import pytest

import golden_cases
from compiler_b200 import harness
from compiler_b200.runtime import abi

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
from make_golden import OPERATORS  # noqa: E402


def _reference_root():
    base = os.environ.get("REFERENCE_ROOT") or str(Path(__file__).resolve().parents[2] / "reference")
    root = Path(base)
    return root if (root / "ops" / "harness" / "opslib").is_dir() else None


class FakeLibrary:
    """Stands in for libb200ops.so: allocations and copies work on host memory, every
    operator entry point is recorded with decoded arguments and returns B200_OK."""

    PLUMBING = {"b200_set_device", "b200_stream_sync", "b200_device_sync", "b200_memset",
                "b200_last_device_status"}

    def __init__(self):
        self.calls = []
        self._blocks = {}

    # ---- memory -----------------------------------------------------------------
    def b200_malloc(self, out, nbytes):
        block = ctypes.create_string_buffer(max(int(nbytes), 1) + 64)
        address = (ctypes.addressof(block) + 63) & ~63
        self._blocks[address] = block
        out._obj.value = address
        return abi.OK

    b200_malloc_host = b200_malloc

    def b200_free(self, ptr):
        self._blocks.pop(int(getattr(ptr, "value", ptr) or 0), None)
        return abi.OK

    b200_free_host = b200_free

    def _copy(self, dst, src, nbytes, stream):
        ctypes.memmove(int(getattr(dst, "value", dst)), int(getattr(src, "value", src)),
                       int(nbytes))
        return abi.OK

    b200_memcpy_h2d = b200_memcpy_d2h = b200_memcpy_d2d = _copy

    def b200_status_string(self, status):
        return b"fake"

    def b200_device_query(self, device, props):
        out = props._obj
        out.name, out.sm_count, out.l2_bytes, out.hbm_bytes = b"fake", 148, 1 << 20, 1 << 34
        out.cc_major, out.cc_minor = 10, 0
        return abi.OK

    def b200_event_create(self, out):
        out._obj.value = 1
        return abi.OK

    def b200_event_elapsed_ms(self, start, stop, ms):
        ms._obj.value = 0.01
        return abi.OK

    def b200_last_error(self):
        return b""

    # ---- everything else --------------------------------------------------------
    @staticmethod
    def _decode(arg):
        target = getattr(arg, "_obj", None)        # ctypes.byref(...)
        if isinstance(target, abi.Tensor):
            n = int(target.ndim)
            return ("tensor", tuple(target.shape[:n]), tuple(target.stride[:n]),
                    int(target.dtype))
        if target is not None:
            return ("out",)
        if arg is None:
            return None
        if isinstance(arg, float):
            return round(arg, 9)
        return arg

    def __getattr__(self, name):
        if not name.startswith("b200_"):
            raise AttributeError(name)

        def call(*args):
            if name not in self.PLUMBING:
                # the trailing argument is the stream; data pointers are not compared
                self.calls.append((name, tuple(self._decode(a) for a in args[:-1])))
            return abi.OK
        return call


@pytest.fixture()
def fake_library(monkeypatch):
    fake = FakeLibrary()
    monkeypatch.setattr(abi, "_lib", fake)
    return fake


def _reference_modules():
    root = _reference_root()
    if root is None:
        pytest.skip("reference tree not present on this host")
    harness_dir = str(root / "ops" / "harness")
    if harness_dir not in sys.path:
        sys.path.insert(0, harness_dir)
    from opslib import device as ref_device, runner
    return root, ref_device, runner


def _tags_of(rel):
    stem = Path(rel).stem
    return [t for t, info in golden_cases.INDEX.items() if info["operator"] == rel
            and t.startswith(stem + "__")]


@pytest.mark.parametrize("rel", sorted(OPERATORS))
def test_reference_stage_case_drives_the_device(rel, fake_library):
    root, ref_device, runner = _reference_modules()
    from compiler_b200.device import B200Device
    module = runner.load_operator(root / "ops" / "suite" / rel)
    tags = _tags_of(rel)
    assert tags, f"no golden fixtures for {rel}"
    checked = 0
    for tag in tags:
        info = golden_cases.INDEX[tag]
        if tuple(info["shape"]) not in {tuple(s) for s in module.SHAPES}:
            continue  # audited mid-size shapes: same code path, skipped for time
        real = module.make_case(shape=tuple(info["shape"]), dtype=info["dtype"])
        # (1) the real kernel object resolves, by name and parameter list
        device = B200Device(0)
        assert device.registry.supports(real["kernel"]), tag
        # (2) the reference's own staging + launch reach the library
        fake_library.calls.clear()
        staged = ref_device.stage_case(real, device)
        staged.launch()
        through_reference = list(fake_library.calls)
        assert through_reference, tag
        # (3) ... with the descriptors the stand-in handle produces through this repo's harness
        stand_in, _ = golden_cases.load(tag)
        device2 = B200Device(0)
        fake_library.calls.clear()
        harness.stage_case(stand_in, device2).launch()
        assert through_reference == list(fake_library.calls), tag
        # outputs come back with the host dtype and shape the reference expects
        for name in real["outputs"]:
            out = staged.outputs()[name]
            assert out.shape == np.asarray(real["expected"][name]).shape
        checked += 1
    assert checked


def test_reference_make_device_builds_this_device(fake_library):
    _, ref_device, _ = _reference_modules()
    device = ref_device.make_device("compiler_b200.device:make_device")
    assert type(device).__name__ == "B200Device" and device.name == "b200-native"
    # the protocol surface the reference's runner and benchmark lane call
    for method in ("alloc", "upload", "download", "pointer", "synchronize", "launch",
                   "upload_aliased", "compare", "timer", "properties", "release"):
        assert callable(getattr(device, method)), method


def test_lane_with_the_corpus_stages_through_the_reference(fake_library, tmp_path, monkeypatch):
    """``python -m compiler_b200.lane --corpus ...``: an entry of the workload file is built by
    the corpus's own loader and staged and launched by the corpus's own
    ``opslib.device.stage_case`` (not this package's stand-in) on ``B200Device``; with the
    recording library every entry must bind, launch and be sampled.  Three entries here (all
    twenty-odd pass the same way; the case builders' float64 oracles take minutes)."""
    import json
    root, _, _ = _reference_modules()
    from compiler_b200 import lane
    monkeypatch.setattr(lane, "_stage_case", lane._stage_case)   # main() swaps it: put it back
    code = lane.main(["--corpus", str(root / "ops"), "--out-dir", str(tmp_path), "--no-verify",
                      "--multiple", "1", "--min-samples", "3", "--samples", "3", "--only",
                      "fast_rms_layernorm,softmax,swiglu_fwd"])
    assert lane._stage_case.__module__ == "opslib.device"
    report = json.loads((tmp_path / "BENCH_REPORT.json").read_text())
    failed = [(e["id"], e.get("error")) for e in report["entries"] if e["status"] != "PASS"]
    assert code == 0 and not failed, failed
    assert len(report["entries"]) == 3 and fake_library.calls
