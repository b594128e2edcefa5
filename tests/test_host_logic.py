"""Host-side logic that needs no GPU: partitioning, argument binding, the registry's
resolution rules, the compile protocol's identity and counters, staging through a fake
device (the pattern of ops/harness/tests/test_runner_contract.py:29-185)."""
import numpy as np
import pytest

import golden_cases
from compiler_b200 import harness, kernels, shard
from compiler_b200.factory import PlanOptions, make_compiler
from compiler_b200.registry import (UnsupportedLaunch, bind_by_name, default_registry,
                                    kernel_signature)


# ------------------------------------------------------------------ partition
@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("total", [0, 1, 7, 8, 256, 4097, 16384])
def test_block_partition_covers_exactly_once(total, world):
    shard.check_partition(total, world, shard.block_range)
    shard.check_partition(total, world, shard.strided_items)
    sizes = [hi - lo for lo, hi in (shard.block_range(total, r, world) for r in range(world))]
    assert max(sizes) - min(sizes) <= 1 and sum(sizes) == total


def test_partition_checker_can_fail():
    with pytest.raises(AssertionError):
        shard.check_partition(10, 2, lambda total, rank, world: (0, 6))  # overlap + hole
    with pytest.raises(ValueError):
        shard.block_range(10, 2, 2)


def test_column_range_keeps_tma_alignment():
    for world in (2, 4, 8):
        edges = [shard.column_range(14336, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == 14336
        assert all(lo % 8 == 0 and hi % 8 == 0 for lo, hi in edges)
        assert all(edges[i][1] == edges[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        shard.column_range(14337, 0, 2)


def test_row_chunks():
    assert shard.row_chunks(4096, 4) == [(0, 1024), (1024, 2048), (2048, 3072), (3072, 4096)]
    assert shard.row_chunks(3, 8) == [(0, 1), (1, 2), (2, 3)]
    assert sum(hi - lo for lo, hi in shard.row_chunks(4097, 4)) == 4097


# ------------------------------------------------------------------ binding
def test_bind_arguments_roundtrip_with_autotuned_kernel():
    case, meta = golden_cases.load("triton_linear_activation__42x32x32__float16")
    values = {**case["args"], **case["meta"]}
    positional, keywords = harness.bind_arguments(case["kernel"], values)
    # autotuned BLOCK_* are omitted, everything else is in signature order
    assert len(positional) == len(meta["parameters"]) - 3 and keywords == {}
    back = bind_by_name(case["kernel"], positional, keywords)
    assert set(back) == set(meta["parameters"]) - {"BLOCK_M", "BLOCK_N", "BLOCK_K"}
    assert back["M"] == 42 and back["stride_wk"] == 32


def test_bind_by_name_accepts_keyword_metas_and_rejects_surplus():
    handle = golden_cases.make_handle("softmax_kernel", ["x_ptr", "y_ptr", "n_cols", "BLOCK_N"])
    values = bind_by_name(handle, ["X", "Y", 97], {"BLOCK_N": 1024, "num_warps": 4})
    assert values["n_cols"] == 97 and values["BLOCK_N"] == 1024
    with pytest.raises(UnsupportedLaunch):
        bind_by_name(handle, ["X", "Y", 97, 1024, "extra"], {})
    with pytest.raises(UnsupportedLaunch):
        bind_by_name(handle, ["X"], {})


def test_reference_harness_binding_agrees(tmp_path):
    """With the reference tree present (``REFERENCE_ROOT``, or next to this repository), its
    own bind_arguments gives the same lists."""
    import os
    import sys
    from pathlib import Path
    base = os.environ.get("REFERENCE_ROOT") or str(Path(__file__).resolve().parents[2] / "reference")
    root = Path(base) / "ops" / "harness"
    if not root.is_dir():
        pytest.skip("reference tree not present on this host")
    sys.path.insert(0, str(root))
    from opslib import device as ref_device
    for tag in ("fast_rms_layernorm__7x67__float32", "swiglu_fwd__4x64__bfloat16",
                "attn_fwd_causal__1x1x8x16__float16"):
        case, _ = golden_cases.load(tag)
        values = {**case["args"], **case["meta"]}
        assert ref_device.bind_arguments(case["kernel"], values) == \
            harness.bind_arguments(case["kernel"], values)


# ------------------------------------------------------------------ registry
def test_registry_resolves_every_golden_kernel_and_native_handle():
    registry = default_registry()
    for tag in golden_cases.tags():
        case, _ = golden_cases.load(tag)
        assert registry.supports(case["kernel"]), tag
    for handle in (kernels.masked_softmax_kernel, kernels.gemm_bias_act_kernel,
                   kernels.attn_fwd_lse_kernel, kernels.swiglu_gemm_kernel):
        assert registry.supports(handle)


def test_registry_keys_on_name_and_signature_not_identity():
    registry = default_registry()
    same = golden_cases.make_handle("softmax_kernel", ["x_ptr", "y_ptr", "n_cols", "BLOCK_N"])
    other_sig = golden_cases.make_handle("softmax_kernel", ["x_ptr", "y_ptr", "n_cols"])
    assert registry.supports(same) and not registry.supports(other_sig)
    with pytest.raises(UnsupportedLaunch) as err:
        registry.resolve(other_sig)
    assert "softmax_kernel" in str(err.value) and "Triton" in str(err.value)


def test_native_handle_is_not_a_launcher():
    with pytest.raises(RuntimeError):
        kernels.masked_softmax_kernel[(4,)]
    name, params, autotuned = kernel_signature(kernels.attn_fwd_lse_kernel)
    assert name == "_attn_fwd_lse_kernel" and "lse_ptr" in params and not autotuned


class _FakeDevice:
    """Records launches; stages numpy arrays as-is (the _AliasProbe idea)."""
    name = "fake"

    def __init__(self):
        self.launches = []
        self.aliased = []

    def upload(self, array, dtype=None):
        return np.array(array, copy=True)

    def upload_aliased(self, group, pointer_types):
        self.aliased.append(sorted(group))
        return dict(group)

    def download(self, buffer):
        return np.asarray(buffer)

    def launch(self, kernel, grid, positional, keywords):
        self.launches.append((kernel, grid, positional, keywords))


def test_stage_case_contract():
    case, meta = golden_cases.load("fast_rms_layernorm__7x67__float32")
    device = _FakeDevice()
    staged = harness.stage_case(case, device)
    staged.launch()
    kernel, grid, positional, keywords = device.launches[0]
    assert grid == (7,) and keywords == {}
    assert len(positional) == len(meta["parameters"])
    assert isinstance(positional[1], int) and positional[1] == 67  # numpy scalars -> python
    assert set(staged.outputs()) == {"Y", "r"}
    # aliased host arrays are staged as one allocation
    base = np.zeros(16, np.float32)
    aliased = {"kernel": case["kernel"], "args": {"a": base, "b": base[4:]}, "grid": (1,),
               "outputs": ()}
    harness.stage_case(aliased, device)
    assert device.aliased == [["a", "b"]]
    with pytest.raises(ValueError):
        harness.stage_case({"args": {}}, device)


# ------------------------------------------------------------------ compile protocol
def test_compile_case_identity_and_counters():
    compiler = make_compiler()
    case, _ = golden_cases.load("matmul__16x16x16__bfloat16")
    bigger, _ = golden_cases.load("matmul__8x32x24__bfloat16")
    other_dtype, _ = golden_cases.load("matmul__16x16x16__float16")
    first = compiler.compile_case(case)
    second = compiler.compile_case(bigger)       # shapes do not enter the identity
    third = compiler.compile_case(other_dtype)   # pointer dtypes do
    assert not first.cache_hit and second.cache_hit and not third.cache_hit
    assert first.identity == second.identity != third.identity
    assert compiler.compile_count == 2 and compiler.cache_hits == 1
    assert first.provenance.startswith("compiler_b200/") and len(first.sha256) == 64
    # every switch that selects a kernel is part of the key
    from compiler_b200.factory import KERNEL_SWITCHES
    base_key = compiler.identity(case)["key"]
    for name in KERNEL_SWITCHES:
        switches = dict(PlanOptions().switches)
        switches[name] = "another-choice"
        alt = make_compiler(PlanOptions(switches=switches))
        assert alt.identity(case)["key"] != base_key, name
    assert make_compiler(PlanOptions()).identity(case)["key"] == base_key


def test_plan_options_sample_the_environment(monkeypatch):
    monkeypatch.setenv("B200OPS_GEMM_PAIR", "0")
    forced = PlanOptions()
    monkeypatch.delenv("B200OPS_GEMM_PAIR")
    assert forced.switches["B200OPS_GEMM_PAIR"] == "0"
    assert forced.identity_part() != PlanOptions().identity_part()


def test_compile_case_refuses_unknown_kernels():
    compiler = make_compiler()
    case = {"kernel": golden_cases.make_handle("fft_kernel", ["x_ptr", "n"]),
            "args": {"x_ptr": np.zeros(4, np.float32), "n": 4}}
    with pytest.raises(UnsupportedLaunch):
        compiler.compile_case(case)
    assert compiler.compile_count == 0


# ------------------------------------------------------------------ graph capture (host logic)
class _FakeGraphLib:
    """Stands in for the C ABI: records the calls of compiler_b200.graph without a GPU."""

    def __init__(self, end_status=0):
        self.calls = []
        self.end_status = end_status

    def b200_stream_create(self, out):
        out._obj.value = 0x1000
        self.calls.append("stream_create")
        return 0

    def b200_stream_destroy(self, stream):
        self.calls.append("stream_destroy")
        return 0

    def b200_stream_sync(self, stream):
        self.calls.append("stream_sync")
        return 0

    def b200_graph_begin_capture(self, stream):
        self.calls.append("begin")
        return 0

    def b200_graph_end_capture(self, stream, out):
        self.calls.append("end")
        if self.end_status == 0:
            out._obj.value = 0x2000
        return self.end_status

    def b200_graph_launch(self, graph, stream):
        self.calls.append("launch")
        return 0

    def b200_graph_destroy(self, graph):
        self.calls.append("destroy")
        return 0

    def b200_last_error(self):
        return b"capture failed"


def test_graph_capture_records_launches_and_releases(monkeypatch):
    from compiler_b200 import graph
    from compiler_b200.runtime import abi

    fake = _FakeGraphLib()
    monkeypatch.setattr(abi, "lib", lambda: fake)
    stream = graph.Stream()
    with graph.capture(stream) as g:
        with pytest.raises(RuntimeError):
            g.launch(stream)  # not ready inside the block
    g.launch(stream)
    g.launch(stream)
    g.close()
    g.close()  # idempotent
    stream.close()
    assert fake.calls == ["stream_create", "begin", "end", "launch", "launch", "destroy",
                          "stream_destroy"]


def test_graph_capture_is_closed_and_discarded_when_the_block_raises(monkeypatch):
    from compiler_b200 import graph
    from compiler_b200.runtime import abi

    fake = _FakeGraphLib()
    monkeypatch.setattr(abi, "lib", lambda: fake)
    stream = graph.Stream()
    with pytest.raises(ValueError):
        with graph.capture(stream):
            raise ValueError("the block failed")
    # the capture was ended (the stream must not stay in capture mode) and its graph dropped
    assert fake.calls[-2:] == ["end", "destroy"]
    stream.close()


def test_graph_capture_reports_a_failed_end(monkeypatch):
    from compiler_b200 import graph
    from compiler_b200.runtime import abi

    fake = _FakeGraphLib(end_status=4)
    monkeypatch.setattr(abi, "lib", lambda: fake)
    stream = graph.Stream()
    with pytest.raises(Exception):
        with graph.capture(stream):
            pass
    stream.close()
