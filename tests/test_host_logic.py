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


class _FakePipelineLib:
    """Host memory as "device memory"; numbered stream / event handles; a log of every call."""

    def __init__(self):
        self.log, self._blocks, self._next = [], {}, 100

    def _handle(self, out, kind):
        self._next += 1
        out._obj.value = self._next
        self.log.append((kind + "_create", self._next))
        return 0

    def b200_stream_create(self, out):
        return self._handle(out, "stream")

    def b200_event_create(self, out):
        return self._handle(out, "event")

    def b200_malloc(self, out, nbytes):
        import ctypes
        block = ctypes.create_string_buffer(int(nbytes) + 64)
        out._obj.value = (ctypes.addressof(block) + 63) & ~63
        self._blocks[out._obj.value] = block
        return 0

    b200_malloc_host = b200_malloc

    def _copy(self, name):
        def copy(dst, src, nbytes, stream):
            import ctypes
            ctypes.memmove(int(dst), int(src), int(nbytes))
            self.log.append((name, stream.value))
            return 0
        return copy

    def __getattr__(self, name):
        if name in ("b200_memcpy_h2d", "b200_memcpy_d2h"):
            return self._copy(name[5:])
        if not name.startswith("b200_"):
            raise AttributeError(name)

        def call(*args):
            self.log.append((name[5:],) + tuple(getattr(a, "value", a) for a in args))
            return 0
        return call


@pytest.mark.parametrize("schedule", ["staged", "in_step", "direct"])
def test_row_pipeline_schedules(monkeypatch, schedule):
    """The host-to-host row pipeline: with a stream per stage every inbound copy is on the first
    stream, every launch on the second after its chunk's copy event, every outbound copy on the
    third after its chunk's launch event; with whole chunks per stream a chunk's three steps
    share one stream; ``direct`` is one launch on the host buffers and no copy.  Every way
    every row arrives."""
    import ctypes
    from compiler_b200 import pipeline
    from compiler_b200.device import PinnedArray
    from compiler_b200.runtime import abi

    fake = _FakePipelineLib()
    monkeypatch.setattr(abi, "lib", lambda: fake)

    class Device:
        def alloc(self, shape, dtype):
            from compiler_b200.device import B200Buffer
            out = ctypes.c_void_p()
            nbytes = int(np.prod(shape)) * 2
            fake.b200_malloc(ctypes.byref(out), nbytes)
            return B200Buffer(out.value, dtype, tuple(shape), nbytes, owner=False)

        def release(self, buffers):
            pass

    rows, cols = 50, 16
    hx, hy = PinnedArray((rows, cols), np.float16), PinnedArray((rows, cols), np.float16)
    hx.array[...] = np.arange(rows * cols, dtype=np.float32).reshape(rows, cols) % 251
    hy.array[...] = -1
    staged = schedule == "staged"
    pipe = pipeline.RowPipeline(Device(), rows, cols, "float16", chunks=4, streams=2,
                                staged=staged, direct=schedule == "direct")
    launches = []

    def launch(x, y, first_row, stream):
        ctypes.memmove(y.ptr, x.ptr, x.shape[0] * cols * 2)   # the "operator": a copy
        launches.append((first_row, x.shape[0], stream))
        fake.log.append(("launch", stream))

    out = pipe.run(launch, hx, hy)
    assert np.array_equal(out, hx.array)
    assert [l[0] for l in launches] == [lo for lo, _ in pipe.chunks]
    assert sum(l[1] for l in launches) == rows
    streams = [h for kind, h in (e[:2] for e in fake.log) if kind == "stream_create"]
    steps = [e for e in fake.log if e[0] in ("memcpy_h2d", "launch", "memcpy_d2h")]
    if schedule == "direct":
        assert [e[0] for e in steps] == ["launch"] and launches == [(0, rows, streams[0])]
        assert (launches[0][2], pipe.x) == (streams[0], None)
    elif staged:
        assert len(streams) == 3
        by_kind = {"memcpy_h2d": streams[0], "launch": streams[1], "memcpy_d2h": streams[2]}
        assert all(e[1] == by_kind[e[0]] for e in steps)
        waits = [e for e in fake.log if e[0] == "stream_wait_event"]
        records = [e for e in fake.log if e[0] == "event_record"]
        assert len(waits) == len(records) == 2 * len(pipe.chunks)
        # every wait names an event recorded just before it, on the stage before
        for (_, event, on), (_, stream, waited) in zip(records, waits):
            assert waited == event and streams.index(stream) == streams.index(on) + 1
        assert fake.log[-1] == ("stream_sync", streams[2])
    else:
        assert len(streams) == 2
        for i in range(len(pipe.chunks)):
            assert {e[1] for e in steps[3 * i:3 * i + 3]} == {streams[i % 2]}
    pipe.close()
    hx.free()
    hy.free()
