"""``B200Device`` against the Device protocol, in the manner of the reference's own
device tests (ops/harness/tests/test_cuda_device.py:33-180): transfer round trips per
dtype, bf16 view vs cast, aliased staging, device-side compare equal to the host
compare, the event timer, properties."""
import numpy as np
import pytest

from compiler_b200 import harness, ops
from compiler_b200.device import B200Buffer, from_bf16_bits, to_bf16_bits
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "float16", "int32", "int64", "uint8", "bool", "float64"])
def test_roundtrip(device, dtype):
    rng = np.random.default_rng(1)
    host = (rng.standard_normal((37, 19)) * 50).astype(dtype)
    buf = device.upload(host)
    assert str(buf.dtype) == dtype and buf.shape == (37, 19) and buf.data_ptr() != 0
    back = device.download(buf)
    assert back.dtype == host.dtype and np.array_equal(back, host)


def test_bf16_cast_and_view(device):
    rng = np.random.default_rng(2)
    host = rng.standard_normal(1000).astype(np.float32)
    cast = device.upload(host, "bfloat16")
    assert str(cast.dtype) == "bfloat16" and cast.nbytes == 2000
    back = device.download(cast)
    assert back.dtype == np.float32 and np.array_equal(back, oracle.bf16_round(host))
    bits = to_bf16_bits(host)
    view = device.upload(bits, "bfloat16")
    assert np.array_equal(device.download(view), bits)  # uint16 hosts round-trip as bits
    assert np.array_equal(from_bf16_bits(bits), oracle.bf16_round(host))
    with pytest.raises(TypeError):
        device.upload(host.astype(np.float64), "bfloat16")


def test_dtype_markers_are_value_keyed(device):
    a, b = device.alloc((4,), "float16"), device.alloc((8,), np.float16)
    assert a.dtype is b.dtype and str(a.dtype) == "float16" and a.dtype.name == "float16"


def test_alloc_release_and_empty(device):
    bufs = {"x": device.alloc((0, 5), "float32"), "y": device.alloc((3,), "int32")}
    assert device.download(bufs["x"]).shape == (0, 5)
    device.release(bufs)
    assert bufs["y"].ptr == 0


def test_aliased_upload_is_one_allocation(device):
    base = np.arange(64, dtype=np.float32)
    group = {"whole": base, "tail": base[32:]}
    out = device.upload_aliased(group, {})
    assert out["tail"].data_ptr() - out["whole"].data_ptr() == 32 * 4
    case = {"kernel": None, "args": {"whole": base, "tail": base[32:], "n": 3}}
    groups = harness._alias_groups({"whole": base, "tail": base[32:], "other": np.zeros(3)})
    assert sorted(map(sorted, groups)) == [["other"], ["tail", "whole"]]
    assert np.array_equal(device.download(out["tail"]), base[32:])
    del case


def test_device_compare_matches_host_compare(device):
    rng = np.random.default_rng(3)
    ref = rng.standard_normal(100000).astype(np.float32)
    got = ref.copy()
    got[17] += 0.5
    got[999] = np.nan
    ref[5] = np.nan
    got[5] = np.nan
    policy = {"comparator": "allclose", "rtol": 1e-3, "atol": 1e-3, "equal_nan": True}
    ok, err = device.compare(device.upload(got), ref, policy)
    assert not ok
    clean = ref.copy()
    clean[3] += 1e-5
    ok, err = device.compare(device.upload(clean), ref, policy)
    host_err = oracle.compare(clean, ref, 1e-3, 1e-3)
    assert ok and err == pytest.approx(host_err, rel=1e-12)
    assert device.compare(device.upload(ref.astype(np.float16)), ref, policy) is None


def test_timer_and_properties(device):
    x = device.upload(np.ones((1024, 1024), np.float32))
    y = device.alloc((1024, 1024), "float32")
    with device.timer() as t:
        ops.softmax(x, y)
    assert t.seconds is not None and 0 < t.seconds < 1.0
    props = device.properties()
    assert props["sm_count"] > 0 and props["llc_bytes"] > 0 and "name" in props
    device.synchronize()


def test_pinned_transfers(device):
    pinned = device.pinned_empty((256, 256), np.float32)
    pinned.array[...] = np.arange(65536, dtype=np.float32).reshape(256, 256)
    buf = device.upload(pinned.array, pinned=pinned)
    out = device.pinned_empty((256, 256), np.float32)
    back = device.download(buf, out=out)
    assert np.array_equal(back, pinned.array)
    assert isinstance(buf, B200Buffer)


def test_page_locked_host_memory_as_operand(device):
    """Page-locked host memory from ``b200_malloc_host`` is addressable from the device: the
    row-wise and elementwise entry points take it as operand memory (loads and stores cross
    PCIe, no staging copy).  RMSNorm host -> host with the weight on the device, SwiGLU with
    one operand on the host, and the results equal those of device-resident operands."""
    from compiler_b200.device import B200Buffer
    rows, cols = 257, 1000
    rng = np.random.default_rng(17)
    hx = device.pinned_empty((rows, cols), np.float32)
    hx.array[...] = rng.standard_normal((rows, cols))
    hy = device.pinned_empty((rows, cols), np.float32)
    hy.array[...] = 0
    w = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    dw, dr = device.upload(w), device.alloc((rows,), "float32")
    as_buffer = lambda p: B200Buffer(p.ptr, "float32", (rows, cols), rows * cols * 4,  # noqa: E731
                                     owner=False)
    ops.rmsnorm(as_buffer(hx), dw, as_buffer(hy), dr, eps=1e-6)
    device.synchronize()
    y_ref, r_ref = oracle.rmsnorm_ref(hx.array, w, 1e-6)
    oracle.compare(hy.array.astype(np.float64), y_ref, 1e-5, 1e-6, name="Y in host memory")
    oracle.compare(device.download(dr).astype(np.float64), r_ref, 1e-5, 1e-6, name="r")
    dx, dy = device.upload(hx.array), device.alloc((rows, cols), "float32")
    ops.rmsnorm(dx, dw, dy, dr, eps=1e-6)
    assert np.array_equal(device.download(dy), hy.array)
    gate = rng.standard_normal((rows, cols)).astype(np.float32)
    dg, dout = device.upload(gate), device.alloc((rows, cols), "float32")
    ops.swiglu(as_buffer(hx), dg, dout)
    expect = hx.array / (1 + np.exp(-hx.array.astype(np.float64))) * gate
    oracle.compare(device.download(dout).astype(np.float64), expect, 1e-5, 1e-6, name="swiglu")
    hx.free()
    hy.free()


@pytest.mark.parametrize("schedule", ["in_step", "staged", "direct"])
def test_row_pipeline_matches_single_launch(device, schedule):
    """Host-to-host softmax gives the same bytes as one launch on device buffers: whole chunks
    spread over streams, a stream per stage (events between the stages), and one launch on
    the page-locked host buffers themselves; a second run over the same buffers gives them
    again."""
    from compiler_b200 import pipeline
    rows, cols = 1000, 4000
    rng = np.random.default_rng(5)
    hx = device.pinned_empty((rows, cols), np.float16)
    hx.array[...] = (rng.standard_normal((rows, cols)) * 2).astype(np.float16)
    hy = device.pinned_empty((rows, cols), np.float16)
    pipe = pipeline.RowPipeline(device, rows, cols, "float16", chunks=7, streams=3,
                                staged=schedule == "staged", direct=schedule == "direct")
    out = pipeline.masked_softmax_host(pipe, hx, hy, row_offset=123).copy()
    hy.array[...] = 0
    assert np.array_equal(pipeline.masked_softmax_host(pipe, hx, hy, row_offset=123), out)
    pipe.close()
    dx, dy = device.upload(hx.array), device.alloc((rows, cols), "float16")
    ops.softmax(dx, dy, causal_mod=True, row_offset=123)
    assert np.array_equal(out, device.download(dy))
    oracle.compare(out.astype(np.float64), oracle.masked_softmax_ref(hx.array, 123), 1e-2, 1e-2)


def test_repeated_launches_replay_the_bound_calls(device):
    """A launch is bound once per (kernel, grid, buffers, scalars): later launches replay the
    recorded library calls, read the buffers' current contents, and a different buffer or
    scalar binds anew; a rejected launch leaves nothing behind."""
    import golden_cases
    from compiler_b200.registry import UnsupportedLaunch
    case, _ = golden_cases.load("softmax__4x97__float32")
    staged = harness.stage_case(case, device)
    before = len(device._plans)
    staged.launch()
    assert len(device._plans) == before + 1
    first = staged.outputs()["y_ptr"]
    x = np.asarray(case["args"]["x_ptr"], dtype=np.float32)
    oracle.compare(first, oracle.softmax_ref(x), 2e-3, 2e-3)
    # same buffers, new contents: the replayed launch computes on what is there now
    device.copy_in(staged.buffer("x_ptr"), np.ascontiguousarray(-x), sync=True)
    count = device.launch_count
    staged.launch()
    assert len(device._plans) == before + 1 and device.launch_count == count + 1
    oracle.compare(staged.outputs()["y_ptr"], oracle.softmax_ref(-x), 2e-3, 2e-3)
    # another staging of the same case has other buffers: a second plan
    other = harness.stage_case(case, device)
    other.launch()
    assert len(device._plans) == before + 2
    oracle.compare(other.outputs()["y_ptr"], oracle.softmax_ref(x), 2e-3, 2e-3)
    # one timer serves many launches (the benchmark runner keeps one for all its samples)
    timer = device.timer()
    seconds = []
    for _ in range(5):
        with timer:
            staged.launch()
        seconds.append(timer.seconds)
    assert all(0 < s < 1.0 for s in seconds)
    timer.close()
    unknown = golden_cases.make_handle("no_such_kernel", ["x_ptr", "y_ptr"])
    size = len(device._plans)
    with pytest.raises(UnsupportedLaunch):
        device.launch(unknown, (1,), [staged.buffer("x_ptr"), staged.buffer("y_ptr")], {})
    assert len(device._plans) == size


def test_bounded_wait_expires_and_the_context_survives(device):
    """The failure path of the device-side waits, without a fault: a wait on a barrier that
    nothing completes gives up after its limit, the status word reports B200_TIMEOUT with the
    waiter's site, reading it clears it, and the next launch on the same context is correct."""
    import ctypes
    import time
    from compiler_b200.runtime import abi
    gave_up = ctypes.c_uint32(0)
    start = time.perf_counter()
    abi.check(abi.lib().b200_wait_selftest(ctypes.byref(gave_up), None))
    elapsed = time.perf_counter() - start
    assert gave_up.value == 1
    assert 1.0 < elapsed < 10.0  # the limit is about two seconds, not forever
    with pytest.raises(abi.B200Error) as caught:
        device.check_status()
    assert caught.value.status == abi.TIMEOUT and "site 31" in str(caught.value)
    device.check_status()  # cleared by the read
    x = np.random.default_rng(12).standard_normal((64, 1000)).astype(np.float32)
    dx, dy = device.upload(x), device.alloc(x.shape, "float32")
    ops.softmax(dx, dy)
    oracle.compare(device.download(dy).astype(np.float64), oracle.softmax_ref(x), 2e-3, 2e-3)


def test_captured_launches_replay_as_one_graph(device):
    """A sequence of operator launches recorded into a CUDA graph gives the same bytes as the
    direct launches, on every replay and with the inputs changed between replays."""
    from compiler_b200 import graph
    from compiler_b200.runtime import abi
    rng = np.random.default_rng(21)
    rows, cols, sets = 256, 4000, 3
    xs = [(rng.standard_normal((rows, cols)) * 2).astype(np.float16) for _ in range(sets)]
    dxs = [device.upload(x) for x in xs]
    dys = [device.alloc((rows, cols), "float16") for _ in range(sets)]
    a = oracle.to_storage(rng.standard_normal((256, 128)).astype(np.float32) / 8, "bfloat16")
    b = oracle.to_storage(rng.standard_normal((128, 512)).astype(np.float32), "bfloat16")
    da, db = device.upload(a, "bfloat16"), device.upload(b, "bfloat16")
    dc = device.alloc((256, 512), "bfloat16")
    stream = graph.Stream()
    # every operator once outside the capture (first calls configure kernels)
    ops.softmax(dxs[0], dys[0], causal_mod=True, stream=stream.handle)
    ops.gemm(da, db, dc, act=abi.ACT_GELU_TANH, stream=stream.handle)
    stream.synchronize()
    with graph.capture(stream) as g:
        for i in range(12):
            ops.softmax(dxs[i % sets], dys[i % sets], causal_mod=True, row_offset=7,
                        stream=stream.handle)
        ops.gemm(da, db, dc, act=abi.ACT_GELU_TANH, stream=stream.handle)
    for replay in range(2):
        for y in dys:
            device.copy_in(y, np.zeros((rows, cols), np.float16), sync=True)
        g.launch(stream)
        stream.synchronize()
        for x, dy in zip(xs, dys):
            oracle.compare(device.download(dy).astype(np.float64), oracle.masked_softmax_ref(x, 7),
                           1e-2, 1e-2)
        oracle.compare(device.download(dc).astype(np.float64),
                       oracle.linear_act_ref(a, b, None, "gelu_tanh"), 2e-2, 2e-2)
        # new contents in the same buffers: the next replay must see them
        xs = [(-x).astype(np.float16) for x in xs]
        for x, dx in zip(xs, dxs):
            device.copy_in(dx, x, sync=True)
    with pytest.raises(abi.B200Error):  # the default stream cannot be captured
        abi.check(abi.lib().b200_graph_begin_capture(None))
    g.close()
    stream.close()


def test_decode_scratch_follows_the_stream(device):
    """Decode attention keeps one scratch buffer per (device, stream) and gives it back when
    the stream is destroyed through the library: streams created per use do not pile buffers
    up, and a new stream (whatever handle value it gets) starts clean and gives the oracle's
    result."""
    from compiler_b200 import graph
    rng = np.random.default_rng(9)
    rows, keys, d = 16, 2000, 128
    q = oracle.bf16_round(rng.standard_normal((rows, d)).astype(np.float32))
    k, v = (oracle.bf16_round(rng.standard_normal((rows, keys, d)).astype(np.float32))
            for _ in range(2))
    dq, dk, dv = (device.upload(t, "bfloat16") for t in (q, k, v))
    ref = oracle.flash_decode_ref(q, k, v, 1.0 / np.sqrt(d))
    for _ in range(6):
        stream = graph.Stream()
        out = device.alloc((rows, d), "bfloat16")
        ops.attention_decode(dq, dk, dv, out, stream=stream.handle)
        stream.synchronize()
        oracle.compare(device.download(out).astype(np.float64), ref, 2e-2, 2e-2, name="decode")
        stream.close()


def test_allreduce_barrier_gives_up_when_a_peer_never_arrives(device):
    """The in-switch all-reduce kernel carries its own cross-rank barriers.  Here its "peer" is
    a flag array that nothing ever signals: the start barrier must run out after about two
    seconds, record B200_TIMEOUT with its site, skip the data phase (the data pointers are
    never touched) and return, and the context must stay usable."""
    import ctypes
    import time
    from compiler_b200.runtime import abi
    lib = abi.lib()
    words = lib.b200_signal_pad_bytes() // 4
    pads = [device.upload(np.zeros(words, np.int32)) for _ in range(2)]
    data = device.alloc((1024,), "bfloat16")
    pad_ptrs = (ctypes.c_void_p * 2)(pads[0].ptr, pads[1].ptr)
    code = abi.DTYPE_CODES["bfloat16"]
    start = time.perf_counter()
    abi.check(lib.b200_multimem_allreduce(data.ptr, code, data.ptr, code, 0, 1024, 0, 2,
                                          pad_ptrs, 1, 1, device.stream))
    with pytest.raises(abi.B200Error) as caught:
        device.check_status()
    elapsed = time.perf_counter() - start
    assert caught.value.status == abi.TIMEOUT and "site 40" in str(caught.value)
    assert 1.0 < elapsed < 10.0
    device.check_status()  # cleared by the read
    # rank 0 signalled both arrays (its own flag and the peer's) before it waited
    assert device.download(pads[0])[0] == 1 and device.download(pads[1])[0] == 1
    # argument checks never reach the device
    assert lib.b200_multimem_allreduce(data.ptr, code, data.ptr, code, 0, 1024, 0, 2, pad_ptrs,
                                       0, 1, device.stream) == abi.REJECTED   # epoch 0
    assert lib.b200_multimem_allreduce(data.ptr, code, data.ptr, code, 0, 1000, 0, 2, None, 0, 0,
                                       device.stream) == abi.REJECTED         # count % 16
    x = np.random.default_rng(13).standard_normal((64, 1000)).astype(np.float32)
    dx, dy = device.upload(x), device.alloc(x.shape, "float32")
    ops.softmax(dx, dy)
    oracle.compare(device.download(dy).astype(np.float64), oracle.softmax_ref(x), 2e-3, 2e-3)
