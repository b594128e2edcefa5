"""Rates of the sibling operators at sizes well above the L2 (one JSON line per operator).

    python -m compiler_b200.sibling_bench            # every operator, bf16 and fp32
    python -m compiler_b200.sibling_bench --only softmax

Each operator runs on four rotating buffer sets (more than 1 GB between reuses of a buffer);
20 launches are captured into a CUDA graph, and two replays are timed with CUDA events on the
capturing stream, so the figure is the steady back-to-back rate without the host's launch
latency.  Bytes are the algorithmic ones (every operand read once, the result written once).
torch is used for device memory and random inputs only.
"""
from __future__ import annotations

import argparse
import ctypes
import json

from compiler_b200 import graph, ops
from compiler_b200.runtime import abi

ROWS, COLS = 16384, 4096
SETS, LAUNCHES = 4, 20


def _timed(stream, launch, sets=SETS):
    lib = abi.lib()
    for i in range(3):
        launch(i % sets)
    stream.synchronize()
    with graph.capture(stream) as g:
        for i in range(LAUNCHES):
            launch(i % sets)
    g.launch(stream)
    stream.synchronize()
    begin, end = ctypes.c_void_p(), ctypes.c_void_p()
    abi.check(lib.b200_event_create(ctypes.byref(begin)))
    abi.check(lib.b200_event_create(ctypes.byref(end)))
    abi.check(lib.b200_event_record(begin, stream._ptr))
    g.launch(stream)
    g.launch(stream)
    abi.check(lib.b200_event_record(end, stream._ptr))
    stream.synchronize()
    ms = ctypes.c_float()
    abi.check(lib.b200_event_elapsed_ms(begin, end, ctypes.byref(ms)))
    lib.b200_event_destroy(begin)
    lib.b200_event_destroy(end)
    g.close()
    return ms.value / (2 * LAUNCHES)


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--only", default="", help="substring of the operator names to run")
    args = parser.parse_args(argv)
    import torch

    torch.manual_seed(0)
    stream = graph.Stream()
    S = stream.handle

    def report(name, launch, nbytes=None, flop=None, sets=SETS):
        if args.only and args.only not in name:
            return
        ms = _timed(stream, launch, sets)
        record = {"op": name, "ms_per_launch": round(ms, 5)}
        if nbytes:
            record["GBps"] = round(nbytes / ms / 1e6, 1)
        if flop:
            record["TFLOPs"] = round(flop / ms / 1e9, 1)
        print(json.dumps(record), flush=True)

    def rnd(shape, dtype, scale=1.0):
        return (torch.randn(shape, device="cuda") * scale).to(dtype)

    for dtype, tag, es in ((torch.bfloat16, "bf16", 2), (torch.float32, "f32", 4)):
        n = ROWS * COLS
        xs = [rnd((ROWS, COLS), dtype) for _ in range(SETS)]
        ys = [rnd((ROWS, COLS), dtype) for _ in range(SETS)]
        outs = [torch.empty((ROWS, COLS), device="cuda", dtype=dtype) for _ in range(SETS)]
        flat = lambda t: t.view(-1)  # noqa: E731
        report(f"swiglu_{tag}", lambda i: ops.swiglu(xs[i], ys[i], outs[i], stream=S), 3 * n * es)
        report(f"gelu_erf_{tag}", lambda i: ops.elementwise(
            abi.EW_GELU_ERF, flat(xs[i]), flat(outs[i]), stream=S), 2 * n * es)
        report(f"add_gelu_erf_{tag}", lambda i: ops.elementwise(
            abi.EW_ADD_GELU_ERF, flat(xs[i]), flat(outs[i]), b=flat(ys[i]), p0=1.5, stream=S),
            3 * n * es)
        report(f"geglu_tanh_{tag}", lambda i: ops.elementwise(
            abi.EW_GEGLU_TANH, flat(xs[i]), flat(outs[i]), b=flat(ys[i]), stream=S), 3 * n * es)
        bias = rnd((COLS,), dtype)
        report(f"bias_scale_clamp_gelu_{tag}", lambda i: ops.elementwise(
            abi.EW_BIAS_SCALE_CLAMP_GELU, flat(xs[i]), flat(outs[i]), b=bias, p0=0.5, p1=-1.0,
            p2=1.0, stream=S), 2 * n * es)
        report(f"softmax_{tag}", lambda i: ops.softmax(xs[i], outs[i], stream=S), 2 * n * es)
        report(f"softmax_mul_{tag}", lambda i: ops.softmax_variant(
            xs[i], outs[i], mul=ys[i], stream=S), 3 * n * es)
        positive = [x.abs() + 0.1 for x in xs]
        report(f"softmax_log_{tag}", lambda i: ops.softmax_variant(
            positive[i], outs[i], log_input=True, stream=S), 2 * n * es)
        del positive
        w = rnd((COLS,), dtype)
        report(f"rmsnorm_zero_centred_gamma_{tag}", lambda i: ops.rmsnorm(
            xs[i], w, outs[i], None, eps=1e-6, gamma_offset=1.0, stream=S), 2 * n * es)
        quarter = [rnd((ROWS, COLS // 4), dtype) for _ in range(SETS)]
        report(f"repeat4_log_softmax_{tag}", lambda i: ops.repeat_log_softmax(
            quarter[i], outs[i], 4, stream=S), (n // 4 + n) * es)
        del xs, ys, outs, quarter
        torch.cuda.empty_cache()

    k, n = 16384, 8192
    q = [torch.randint(-128, 127, (k, n), device="cuda", dtype=torch.int8) for _ in range(SETS)]
    scale = rnd((n,), torch.bfloat16)
    deq = [torch.empty((k, n), device="cuda", dtype=torch.bfloat16) for _ in range(SETS)]
    report("dequantize_int8_to_bf16", lambda i: ops.dequantize_cols(q[i], scale, deq[i], stream=S),
           k * n * 3)
    del q, deq
    torch.cuda.empty_cache()

    m, k, n = 8192, 4096, 8192
    xs = [rnd((m, k), torch.bfloat16) for _ in range(3)]
    w = rnd((k, n), torch.bfloat16, 0.02)
    w2 = rnd((k, n), torch.bfloat16, 0.02)
    g = rnd((k,), torch.bfloat16)
    outs = [torch.empty((m, n), device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    scratch_w = torch.empty((k, n), device="cuda", dtype=torch.bfloat16)
    scratch_r = torch.empty((m,), device="cuda")
    report("rms_matmul_bf16_8192x8192x4096", lambda i: ops.rms_matmul(
        xs[i], g, w, outs[i], scratch_w, scratch_r, stream=S), flop=2 * m * n * k, sets=3)
    gamma, beta, bias = (rnd((n,), torch.bfloat16) for _ in range(3))
    mins = torch.full((m,), float("inf"), device="cuda")
    report("gemm_groupnorm_rowmin_bf16_8192x8192x4096", lambda i: ops.gemm_groupnorm_rowmin(
        xs[i], w, gamma, beta, mins, bias=bias, group_size=32, stream=S), flop=2 * m * n * k,
        sets=3)
    report("gemm_swiglu_dual_bf16_8192x8192x4096", lambda i: ops.gemm(
        xs[i], w, outs[i], b2=w2, act=abi.ACT_SWIGLU, stream=S), flop=4 * m * n * k, sets=3)
    rows = 65536
    x2 = [rnd((rows, 4096), torch.bfloat16) for _ in range(3)]
    wl = rnd((64, 4096), torch.bfloat16, 0.02)
    y2 = [torch.empty((rows, 64), device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    report("linear_log_softmax_bf16_65536x64x4096", lambda i: ops.linear_log_softmax(
        x2[i], wl, y2[i], stream=S), (rows * 4096 + rows * 64 + 64 * 4096) * 2, sets=3)
    torch.cuda.synchronize()
    ops.device_status(S)


if __name__ == "__main__":
    main()
