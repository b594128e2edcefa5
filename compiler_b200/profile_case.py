"""Launch ONE operator a few times at a given shape -- the small, self-ending command to put
under a profiler (``ncu -k regex:<kernel> -c 3 python -m compiler_b200.profile_case ...``) or to
time a single shape by hand.

    python -m compiler_b200.profile_case softmax   --shape 16384 4000 --dtype float16
    python -m compiler_b200.profile_case rmsnorm   --shape 8192 4096  --dtype float32
    python -m compiler_b200.profile_case gemm      --shape 8192 8192 8192
    python -m compiler_b200.profile_case linear    --shape 8192 8192 4096   (weight as [N,K])
    python -m compiler_b200.profile_case attention --shape 2 8 4096 128
    python -m compiler_b200.profile_case attention_decode --shape 256 4096 128
    python -m compiler_b200.profile_case swiglu_gemm --shape 4096 1792 4096
    python -m compiler_b200.profile_case gemm_allreduce_beside --shape 4096 4096 7168

``gemm_allreduce_beside`` is the down-projection of the tensor-parallel MLP with its all-reduce
kernel running beside it, as one rank (the "all-reduce" then only rounds the float16 partial to
bfloat16): the product with progress counters per block of rows and the dependent kernel that
takes each block when it is counted complete.  Its record carries the kernel's own time
stamps: when it started and, per block of rows, when the GEMM had counted the block complete
and when the block was reduced (microseconds after the start of the all-reduce kernel).

Inputs are seeded random values generated on the host and uploaded through ``B200Device``
(no torch); every launch is timed with CUDA events and the times are printed as JSON.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from compiler_b200 import ops
from compiler_b200.device import B200Device, to_bf16_bits
from compiler_b200.runtime import abi


def _upload(device, array, dtype):
    if dtype == "bfloat16":
        return device.upload(to_bf16_bits(array.astype(np.float32)), "bfloat16")
    return device.upload(array.astype(dtype), dtype)


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("op", choices=["softmax", "rmsnorm", "gemm", "attention", "attention_decode",
                                       "linear", "linear_log_softmax", "swiglu_gemm",
                                       "gemm_allreduce_beside"])
    parser.add_argument("--blocks", type=int, default=4,
                        help="gemm_allreduce_beside: blocks of rows")
    parser.add_argument("--shape", type=int, nargs="+", required=True)
    parser.add_argument("--dtype", default=None)
    parser.add_argument("--launches", type=int, default=3)
    parser.add_argument("--repeat", type=int, default=1,
                        help="launches per timed sample, back to back (hides the host's launch "
                             "latency for kernels of tens of microseconds); times are per launch")
    parser.add_argument("--device", type=int, default=0)
    parser.add_argument("--no-mask", action="store_true", help="softmax/attention without mask")
    parser.add_argument("--act", default="gelu_tanh", choices=["none", "gelu_tanh", "gelu_erf"],
                        help="gemm epilogue")
    parser.add_argument("--no-bias", action="store_true", help="gemm without the bias add")
    parser.add_argument("--sets", type=int, default=1,
                        help="softmax: rotate over this many input / output buffer sets, so a "
                             "launch meets the cache state of a steady sequence (dirty lines of "
                             "the launches before it) instead of its own previous output")
    args = parser.parse_args(argv)
    device = B200Device(args.device)
    rng = np.random.default_rng(0)
    shape = tuple(args.shape)

    if args.op == "softmax":
        dtype = args.dtype or "float16"
        host = rng.standard_normal(shape, dtype=np.float32) * 2
        xs = [_upload(device, host, dtype) for _ in range(max(1, args.sets))]
        ys = [device.alloc(shape, dtype) for _ in xs]
        turn = iter(range(1 << 30))

        def launch():
            i = next(turn) % len(xs)
            ops.softmax(xs[i], ys[i], causal_mod=not args.no_mask)
        work = {"bytes": 2 * int(np.prod(shape)) * abi.DTYPE_SIZES[dtype]}
    elif args.op == "rmsnorm":
        dtype = args.dtype or "float32"
        x = _upload(device, rng.standard_normal(shape, dtype=np.float32), dtype)
        w = _upload(device, rng.uniform(0.5, 1.5, shape[1]).astype(np.float32), dtype)
        y, r = device.alloc(shape, dtype), device.alloc((shape[0],), dtype)
        launch = lambda: ops.rmsnorm(x, w, y, r, eps=1e-6)  # noqa: E731
        work = {"bytes": 2 * int(np.prod(shape)) * abi.DTYPE_SIZES[dtype]}
    elif args.op in ("gemm", "swiglu_gemm"):
        dtype = args.dtype or "bfloat16"
        m, n, k = shape
        a = _upload(device, rng.standard_normal((m, k), dtype=np.float32) / np.sqrt(k), dtype)
        b = _upload(device, rng.standard_normal((k, n), dtype=np.float32) / np.sqrt(k), dtype)
        c = device.alloc((m, n), dtype)
        if args.op == "gemm":
            bias = None if args.no_bias else _upload(
                device, rng.normal(0, 0.1, n).astype(np.float32), dtype)
            act = {"none": abi.ACT_NONE, "gelu_tanh": abi.ACT_GELU_TANH,
                   "gelu_erf": abi.ACT_GELU_ERF}[args.act]
            launch = lambda: ops.gemm(a, b, c, bias=bias, act=act)  # noqa: E731
            work = {"flop": 2 * m * n * k}
        else:
            b2 = _upload(device, rng.standard_normal((k, n), dtype=np.float32) / np.sqrt(k), dtype)
            launch = lambda: ops.gemm(a, b, c, b2=b2, act=abi.ACT_SWIGLU)  # noqa: E731
            work = {"flop": 4 * m * n * k}
    elif args.op == "gemm_allreduce_beside":
        dtype = "bfloat16"
        m, n, k = shape
        a = _upload(device, rng.standard_normal((m, k), dtype=np.float32) / np.sqrt(k), dtype)
        b = _upload(device, rng.standard_normal((k, n), dtype=np.float32) / np.sqrt(k), dtype)
        partial, out = device.alloc((m, n), "float16"), device.alloc((m, n), dtype)
        words = abi.lib().b200_progress_words()
        counters = device.upload(np.zeros(words, np.int32))
        rows = max(256, m // max(1, args.blocks) // 256 * 256)
        extra = {"rows_per_block": rows}

        def launch():
            targets = ops.gemm_progress(a, b, partial, rows, counters)
            ops.peer_allreduce_blocks([partial.ptr], [out.ptr], m * n, rows * n, counters, targets,
                                      0, 1, in_dtype="float16", out_dtype=dtype)
            extra["blocks"] = len(targets)
        work = {"flop": 2 * m * n * k}
    elif args.op == "linear":
        dtype = args.dtype or "bfloat16"
        m, n, k = shape
        x = _upload(device, rng.standard_normal((m, k), dtype=np.float32) / np.sqrt(k), dtype)
        w = _upload(device, rng.standard_normal((n, k), dtype=np.float32) / np.sqrt(k), dtype)
        y = device.alloc((m, n), dtype)
        bias = None if args.no_bias else _upload(
            device, rng.normal(0, 0.1, n).astype(np.float32), dtype)
        act = {"none": abi.ACT_NONE, "gelu_tanh": abi.ACT_GELU_TANH,
               "gelu_erf": abi.ACT_GELU_ERF}[args.act]
        launch = lambda: ops.linear(x, w, y, bias=bias, act=act)  # noqa: E731
        work = {"flop": 2 * m * n * k}
    elif args.op == "linear_log_softmax":
        dtype = args.dtype or "bfloat16"
        m, n, k = shape
        x = _upload(device, rng.standard_normal((m, k), dtype=np.float32), dtype)
        w = _upload(device, rng.standard_normal((n, k), dtype=np.float32) / np.sqrt(k), dtype)
        y = device.alloc((m, n), dtype)
        launch = lambda: ops.linear_log_softmax(x, w, y)  # noqa: E731
        work = {"bytes": (m * k + n * k + m * n) * abi.DTYPE_SIZES[dtype]}
    elif args.op == "attention_decode":
        dtype = args.dtype or "bfloat16"
        rows, n, d = shape
        q = _upload(device, rng.standard_normal((rows, d), dtype=np.float32), dtype)
        k, v = (_upload(device, rng.standard_normal((rows, n, d), dtype=np.float32), dtype)
                for _ in range(2))
        o = device.alloc((rows, d), dtype)
        launch = lambda: ops.attention_decode(q, k, v, o)  # noqa: E731
        work = {"bytes": 2 * rows * n * d * abi.DTYPE_SIZES[dtype]}
    else:
        dtype = args.dtype or "bfloat16"
        z, h, n, d = shape
        q, k, v = (_upload(device, rng.standard_normal(shape, dtype=np.float32), dtype)
                   for _ in range(3))
        o, lse = device.alloc(shape, dtype), device.alloc((z, h, n), "float32")
        causal = not args.no_mask
        launch = lambda: ops.attention(q, k, v, o, lse=lse, causal=causal)  # noqa: E731
        work = {"flop": 4 * z * h * d * (n * (n + 1) // 2 if causal else n * n)}

    times = []
    for _ in range(args.launches):
        with device.timer() as t:
            for _ in range(max(1, args.repeat)):
                launch()
        times.append(t.seconds / max(1, args.repeat))
    device.check_status()
    record = {"op": args.op, "shape": shape, "dtype": dtype, "launch_seconds": times, **work}
    if args.op == "gemm_allreduce_beside":
        # 16 counters + the count of CTAs done + one word of padding, then the time stamps
        stamps = device.download(counters)[18:].view(np.uint64)
        record.update(extra)
        record["allreduce_us_after_its_start"] = [
            {"counted_complete": round((int(stamps[1 + 2 * i]) - int(stamps[0])) / 1e3, 1),
             "reduced": round((int(stamps[2 + 2 * i]) - int(stamps[0])) / 1e3, 1)}
            for i in range(extra["blocks"])]
    best = min(times)
    if "bytes" in work:
        record["best_GBps"] = work["bytes"] / best / 1e9
    else:
        record["best_TFLOPs"] = work["flop"] / best / 1e12
    print(json.dumps(record))


if __name__ == "__main__":
    main()
