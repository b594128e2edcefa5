"""Benchmark of the native operator path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--ops LIST]

Headline workload (the JSON line's ``value``): row-wise masked softmax fp16 over
X[16384, 4000] with the causal-mod mask, one launch per step, inputs resident in HBM.
With N > 1 (launched under torchrun, one rank per GPU) every rank runs that workload
on its own rows -- rows are independent, no collective -- and ``value`` is the sum over
ranks divided by the slowest rank's time (weak scaling).

The same line carries ``roofline`` (algorithmic bytes per launch / CUDA-event launch
time against the measured HBM copy bandwidth), ``e2e`` (host buffers in pinned memory,
host->device copy + launch + device->host copy inside the timed region, through
``B200Device``), ``cpu_baseline`` (the numpy oracle on a bounded row sample, rank 0 at
N=1 only), ``clocks`` (nvidia-smi samples taken while the kernels ran) and ``ops``: the
other operators of the path (RMSNorm fp32, bf16 GEMM + bias + GELU square and ragged,
causal attention forward, and at N > 1 the tensor-parallel SwiGLU MLP), each with its own
roofline.

``--impl reference`` times the reference's CPU implementation of the headline workload
(the numpy float64 oracle) on the host cores and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS, COLS = 16384, 4000
SOFTMAX_BYTES = 2 * ROWS * COLS * 2          # read X + write Y, fp16
RMS_ROWS, RMS_COLS = 8192, 4096
RMS_BYTES = 2 * RMS_ROWS * RMS_COLS * 4 + RMS_COLS * 4 + RMS_ROWS * 4
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch, from one `ncu --set full` capture of
# `python -m compiler_b200.profile_case <op> --shape ...` per kernel at the bench shape (attention:
# captured at [4,16,4096,128] and scaled by 4, traffic is proportional to batch x heads)
NCU_TRAFFIC = {
    "softmax": 141_064_000,
    "rmsnorm": 212_674_000,
    "gemm_8192": 1_181_803_000,
    "gemm_ragged": 203_472_000,
    "attention": 1_036_044_000,
    "attention_decode": 540_428_000,
}


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            return {k: float(data[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:  # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """SM clock, power and throttle reasons sampled while kernels run: NVML polled from a
    thread every 2 ms (read-only queries), or ``nvidia-smi -lms`` lines where NVML cannot be
    loaded.  Each sample carries the flags hw_slowdown, hw_thermal_slowdown,
    sw_thermal_slowdown, sw_power_cap in that order."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    # nvmlClocksEventReason bits: hw slowdown, hw thermal, sw thermal, sw power cap
    REASON_BITS = (0x8, 0x40, 0x20, 0x4)

    def __init__(self, index: int, uuid: str | None = None):
        self.samples = []
        self.source = None
        self._proc = None
        self._thread = None
        self._index = index
        self._uuid = uuid
        self._stop = threading.Event()

    def start(self):
        if self._start_nvml():
            return
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "25", "-i", str(self._index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.source = "nvidia-smi"
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

    def _start_nvml(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = None
            if self._uuid:
                try:
                    handle = pynvml.nvmlDeviceGetHandleByUUID(self._uuid.encode())
                except Exception:  # noqa: BLE001 - unknown spelling of the id: use the index
                    handle = None
            if handle is None:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self._index)
            max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001 - no NVML here: fall back to nvidia-smi
            return False

        def poll():
            while not self._stop.is_set():
                try:
                    mhz = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                    watts = pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0
                    mask = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                except Exception:  # noqa: BLE001
                    break
                flags = ["Active" if mask & bit else "Not Active" for bit in self.REASON_BITS]
                self.samples.append({"t": time.monotonic(), "sm": mhz, "max": max_mhz,
                                     "power": watts, "flags": flags})
                time.sleep(0.002)

        self.source = "nvml"
        self._thread = threading.Thread(target=poll, daemon=True)
        self._thread.start()
        return True

    def _read(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                self.samples.append({"t": time.monotonic(), "sm": float(parts[0]),
                                     "max": float(parts[1]), "power": float(parts[2]),
                                     "flags": parts[3:7]})
            except ValueError:
                continue

    def stop(self):
        self._stop.set()
        if self._thread is not None and self.source == "nvml":
            self._thread.join(timeout=2)
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()

    def summary(self, t0, t1, label="headline timed region"):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        window = [s for s in self.samples if t0 <= s["t"] <= t1]
        if not window:  # region shorter than the sampling period: use the loaded samples
            busy = [s for s in self.samples if s["power"] > 250.0]
            window, label = (busy or self.samples), "whole run, samples under load"
        if not window:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0,
                    "window": "no clock samples"}
        reasons = sorted({names[i] for s in window for i, f in enumerate(s["flags"])
                          if f.lower().startswith("active")})
        return {"sm_mhz": float(np.median([s["sm"] for s in window])),
                "sm_max_mhz": float(window[0]["max"]), "reasons": reasons,
                "sm_min_mhz": float(min(s["sm"] for s in window)),
                "samples": len(window), "window": label, "source": self.source,
                "power_w_max": float(max(s["power"] for s in window))}


# --------------------------------------------------------------------------- timing
class Dist:
    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.enabled = self.world > 1

    def init(self, torch):
        if self.enabled:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
        self.torch = torch

    def barrier(self):
        if self.enabled:
            import torch.distributed as dist
            dist.barrier()

    def max(self, value: float) -> float:
        if not self.enabled:
            return value
        import torch.distributed as dist
        t = self.torch.tensor([value], dtype=self.torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def finish(self):
        if self.enabled:
            import torch.distributed as dist
            dist.destroy_process_group()


def time_steps(torch, dist, launch, steps, warmup):
    """W untimed steps, then exactly K timed steps between barrier+synchronize pairs.
    Returns (ms per step over the whole region, max over ranks; mean per-launch ms from
    CUDA-event pairs around each launch on the launching stream; wall-clock window)."""
    for i in range(warmup):
        launch(i)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
             for _ in range(steps)]
    t0 = time.monotonic()
    begin.record()
    for i in range(steps):
        pairs[i][0].record()
        launch(warmup + i)
        pairs[i][1].record()
    end.record()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    t1 = time.monotonic()
    region_ms = dist.max(begin.elapsed_time(end)) / steps
    launch_ms = float(np.mean([a.elapsed_time(b) for a, b in pairs]))
    return region_ms, launch_ms, (t0, t1)


GRAPH_LAUNCHES = 100


def time_graph_region(torch, dist, launch_on, steps, warmup):
    """Exactly ``steps`` launches between barrier + synchronize pairs, issued as replays of a
    captured graph of GRAPH_LAUNCHES launches (plus single launches for the remainder) on a
    stream of the library; timed with CUDA events on that stream, max over ranks.
    ``launch_on(stream_handle, i)`` enqueues step i.  Returns (ms per step, wall-clock window)."""
    import ctypes
    from compiler_b200 import graph
    from compiler_b200.runtime import abi
    lib = abi.lib()
    stream = graph.Stream()
    for i in range(warmup):
        launch_on(stream.handle, i)
    stream.synchronize()
    per_graph = min(GRAPH_LAUNCHES, steps)
    with graph.capture(stream) as g:
        for i in range(per_graph):
            launch_on(stream.handle, i)
    g.launch(stream)  # one untimed replay
    stream.synchronize()
    begin, end = ctypes.c_void_p(), ctypes.c_void_p()
    abi.check(lib.b200_event_create(ctypes.byref(begin)))
    abi.check(lib.b200_event_create(ctypes.byref(end)))
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.monotonic()
    abi.check(lib.b200_event_record(begin, stream._ptr))
    for _ in range(steps // per_graph):
        g.launch(stream)
    for i in range(steps % per_graph):
        launch_on(stream.handle, i)
    abi.check(lib.b200_event_record(end, stream._ptr))
    stream.synchronize()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    t1 = time.monotonic()
    ms = ctypes.c_float()
    abi.check(lib.b200_event_elapsed_ms(begin, end, ctypes.byref(ms)))
    lib.b200_event_destroy(begin)
    lib.b200_event_destroy(end)
    abi.check(lib.b200_last_device_status(stream._ptr))
    g.close()
    stream.close()
    return dist.max(ms.value) / steps, (t0, t1)


def roofline(bound, algorithmic, launch_ms, peaks, source, traffic, sustained=False):
    if bound == "hbm":
        achieved = algorithmic / (launch_ms * 1e-3) / 1e9
        peak, unit = peaks["hbm_gbs"], "GB/s"
    else:
        achieved = algorithmic / (launch_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"]
        unit = "TFLOP/s"
    return {"bound": bound, "achieved": round(achieved, 2), "peak": peak, "unit": unit,
            "frac": round(achieved / peak, 4), "peak_source": f"of {source}", "traffic": traffic,
            "algorithmic_per_launch": algorithmic, "launch_ms": round(launch_ms, 5)}


# --------------------------------------------------------------------------- workloads
def bench_softmax(torch, ops, dist, steps, warmup, peaks, source):
    stream = torch.cuda.current_stream().cuda_stream
    nsets = 4  # rotating buffer sets: 4 x 262 MB of traffic between reuses of a buffer > 126 MB L2
    gen = torch.Generator(device="cuda").manual_seed(30 + dist.rank)
    xs = [(torch.randn((ROWS, COLS), generator=gen, device="cuda") * 2).to(torch.float16)
          for _ in range(nsets)]
    ys = [torch.empty_like(x) for x in xs]
    offset = dist.rank * ROWS  # this rank's rows of the N-times-larger job

    def launch_on(handle, i):
        ops.softmax(xs[i % nsets], ys[i % nsets], causal_mod=True, row_offset=offset,
                    stream=handle)

    def launch(i):
        launch_on(stream, i)

    # pass 1: CUDA-event pairs around single launches (reported beside the roofline; the
    # records between launches keep consecutive kernels from overlapping their ramps)
    _, launch_ms, _ = time_steps(torch, dist, launch, min(steps, 500), warmup)
    ops.device_status(stream)
    # pass 2, the timed region of the headline: exactly `steps` launches, replayed from CUDA
    # graphs of GRAPH_LAUNCHES launches each (the loop is launch-latency bound: a 40 us kernel
    # against a few microseconds of host work per launch), CUDA events around the region;
    # region / steps is the average launch duration the roofline uses
    region_ms, window = time_graph_region(torch, dist, launch_on, steps, warmup)
    roof = roofline("hbm", SOFTMAX_BYTES, region_ms, peaks, source, NCU_TRAFFIC["softmax"])
    roof["launch_ms_event_pairs"] = round(launch_ms, 5)
    return {"region_ms": region_ms, "launch_ms": launch_ms, "window": window, "roofline": roof}


def bench_softmax_e2e(dist, steps, warmup):
    """Host buffers -> device -> kernel -> host, every step, through the library's public host
    API (``compiler_b200.pipeline``): the rows are cut into chunks on two streams so the
    two PCIe directions and the kernel overlap.  Timed with the host clock around the call
    (several streams take part; the call returns when the result is in host memory)."""
    from compiler_b200 import pipeline
    from compiler_b200.device import B200Device
    device = B200Device(dist.local_rank)
    rng = np.random.default_rng(30 + dist.rank)
    hx = device.pinned_empty((ROWS, COLS), np.float16)
    hx.array[...] = (rng.standard_normal((ROWS, COLS), dtype=np.float32) * 2).astype(np.float16)
    hy = device.pinned_empty((ROWS, COLS), np.float16)
    pipe = pipeline.RowPipeline(device, ROWS, COLS, "float16", chunks=8, streams=2)
    offset = dist.rank * ROWS

    for _ in range(warmup):
        pipeline.masked_softmax_host(pipe, hx, hy, offset)
    device.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        pipeline.masked_softmax_host(pipe, hx, hy, offset)
    device.synchronize()
    ms = dist.max((time.perf_counter() - t0) * 1e3) / steps
    dist.barrier()
    checksum = float(hy.array[:64].astype(np.float64).sum())  # rows sum to 1 -> 64
    pipe.close()
    return {"value": round(SOFTMAX_BYTES * dist.world / (ms * 1e-3) / 1e9, 2), "unit": "GB/s",
            "h2d_bytes_per_step": ROWS * COLS * 2, "d2h_bytes_per_step": ROWS * COLS * 2,
            "ms_per_step": round(ms, 4), "steps": steps, "chunks": 8, "streams": 2,
            "timer": "host clock around the blocking call",
            "result_check_rowsum64": round(checksum, 3)}


def bench_softmax_unmasked(torch, ops, dist, steps, warmup, peaks, source):
    """The headline's shape without the mask (the reference's softmax.py operator itself):
    every element is read and written, so algorithmic bytes and DRAM traffic coincide."""
    stream = torch.cuda.current_stream().cuda_stream
    nsets = 4
    gen = torch.Generator(device="cuda").manual_seed(35 + dist.rank)
    xs = [(torch.randn((ROWS, COLS), generator=gen, device="cuda") * 2).to(torch.float16)
          for _ in range(nsets)]
    ys = [torch.empty_like(x) for x in xs]

    def launch_on(handle, i):
        ops.softmax(xs[i % nsets], ys[i % nsets], stream=handle)

    _, launch_ms, _ = time_steps(torch, dist, lambda i: launch_on(stream, i), steps, warmup)
    region_ms, window = time_graph_region(torch, dist, launch_on, steps, warmup)
    out = roofline("hbm", SOFTMAX_BYTES, region_ms, peaks, source, None)
    out["launch_ms_event_pairs"] = round(launch_ms, 5)
    out["window"] = window
    out.update({"workload": "softmax_fp16_16384x4000_unmasked", "ms_per_step": round(region_ms, 5),
                "value": round(SOFTMAX_BYTES * dist.world / (region_ms * 1e-3) / 1e9, 2),
                "unit": "GB/s", "gpu_launches": steps})
    return out


def bench_rmsnorm(torch, ops, dist, steps, warmup, peaks, source):
    stream = torch.cuda.current_stream().cuda_stream
    nsets = 4
    gen = torch.Generator(device="cuda").manual_seed(31 + dist.rank)
    xs = [torch.randn((RMS_ROWS, RMS_COLS), generator=gen, device="cuda") for _ in range(nsets)]
    w = torch.rand((RMS_COLS,), generator=gen, device="cuda") + 0.5
    ys = [torch.empty_like(x) for x in xs]
    r = torch.empty((RMS_ROWS,), device="cuda")

    def launch_on(handle, i):
        ops.rmsnorm(xs[i % nsets], w, ys[i % nsets], r, eps=1e-6, stream=handle)

    _, launch_ms, _ = time_steps(torch, dist, lambda i: launch_on(stream, i), steps, warmup)
    region_ms, window = time_graph_region(torch, dist, launch_on, steps, warmup)
    out = roofline("hbm", RMS_BYTES, region_ms, peaks, source, NCU_TRAFFIC["rmsnorm"])
    out["launch_ms_event_pairs"] = round(launch_ms, 5)
    out["window"] = window
    out.update({"workload": "rmsnorm_fp32_8192x4096", "ms_per_step": round(region_ms, 5),
                "value": round(RMS_BYTES * dist.world / (region_ms * 1e-3) / 1e9, 2),
                "unit": "GB/s", "gpu_launches": steps})
    return out


def bench_gemm(torch, ops, dist, steps, warmup, peaks, source, shape, key):
    from compiler_b200.runtime import abi
    stream = torch.cuda.current_stream().cuda_stream
    m, n, k = shape
    nsets = 2  # A, B, C rotate: > 126 MB L2 between reuses
    gen = torch.Generator(device="cuda").manual_seed(32 + dist.rank)
    sets = []
    for _ in range(nsets):
        a = (torch.randn((m, k), generator=gen, device="cuda") / k ** 0.5).to(torch.bfloat16)
        b = (torch.randn((k, n), generator=gen, device="cuda") / k ** 0.5).to(torch.bfloat16)
        sets.append((a, b, torch.empty((m, n), device="cuda", dtype=torch.bfloat16)))
    bias = (torch.randn((n,), generator=gen, device="cuda") * 0.1).to(torch.bfloat16)

    def launch_on(handle, i):
        a, b, c = sets[i % nsets]
        ops.gemm(a, b, c, bias=bias, act=abi.ACT_GELU_TANH, stream=handle)

    _, launch_ms, _ = time_steps(torch, dist, lambda i: launch_on(stream, i), steps, warmup)
    ops.device_status(stream)
    region_ms, window = time_graph_region(torch, dist, launch_on, steps, warmup)
    flops = 2 * m * n * k
    out = roofline("tensor", flops, region_ms, peaks, source, NCU_TRAFFIC[key])
    out["launch_ms_event_pairs"] = round(launch_ms, 5)
    out["window"] = window
    out.update({"workload": f"gemm_bf16_bias_gelu_tanh_{m}x{n}x{k}",
                "ms_per_step": round(region_ms, 5),
                "value": round(flops * dist.world / (region_ms * 1e-3) / 1e12, 2),
                "unit": "TFLOP/s", "gpu_launches": steps})
    return out


def bench_attention(torch, ops, dist, steps, warmup, peaks, source):
    stream = torch.cuda.current_stream().cuda_stream
    z, h, n, d = 8, 32, 4096, 128
    gen = torch.Generator(device="cuda").manual_seed(33 + dist.rank)
    q, k, v = (torch.randn((z, h, n, d), generator=gen, device="cuda").to(torch.bfloat16)
               for _ in range(3))
    o = torch.empty_like(q)
    lse = torch.empty((z, h, n), device="cuda")

    def launch_on(handle, i):
        ops.attention(q, k, v, o, lse=lse, scale=1.0 / d ** 0.5, causal=True, stream=handle)

    _, launch_ms, _ = time_steps(torch, dist, lambda i: launch_on(stream, i), steps, warmup)
    ops.device_status(stream)
    region_ms, window = time_graph_region(torch, dist, launch_on, steps, warmup)
    flops = 4 * z * h * d * n * (n + 1) // 2  # causal-exact: 2 matmuls over the kept triangle
    out = roofline("tensor", flops, region_ms, peaks, source, NCU_TRAFFIC["attention"])
    out["launch_ms_event_pairs"] = round(launch_ms, 5)
    out["window"] = window
    out.update({"workload": "attn_fwd_causal_bf16_8x32x4096x128", "flop_convention": "causal-exact",
                "ms_per_step": round(region_ms, 5),
                "value": round(flops * dist.world / (region_ms * 1e-3) / 1e12, 2),
                "unit": "TFLOP/s", "gpu_launches": steps})
    return out


def bench_attention_decode(torch, ops, dist, steps, warmup, peaks, source):
    """One query row per (batch, head) against a K / V cache of 4096 keys: the K and V of
    8 x 32 heads are 537 MB, read once per launch (four times the L2)."""
    stream = torch.cuda.current_stream().cuda_stream
    rows, n, d = 8 * 32, 4096, 128
    gen = torch.Generator(device="cuda").manual_seed(36 + dist.rank)
    q = torch.randn((rows, d), generator=gen, device="cuda").to(torch.bfloat16)
    k, v = (torch.randn((rows, n, d), generator=gen, device="cuda").to(torch.bfloat16)
            for _ in range(2))
    o = torch.empty_like(q)

    def launch_on(handle, i):
        ops.attention_decode(q, k, v, o, scale=1.0 / d ** 0.5, stream=handle)

    _, launch_ms, _ = time_steps(torch, dist, lambda i: launch_on(stream, i), steps, warmup)
    region_ms, window = time_graph_region(torch, dist, launch_on, steps, warmup)
    nbytes = 2 * rows * n * d * 2
    out = roofline("hbm", nbytes, region_ms, peaks, source, NCU_TRAFFIC["attention_decode"])
    out["launch_ms_event_pairs"] = round(launch_ms, 5)
    out["window"] = window
    out.update({"workload": "attn_decode_bf16_256rows_4096keys_128", "ms_per_step": round(region_ms, 5),
                "value": round(nbytes * dist.world / (region_ms * 1e-3) / 1e9, 2),
                "unit": "GB/s", "gpu_launches": 2 * steps})
    return out


def bench_tp_mlp(torch, dist, steps, warmup, peaks, source, collective="nccl"):
    from compiler_b200 import tp_mlp
    mlp = tp_mlp.TensorParallelMLP.synthetic(hidden=4096, ffn=14336, rank=dist.rank,
                                             world=dist.world, seed=34, collective=collective)
    gen = torch.Generator(device="cuda").manual_seed(35)  # x is replicated: same seed on all ranks
    x = torch.randn((4096, 4096), generator=gen, device="cuda").to(torch.bfloat16)
    y = torch.empty((4096, 4096), device="cuda", dtype=torch.bfloat16)

    def launch(i):
        mlp.forward(x, y)

    region_ms, launch_ms, window = time_steps(torch, dist, launch, steps, warmup)
    flops = 3 * 2 * 4096 * 4096 * 14336
    out = roofline("tensor", flops // dist.world, launch_ms, peaks, source, None)
    out["window"] = window
    out.update({"workload": f"tp_swiglu_mlp_bf16_tp{dist.world}", "scaling": "strong",
                "collective": ("NCCL all-reduce per row chunk, overlapped with the next chunk's GEMM"
                               if collective == "nccl" else
                               "reduce-scatter by peer stores in the GEMM epilogue + sum and "
                               "broadcast kernel"),
                "ms_per_step": round(region_ms, 5),
                "value": round(flops / (region_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "allreduce_bytes_per_rank": 4096 * 4096 * 2,
                "gpu_launches": steps * mlp.kernels_per_forward})
    return out


# --------------------------------------------------------------------------- CPU legs
def cpu_softmax_sample(rows):
    """The numpy oracle on the first `rows` rows of the headline workload."""
    from oracle import oracle
    rng = np.random.default_rng(30)
    x = (rng.standard_normal((rows, COLS), dtype=np.float32) * 2).astype(np.float16)
    t0 = time.perf_counter()
    y = oracle.masked_softmax_ref(x, 0).astype(np.float16)
    return time.perf_counter() - t0, y


def cpu_baseline():
    # about ten seconds of host work: an eighth of the workload's rows per repetition
    rows, elapsed, reps = 2048, 0.0, 0
    best = None
    while elapsed < 10.0 and reps < 64:
        t, _ = cpu_softmax_sample(rows)
        best = t if best is None else min(best, t)
        elapsed += t
        reps += 1
    return {"value": round(2 * rows * COLS * 2 / best / 1e9, 4), "unit": "GB/s", "cores": 1,
            "kind": "port",
            "sample": f"numpy float64 oracle on {rows} of {ROWS} rows x {COLS} cols, best of "
                      f"{reps} ({best:.3f} s); elementwise numpy is single-threaded",
            "host_cores_available": len(os.sched_getaffinity(0))}


def reference_arm(args):
    """Reference arm: the reference's CPU implementation (numpy float64 ``ref``, restated in
    oracle/oracle.py) of the headline workload on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 1024
    for _ in range(max(args.warmup, 1)):
        cpu_softmax_sample(rows)
    times = [cpu_softmax_sample(rows)[0] for _ in range(args.steps)]
    ms = float(np.mean(times)) * 1e3
    value = round(2 * rows * COLS * 2 / (ms * 1e-3) / 1e9, 4)
    line = {
        "impl": "reference", "metric": "masked_softmax_fp16_hbm_throughput", "value": value,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "masked_softmax_fp16_16384x4000",
                   "step": f"numpy oracle on a {rows}-row sample of the workload"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": 1, "kind": "port",
                         "sample": f"{rows} of {ROWS} rows per step; the reference's ref() is "
                                   "single-threaded elementwise numpy"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- main
def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=6000)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", default="native", choices=["native", "reference"])
    parser.add_argument("--ops", default="all",
                        help="comma list of extra operators: softmax_unmasked,rmsnorm,gemm,gemm_ragged,attention,attention_decode,"
                             "tp_mlp,none,all")
    args = parser.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    from compiler_b200 import ops
    from compiler_b200.runtime import abi

    dist = Dist()
    torch.cuda.set_device(dist.local_rank)
    abi.check(abi.lib().b200_set_device(dist.local_rank))
    dist.init(torch)
    peaks, source = load_peaks()
    warmup = max(args.warmup, 3)
    uuid = getattr(torch.cuda.get_device_properties(dist.local_rank), "uuid", None)
    sampler = ClockSampler(dist.local_rank, f"GPU-{uuid}" if uuid is not None else None)
    if dist.rank == 0:
        sampler.start()

    head = bench_softmax(torch, ops, dist, args.steps, warmup, peaks, source)
    e2e = bench_softmax_e2e(dist, min(args.steps, 20), 3)

    wanted = args.ops.split(",")
    extra_steps = max(3, min(args.steps, 20))
    extras = {}

    def want(name):
        if "none" in wanted or not ("all" in wanted or name in wanted):
            return False
        # each operator is timed alone, as the burst peaks it is compared with were: let the
        # board's power average settle after the previous operator's burst
        torch.cuda.synchronize()
        time.sleep(1.0)
        return True

    if want("softmax_unmasked"):
        extras["softmax_unmasked"] = bench_softmax_unmasked(
            torch, ops, dist, max(extra_steps, min(args.steps, 200)), warmup, peaks, source)
    if want("rmsnorm"):
        extras["rmsnorm"] = bench_rmsnorm(torch, ops, dist, max(extra_steps, min(args.steps, 200)),
                                          warmup, peaks, source)
    if want("gemm"):
        extras["gemm"] = bench_gemm(torch, ops, dist, extra_steps, 3, peaks, source,
                                    (8192, 8192, 8192), "gemm_8192")
    if want("gemm_ragged"):
        extras["gemm_ragged"] = bench_gemm(torch, ops, dist, extra_steps, 3, peaks, source,
                                           (4097, 11008, 4096), "gemm_ragged")
    if want("attention"):
        extras["attention"] = bench_attention(torch, ops, dist, max(3, min(args.steps, 10)), 3,
                                              peaks, source)
    if want("attention_decode"):
        extras["attention_decode"] = bench_attention_decode(torch, ops, dist, extra_steps, 3,
                                                            peaks, source)
    if want("tp_mlp") and dist.world > 1:
        extras["tp_mlp"] = bench_tp_mlp(torch, dist, extra_steps, 3, peaks, source)
        if 4096 % (128 * dist.world) == 0:
            try:
                extras["tp_mlp_peer"] = bench_tp_mlp(torch, dist, extra_steps, 3, peaks, source,
                                                     collective="peer")
            except Exception as exc:  # noqa: BLE001 - symmetric memory may be unavailable
                extras["tp_mlp_peer"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}

    baseline = cpu_baseline() if (dist.rank == 0 and dist.world == 1) else None
    if dist.rank != 0:
        for extra in extras.values():
            extra.pop("window", None)
    if dist.rank == 0:
        sampler.stop()
        clocks = sampler.summary(*head["window"])
        for extra in extras.values():  # each operator's own clock record
            if "window" in extra:
                extra["clocks"] = sampler.summary(*extra.pop("window"),
                                                  label="this operator's timed region")
        value = SOFTMAX_BYTES * dist.world / (head["region_ms"] * 1e-3) / 1e9
        line = {
            "metric": "masked_softmax_fp16_hbm_throughput", "value": round(value, 2),
            "unit": "GB/s", "n_gpus": dist.world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": round(head["region_ms"], 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "masked_softmax_fp16_16384x4000",
                       "mask": "col > row % 4000 -> -inf", "io_dtype": "f16",
                       "rows_per_gpu": ROWS, "sharding": "rows, no collective",
                       "l2": "4 rotating buffer sets (1.05 GB) between reuses, L2 is 126 MB",
                       "launching": f"CUDA graphs of {GRAPH_LAUNCHES} launches"},
            "roofline": head["roofline"], "e2e": e2e, "gpu_launches": args.steps,
            "clocks": clocks, "ops": extras,
        }
        if baseline is not None:
            line["cpu_baseline"] = baseline
        print(json.dumps(line))
    dist.finish()


if __name__ == "__main__":
    main()
