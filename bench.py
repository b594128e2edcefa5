"""Benchmark of the native operator path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--ops LIST]

Headline workload (the JSON line's ``value``): row-wise masked softmax fp16 over
X[16384, 4000] with the causal-mod mask, inputs resident in HBM.  One STEP is one replay of a
CUDA graph of 100 launches (100 passes over the workload on rotating buffer sets), so K = 20
steps are a timed region of about 80 ms whatever K is.  With N > 1 (launched under torchrun,
one rank per GPU) every rank runs that workload on its own rows -- rows are independent, no
collective -- and ``value`` is the sum over ranks divided by the slowest rank's time (weak
scaling); the ``strong`` block of the same line times the BASELINE tensor split N ways.

The same line carries ``roofline`` (algorithmic bytes per launch / average launch duration
against the measured HBM copy bandwidth, plus the same with the bytes the mask makes
necessary), ``e2e`` (host buffers in pinned memory, host->device copy + launch + device->host
copy inside the timed region, through the library's host API), ``cpu_baseline`` (the numpy
oracle over the whole workload on the host cores, rank 0 at N=1 only), ``clocks`` (samples
taken while the kernels ran) and ``ops``: the other operators of the path (RMSNorm fp32, bf16
GEMM + bias + GELU square and ragged, causal attention forward, decode attention, the sibling
kernels, and the tensor-parallel SwiGLU MLP with a parity check and per-phase times), each
with its own roofline.

``--impl reference`` times the reference's CPU implementation of the headline workload
(the numpy float64 oracle, whole workload per step) on the host cores and prints the same
line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS, COLS = 16384, 4000
SOFTMAX_BYTES = 2 * ROWS * COLS * 2          # read X + write Y, fp16 (the algorithmic count)
RMS_ROWS, RMS_COLS = 8192, 4096
RMS_BYTES = 2 * RMS_ROWS * RMS_COLS * 4 + RMS_COLS * 4 + RMS_ROWS * 4
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
LAUNCHES_PER_STEP = 100                       # launches in the graph that is one step

# dram__bytes_read.sum + dram__bytes_write.sum per launch from ncu captures of
# `python -m compiler_b200.profile_case <op> --shape ...` at the bench shape (attention:
# captured at [4,16,4096,128] and scaled by 4, traffic is proportional to batch x heads).
# softmax: launches 5..8 of a run over four rotating buffer sets, i.e. with the write-backs of
# the launches before them -- the steady state, not a first launch into a clean L2.
NCU_TRAFFIC = {
    "softmax": 197_000_000,
    "rmsnorm": 212_674_000,
    "gemm_8192": 1_181_803_000,
    "gemm_ragged": 203_472_000,
    "attention": 1_036_044_000,
    "attention_decode": 540_428_000,
}


def softmax_necessary_bytes(rows=ROWS, cols=COLS, row_offset=0):
    """Bytes the mask makes necessary: row g keeps g % cols + 1 columns (2 B each) and every
    output element is written."""
    kept = (np.arange(rows, dtype=np.int64) + row_offset) % cols + 1
    return int(kept.sum()) * 2 + rows * cols * 2


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

    def _reduce(self, value: float, op_name: str) -> float:
        if not self.enabled:
            return value
        import torch.distributed as dist
        t = self.torch.tensor([value], dtype=self.torch.float64, device="cuda")
        dist.all_reduce(t, op=getattr(dist.ReduceOp, op_name))
        return float(t.item())

    def max(self, value: float) -> float:
        return self._reduce(value, "MAX")

    def min(self, value: float) -> float:
        return self._reduce(value, "MIN")

    def sum(self, value: float) -> float:
        return self._reduce(value, "SUM")

    def finish(self):
        if self.enabled:
            import torch.distributed as dist
            dist.destroy_process_group()


def time_event_pairs(torch, dist, launch, launches, warmup):
    """Mean duration of single launches, each between its own pair of CUDA events on the
    launching stream (the records between launches keep consecutive kernels from overlapping
    their ramp-up and tail).  Also returns the whole region / launches (max over ranks) and
    the wall-clock window."""
    for i in range(warmup):
        launch(i)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
             for _ in range(launches)]
    t0 = time.monotonic()
    begin.record()
    for i in range(launches):
        pairs[i][0].record()
        launch(warmup + i)
        pairs[i][1].record()
    end.record()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    t1 = time.monotonic()
    region_ms = dist.max(begin.elapsed_time(end)) / launches
    launch_ms = float(np.mean([a.elapsed_time(b) for a, b in pairs]))
    return region_ms, launch_ms, (t0, t1)


def time_back_to_back(torch, dist, launch, launches, warmup):
    """``launches`` launches enqueued back to back between ONE pair of CUDA events (no records
    in between), after ``warmup`` untimed ones and a barrier: the region / launches, max over
    ranks, and the wall-clock window."""
    for i in range(warmup):
        launch(i)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.monotonic()
    begin.record()
    for i in range(launches):
        launch(warmup + i)
    end.record()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    t1 = time.monotonic()
    return dist.max(begin.elapsed_time(end)) / launches, (t0, t1)


def time_graph_steps(torch, dist, launch_on, steps, warmup, per_step):
    """``warmup`` untimed steps, then exactly ``steps`` timed steps between barrier +
    synchronize pairs.  A step is one replay of a captured graph of ``per_step`` launches on a
    stream of the library; CUDA events on that stream bracket the region, max over ranks.
    ``launch_on(stream_handle, i)`` enqueues launch i.  Returns (ms per step, window)."""
    import ctypes
    from compiler_b200 import graph
    from compiler_b200.runtime import abi
    lib = abi.lib()
    stream = graph.Stream()
    for i in range(3):
        launch_on(stream.handle, i)
    stream.synchronize()
    with graph.capture(stream) as g:
        for i in range(per_step):
            launch_on(stream.handle, i)
    for _ in range(max(1, warmup)):
        g.launch(stream)
    stream.synchronize()
    begin, end = ctypes.c_void_p(), ctypes.c_void_p()
    abi.check(lib.b200_event_create(ctypes.byref(begin)))
    abi.check(lib.b200_event_create(ctypes.byref(end)))
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.monotonic()
    abi.check(lib.b200_event_record(begin, stream._ptr))
    for _ in range(steps):
        g.launch(stream)
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
    out = {"bound": bound, "achieved": round(achieved, 2), "peak": peak, "unit": unit,
           "frac": round(achieved / peak, 4), "peak_source": f"of {source}", "traffic": traffic,
           "algorithmic_per_launch": algorithmic, "launch_ms": round(launch_ms, 5)}
    if bound == "tensor":
        out["peak_kind"] = "sustained" if sustained else "burst"
    return out


def hbm_op(torch, dist, launch_on, steps, warmup, nbytes, peaks, source, traffic, workload,
           launches_per_launch=1):
    """A bandwidth-bound operator: event-pair launches first, then ``steps`` steps of
    LAUNCHES_PER_STEP graph-replayed launches (the figure the roofline uses)."""
    stream = torch.cuda.current_stream().cuda_stream
    _, pair_ms, _ = time_event_pairs(torch, dist, lambda i: launch_on(stream, i), 50, 5)
    step_ms, window = time_graph_steps(torch, dist, launch_on, steps, warmup, LAUNCHES_PER_STEP)
    launch_ms = step_ms / LAUNCHES_PER_STEP
    out = roofline("hbm", nbytes, launch_ms, peaks, source, traffic)
    out["launch_ms_event_pairs"] = round(pair_ms, 5)
    out["frac_event_pairs"] = round(nbytes / (pair_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
    out["window"] = window
    out.update({"workload": workload, "ms_per_step": round(step_ms, 4), "steps": steps,
                "launches_per_step": LAUNCHES_PER_STEP,
                "value": round(nbytes * dist.world / (launch_ms * 1e-3) / 1e9, 2),
                "unit": "GB/s",
                "gpu_launches": steps * LAUNCHES_PER_STEP * launches_per_launch})
    return out


def tensor_op(torch, dist, launch_on, launches, flops, peaks, source, traffic, workload,
              sustained_seconds=1.5):
    """A tensor-core-bound operator.  ``burst``: ``launches`` graph-replayed launches after
    a pause, compared with the burst peak (the cuBLAS figure that was timed the same way);
    ``sustained``: about ``sustained_seconds`` of back-to-back launches under the power cap,
    compared with the sustained peak."""
    stream = torch.cuda.current_stream().cuda_stream
    _, pair_ms, _ = time_event_pairs(torch, dist, lambda i: launch_on(stream, i),
                                     min(launches, 10), 3)
    torch.cuda.synchronize()
    time.sleep(1.0)  # let the board's power average settle: the burst peak was taken that way
    step_ms, window = time_graph_steps(torch, dist, launch_on, 1, 1, launches)
    launch_ms = step_ms / launches
    out = roofline("tensor", flops, launch_ms, peaks, source, traffic)
    out["launch_ms_event_pairs"] = round(pair_ms, 5)
    out["window"] = window
    out.update({"workload": workload, "ms_per_step": round(launch_ms, 5),
                "value": round(flops * dist.world / (launch_ms * 1e-3) / 1e12, 2),
                "unit": "TFLOP/s", "gpu_launches": launches})
    if sustained_seconds > 0:
        per_step = 20
        steps = max(2, int(sustained_seconds * 1e3 / (launch_ms * per_step)) + 1)
        s_ms, s_window = time_graph_steps(torch, dist, launch_on, steps, 2, per_step)
        s_launch = s_ms / per_step
        rate = flops / (s_launch * 1e-3) / 1e12
        out["sustained"] = {"achieved": round(rate, 2), "peak": peaks["bf16_tflops_sustained"],
                            "frac": round(rate / peaks["bf16_tflops_sustained"], 4),
                            "launch_ms": round(s_launch, 5), "launches": steps * per_step,
                            "seconds": round(s_ms * steps * 1e-3, 3), "window": s_window}
        out["gpu_launches"] += steps * per_step
    return out


# --------------------------------------------------------------------------- workloads
def softmax_buffers(torch, rows, seed, nsets=4):
    """Rotating buffer sets: 4 x 262 MB of traffic between reuses of a buffer > 126 MB L2."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    xs = [(torch.randn((rows, COLS), generator=gen, device="cuda") * 2).to(torch.float16)
          for _ in range(nsets)]
    return xs, [torch.empty_like(x) for x in xs]


def check_softmax_rows(torch, dist, ops, x, y, offset, sample):
    """Oracle check of a few rows of one launch (outside every timed region)."""
    from oracle import oracle
    y.zero_()
    ops.softmax(x, y, causal_mod=True, row_offset=offset,
                stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    worst, ok = 0.0, True
    for r in sample:
        got = y[r:r + 1].float().cpu().numpy().astype(np.float64)
        ref = oracle.masked_softmax_ref(x[r:r + 1].cpu().numpy(), offset + r)
        err = float(np.abs(got - ref).max())
        worst = max(worst, err)
        keep = (offset + r) % COLS + 1
        ok = ok and bool(np.isclose(got, ref, rtol=1e-2, atol=1e-2).all()) \
            and not got[0, keep:].any()
    return {"ok": bool(dist.min(1.0 if ok else 0.0) == 1.0),
            "max_abs_err": dist.max(worst), "rows_per_rank": len(sample),
            "oracle": "masked_softmax_ref, rtol = atol = 1e-2, masked outputs exactly 0"}


def bench_softmax(torch, ops, dist, steps, warmup, peaks, source):
    xs, ys = softmax_buffers(torch, ROWS, 30 + dist.rank)
    offset = dist.rank * ROWS  # this rank's rows of the N-times-larger job
    nsets = len(xs)

    def launch_on(handle, i):
        ops.softmax(xs[i % nsets], ys[i % nsets], causal_mod=True, row_offset=offset,
                    stream=handle)

    out = hbm_op(torch, dist, launch_on, steps, warmup, SOFTMAX_BYTES, peaks, source,
                 NCU_TRAFFIC["softmax"], "masked_softmax_fp16_16384x4000")
    necessary = softmax_necessary_bytes(ROWS, COLS, offset)
    rate = necessary / (out["launch_ms"] * 1e-3) / 1e9
    out.update({"necessary_bytes_per_launch": necessary, "achieved_dram": round(rate, 2),
                "frac_dram": round(rate / peaks["hbm_gbs"], 4),
                "note": "frac counts the whole tensor read and written (the algorithmic "
                        "figure); frac_dram counts the bytes the mask makes necessary (kept "
                        "columns read, every output written), which is what crosses HBM"})
    out["parity"] = check_softmax_rows(torch, dist, ops, xs[0], ys[0], offset,
                                       [0, 1, 3999 - offset % COLS, ROWS - 1])
    return out


def bench_softmax_strong(torch, ops, dist, steps, warmup, peaks, source):
    """The BASELINE tensor [16384, 4000] split into N contiguous row blocks, one per rank
    (global row offsets), same protocol: what the fixed problem costs on N GPUs."""
    rows = ROWS // dist.world
    xs, ys = softmax_buffers(torch, rows, 40 + dist.rank, nsets=4 * dist.world)
    offset = dist.rank * rows
    nsets = len(xs)

    def launch_on(handle, i):
        ops.softmax(xs[i % nsets], ys[i % nsets], causal_mod=True, row_offset=offset,
                    stream=handle)

    step_ms, _ = time_graph_steps(torch, dist, launch_on, steps, warmup, LAUNCHES_PER_STEP)
    launch_ms = step_ms / LAUNCHES_PER_STEP
    rate = SOFTMAX_BYTES / (launch_ms * 1e-3) / 1e9
    return {"scaling": "strong", "rows_per_gpu": rows, "launch_ms": round(launch_ms, 5),
            "value": round(rate, 2), "unit": "GB/s",
            "frac_of_n_gpus": round(rate / (peaks["hbm_gbs"] * dist.world), 4),
            "parity": check_softmax_rows(torch, dist, ops, xs[0], ys[0], offset,
                                         [0, 1, rows // 2, rows - 1])}


def _copy_rates(device, dist, hx, hy, x, y, reps=5):
    """Pinned host <-> device copies alone, all ranks at once: what the host side gives each
    rank with nothing else in the way (GB/s per rank, slowest rank)."""
    from compiler_b200.runtime import abi
    lib = abi.lib()
    rates = {}
    for name in ("h2d", "d2h"):
        device.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            if name == "h2d":
                abi.check(lib.b200_memcpy_h2d(x.ptr, hx.ptr, x.nbytes, device.stream))
            else:
                abi.check(lib.b200_memcpy_d2h(hy.ptr, y.ptr, y.nbytes, device.stream))
        device.synchronize()
        seconds = dist.max(time.perf_counter() - t0) / reps
        dist.barrier()
        rates[name] = round(x.nbytes / seconds / 1e9, 2)
    # both directions at once on two streams (what a pipelined step asks of the link)
    from compiler_b200 import graph
    inbound, outbound = graph.Stream(), graph.Stream()
    device.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(reps):
        abi.check(lib.b200_memcpy_h2d(x.ptr, hx.ptr, x.nbytes, inbound.handle))
        abi.check(lib.b200_memcpy_d2h(hy.ptr, y.ptr, y.nbytes, outbound.handle))
    inbound.synchronize()
    outbound.synchronize()
    seconds = dist.max(time.perf_counter() - t0) / reps
    dist.barrier()
    inbound.close()
    outbound.close()
    rates["both_at_once_each"] = round(x.nbytes / seconds / 1e9, 2)
    return rates


def bench_softmax_e2e(dist, steps, warmup):
    """Host buffers -> device -> kernel -> host, every step, through the library's public host
    API (``compiler_b200.pipeline``).  Two schedules are timed, the same blocking call either
    way.  ``direct`` (the headline): ONE launch whose loads read the rows from the page-locked
    host buffer and whose stores write the result into the page-locked host buffer -- no
    staging copy; what crosses PCIe inbound is what the kernel loads, the kept columns of
    every row.  ``staged_copies``: the rows cut into chunks on two streams, copy engine in,
    kernel, copy engine out, so that the two PCIe directions and the kernel overlap.  Timed
    with the host clock around the call (it returns when the result is in host memory)."""
    from compiler_b200 import pipeline
    from compiler_b200.device import B200Device
    device = B200Device(dist.local_rank)
    rng = np.random.default_rng(30 + dist.rank)
    hx = device.pinned_empty((ROWS, COLS), np.float16)
    hx.array[...] = (rng.standard_normal((ROWS, COLS), dtype=np.float32) * 2).astype(np.float16)
    hy = device.pinned_empty((ROWS, COLS), np.float16)
    offset = dist.rank * ROWS
    nbytes = ROWS * COLS * 2

    def timed(pipe):
        hy.array[...] = 0
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
        # rows sum to 1 -> 64; the last row of the block keeps (offset + ROWS - 1) % COLS + 1
        # columns, everything after them is zero
        checksum = float(hy.array[:64].astype(np.float64).sum())
        keep = (offset + ROWS - 1) % COLS + 1
        tail_zero = bool(not hy.array[-1, keep:].any()) and float(hy.array[-1, :keep].sum()) > 0.9
        return ms, round(checksum, 3), tail_zero

    pipe = pipeline.RowPipeline(device, ROWS, COLS, "float16", chunks=8, streams=2)
    staged_ms, staged_sum, staged_tail = timed(pipe)
    copies = _copy_rates(device, dist, hx, hy, pipe.x, pipe.y)
    pipe.close()
    pipe = pipeline.RowPipeline(device, ROWS, COLS, "float16", direct=True)
    ms, checksum, tail = timed(pipe)
    pipe.close()
    loaded = softmax_necessary_bytes(ROWS, COLS, offset) - nbytes   # the kept columns
    rate = lambda t: round(SOFTMAX_BYTES * dist.world / (t * 1e-3) / 1e9, 2)  # noqa: E731
    return {"value": rate(ms), "unit": "GB/s",
            "schedule": "direct: one launch on the page-locked host buffers, no staging copy",
            "h2d_bytes_per_step": loaded, "d2h_bytes_per_step": nbytes,
            "h2d_note": "bytes the kernel's loads fetch from host memory (the kept columns "
                        "of each row); the host tensor is %d B" % nbytes,
            "ms_per_step": round(ms, 4), "steps": steps,
            "timer": "host clock around the blocking call",
            "result_check_rowsum64": checksum, "result_check_last_row": tail,
            "staged_copies": {"value": rate(staged_ms), "unit": "GB/s",
                              "ms_per_step": round(staged_ms, 4), "chunks": 8, "streams": 2,
                              "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
                              "result_check_rowsum64": staged_sum,
                              "result_check_last_row": staged_tail},
            "copy_only_gbs_per_rank": copies,
            "copy_bound_ms": round(nbytes / (copies["both_at_once_each"] * 1e6), 4),
            "limit": "PCIe: every step brings the result (131 MB per rank) out and the input "
                     "in.  copy_only_gbs_per_rank is what the copy engines get when all "
                     "ranks copy at once (one direction at a time, and both directions at "
                     "once), copy_bound_ms the time both whole tensors take at once with no "
                     "kernel and no chunking"}


def bench_softmax_unmasked(torch, ops, dist, steps, warmup, peaks, source):
    """The headline's shape without the mask (the reference's softmax.py operator itself):
    every element is read and written, so algorithmic bytes and DRAM traffic coincide."""
    xs, ys = softmax_buffers(torch, ROWS, 35 + dist.rank)
    nsets = len(xs)

    def launch_on(handle, i):
        ops.softmax(xs[i % nsets], ys[i % nsets], stream=handle)

    return hbm_op(torch, dist, launch_on, steps, warmup, SOFTMAX_BYTES, peaks, source, None,
                  "softmax_fp16_16384x4000_unmasked")


def bench_rmsnorm(torch, ops, dist, steps, warmup, peaks, source, strong=False):
    rows = RMS_ROWS // dist.world if strong else RMS_ROWS
    nsets = 4 * (dist.world if strong else 1)
    gen = torch.Generator(device="cuda").manual_seed(31 + dist.rank)
    xs = [torch.randn((rows, RMS_COLS), generator=gen, device="cuda") for _ in range(nsets)]
    w = torch.rand((RMS_COLS,), generator=gen, device="cuda") + 0.5
    ys = [torch.empty_like(x) for x in xs]
    r = torch.empty((rows,), device="cuda")

    def launch_on(handle, i):
        ops.rmsnorm(xs[i % nsets], w, ys[i % nsets], r, eps=1e-6, stream=handle)

    if strong:
        step_ms, _ = time_graph_steps(torch, dist, launch_on, steps, warmup, LAUNCHES_PER_STEP)
        launch_ms = step_ms / LAUNCHES_PER_STEP
        rate = RMS_BYTES / (launch_ms * 1e-3) / 1e9
        return {"scaling": "strong", "rows_per_gpu": rows, "launch_ms": round(launch_ms, 5),
                "value": round(rate, 2), "unit": "GB/s",
                "frac_of_n_gpus": round(rate / (peaks["hbm_gbs"] * dist.world), 4)}
    return hbm_op(torch, dist, launch_on, steps, warmup, RMS_BYTES, peaks, source,
                  NCU_TRAFFIC["rmsnorm"], "rmsnorm_fp32_8192x4096")


def bench_gemm(torch, ops, dist, launches, peaks, source, shape, key, strong=False):
    from compiler_b200.runtime import abi
    m_full, n, k = shape
    m = -(-m_full // dist.world) if strong else m_full   # row blocks of A / C
    nsets = 2 if not strong else 2 * dist.world  # A, B, C rotate: > 126 MB L2 between reuses
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

    flops = 2 * m_full * n * k
    if strong:
        time.sleep(1.0)
        step_ms, _ = time_graph_steps(torch, dist, launch_on, 1, 1, launches)
        launch_ms = step_ms / launches
        rate = flops / (launch_ms * 1e-3) / 1e12
        return {"scaling": "strong", "rows_per_gpu": m, "launch_ms": round(launch_ms, 5),
                "value": round(rate, 2), "unit": "TFLOP/s",
                "frac_of_n_gpus": round(rate / (peaks["bf16_tflops"] * dist.world), 4)}
    return tensor_op(torch, dist, launch_on, launches, flops, peaks, source, NCU_TRAFFIC[key],
                     f"gemm_bf16_bias_gelu_tanh_{m_full}x{n}x{k}",
                     sustained_seconds=1.5 if key == "gemm_8192" else 0)


def bench_attention(torch, ops, dist, launches, peaks, source, strong=False):
    z_full, h, n, d = 8, 32, 4096, 128
    z = max(1, z_full // dist.world) if strong else z_full  # batch x heads blocks
    gen = torch.Generator(device="cuda").manual_seed(33 + dist.rank)
    q, k, v = (torch.randn((z, h, n, d), generator=gen, device="cuda").to(torch.bfloat16)
               for _ in range(3))
    o = torch.empty_like(q)
    lse = torch.empty((z, h, n), device="cuda")

    def launch_on(handle, i):
        ops.attention(q, k, v, o, lse=lse, scale=1.0 / d ** 0.5, causal=True, stream=handle)

    flops = 4 * z_full * h * d * n * (n + 1) // 2  # causal-exact: 2 matmuls over the kept triangle
    if strong:
        time.sleep(1.0)
        step_ms, _ = time_graph_steps(torch, dist, launch_on, 1, 1, launches)
        launch_ms = step_ms / launches
        rate = flops / (launch_ms * 1e-3) / 1e12
        return {"scaling": "strong", "batch_per_gpu": z, "launch_ms": round(launch_ms, 5),
                "value": round(rate, 2), "unit": "TFLOP/s",
                "frac_of_n_gpus": round(rate / (peaks["bf16_tflops"] * dist.world), 4)}
    out = tensor_op(torch, dist, launch_on, launches, flops, peaks, source,
                    NCU_TRAFFIC["attention"], "attn_fwd_causal_bf16_8x32x4096x128")
    out["flop_convention"] = "causal-exact"
    return out


def bench_attention_decode(torch, ops, dist, steps, warmup, peaks, source):
    """One query row per (batch, head) against a K / V cache of 4096 keys: the K and V of
    8 x 32 heads are 537 MB, read once per launch (four times the L2)."""
    rows, n, d = 8 * 32, 4096, 128
    gen = torch.Generator(device="cuda").manual_seed(36 + dist.rank)
    q = torch.randn((rows, d), generator=gen, device="cuda").to(torch.bfloat16)
    k, v = (torch.randn((rows, n, d), generator=gen, device="cuda").to(torch.bfloat16)
            for _ in range(2))
    o = torch.empty_like(q)

    def launch_on(handle, i):
        ops.attention_decode(q, k, v, o, scale=1.0 / d ** 0.5, stream=handle)

    nbytes = 2 * rows * n * d * 2
    return hbm_op(torch, dist, launch_on, steps, warmup, nbytes, peaks, source,
                  NCU_TRAFFIC["attention_decode"], "attn_decode_bf16_256rows_4096keys_128",
                  launches_per_launch=2)


# --------------------------------------------------------------------------- TP MLP
MLP_M, MLP_HIDDEN, MLP_FFN = 4096, 4096, 14336


def _mlp_expected_rows(torch, dist, mlp, x, rows):
    """float64 oracle of the selected rows of y from the gathered weight shards (rank 0
    computes, every rank receives)."""
    import torch.distributed as tdist
    from oracle import oracle

    def gathered(t, dim):
        if not dist.enabled:
            return t
        parts = [torch.empty_like(t) for _ in range(dist.world)]
        tdist.all_gather(parts, t.contiguous())
        return torch.cat(parts, dim=dim)

    wg, wu, wd = gathered(mlp.wg, 1), gathered(mlp.wu, 1), gathered(mlp.wd, 0)
    expected = torch.empty((len(rows), MLP_HIDDEN), dtype=torch.float64, device="cuda")
    if dist.rank == 0:
        host = lambda t: t.float().cpu().numpy()  # noqa: E731
        ref = oracle.swiglu_mlp_ref(host(x[rows]), host(wg), host(wu), host(wd))
        expected.copy_(torch.from_numpy(ref))
    del wg, wu, wd
    if dist.enabled:
        tdist.broadcast(expected, src=0)
    return expected.cpu().numpy()


def bench_tp_mlp(torch, ops, dist, launches, peaks, source, collective, **options):
    """y = (silu(x Wg) * (x Wu)) Wd with the ffn dimension sharded over the ranks (strong
    scaling: the problem is fixed).  Outside the timed region every rank compares a spread of
    rows of ITS y with the float64 oracle of the unsharded MLP, and one more pass records a
    CUDA event after each phase."""
    from compiler_b200 import tp_mlp
    mlp = tp_mlp.TensorParallelMLP.synthetic(hidden=MLP_HIDDEN, ffn=MLP_FFN, rank=dist.rank,
                                             world=dist.world, seed=34, collective=collective,
                                             **options)
    gen = torch.Generator(device="cuda").manual_seed(35)  # x is replicated: same seed on all ranks
    x = torch.randn((MLP_M, MLP_HIDDEN), generator=gen, device="cuda").to(torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    result = {}
    # the NCCL path (and one GPU) writes into a caller's buffer; the peer and in-switch paths
    # return their own symmetric output buffer
    y_buf = (torch.empty((MLP_M, MLP_HIDDEN), device="cuda", dtype=torch.bfloat16)
             if (collective == "nccl" or not dist.enabled) else None)

    def launch(i):
        result["y"] = mlp.forward(x, y_buf)

    _, pair_ms, _ = time_event_pairs(torch, dist, launch, launches, 3)
    # the figure of the line: forwards enqueued back to back, as a model's layers are (the
    # event records of the pass above put a few microseconds between consecutive forwards)
    region_ms, window = time_back_to_back(torch, dist, launch, launches, 3)
    ops.device_status(stream)

    # ---- parity: first and last row of every owner's block, tile edges, against the oracle
    block = MLP_M // max(dist.world, 1)
    rows = sorted({r for k in range(dist.world) for r in (k * block, (k + 1) * block - 1)}
                  | {127, 128, 255, 256, MLP_M // 2 + 3})
    result["y"].zero_()
    torch.cuda.synchronize()
    dist.barrier()
    y = mlp.forward(x, y_buf)
    torch.cuda.synchronize()
    ops.device_status(stream)
    got = y[rows].float().cpu().numpy().astype(np.float64)
    expected = _mlp_expected_rows(torch, dist, mlp, x, rows)
    err = float(np.abs(got - expected).max())
    ok = bool(np.isclose(got, expected, rtol=2e-2, atol=2e-2).all())
    parity = {"ok": bool(dist.min(1.0 if ok else 0.0) == 1.0), "max_abs_err": dist.max(err),
              "rows": len(rows), "checked_on": "every rank's own output",
              "oracle": "swiglu_mlp_ref (float64, unsharded), rtol = atol = 2e-2"}

    # ---- per-phase times: events after each phase of `launches` further passes, enqueued
    # back to back (no synchronisation between passes, so that the host's launch latency is
    # hidden behind the device's work as it is in the timed loop) and read at the end
    passes = []
    for _ in range(launches):
        marks = [torch.cuda.Event(enable_timing=True)]
        marks[0].record()
        labels = []

        def mark(name, marks=marks, labels=labels):
            event = torch.cuda.Event(enable_timing=True)
            event.record()
            marks.append(event)
            labels.append(name)

        mlp.forward(x, y_buf, mark=mark)
        passes.append((marks, labels))
    torch.cuda.synchronize()
    names = passes[-1][1]
    samples = [[m[i].elapsed_time(m[i + 1]) for i in range(len(names))] for m, _ in passes[1:]]
    phases = {name: round(dist.max(float(np.mean([s[i] for s in samples]))), 5)
              for i, name in enumerate(names)}

    flops = 3 * 2 * MLP_M * MLP_HIDDEN * MLP_FFN
    out = roofline("tensor", flops // dist.world, region_ms, peaks, source, None)
    out["launch_ms_event_pairs"] = round(pair_ms, 5)
    out["window"] = window
    described = {
        "nccl": "fp32 partials, NCCL all-reduce per row chunk overlapped with the next chunk's GEMM",
        "peer": "reduce-scatter by peer stores in the GEMM epilogue (float16 partials) + sum and "
                "broadcast kernel",
        "nvls": f"{str(mlp.partial_dtype).rsplit('.', 1)[-1]} partials in symmetric memory, "
                "in-switch sum and broadcast (multimem.ld_reduce / multimem.st), barriers "
                "inside the kernel"
                + (f"; the all-reduce kernel is the programmatic dependent of the "
                   f"down-projection and takes each of {mlp.overlap_blocks} blocks of rows as "
                   "soon as every rank's GEMM has counted it complete"
                   if mlp.overlap_blocks > 0 else ""),
        "pull": "float16 partials in symmetric memory, summed by plain peer loads and "
                "broadcast by peer stores, barriers inside the kernel"
                + (f"; the MLP runs in {mlp.row_splits} blocks of rows, a block's all-reduce "
                   "beside both projections of the next block" if mlp.row_splits > 1 else "")
                + (f"; the all-reduce kernel is the programmatic dependent of the "
                   f"down-projection and takes each of {mlp.overlap_blocks} blocks of rows as "
                   "soon as every rank's GEMM has counted it complete"
                   if mlp.overlap_blocks > 0 else ""),
        "none": "one GPU: the two GEMMs alone (anchor of the strong-scaling curve)",
    }
    partial_bytes = MLP_M * MLP_HIDDEN * (4 if collective == "nccl"
                                          else mlp.partial_dtype.itemsize)
    out.update({"workload": f"tp_swiglu_mlp_bf16_tp{dist.world}", "scaling": "strong",
                "collective": described[collective if dist.enabled else "none"],
                "ms_per_step": round(region_ms, 5),
                "value": round(flops / (region_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "allreduce_bytes_per_rank": partial_bytes if dist.enabled else 0,
                "parity": parity, "phases_ms": phases,
                "timing": "forwards enqueued back to back between one pair of CUDA events, "
                          "max over ranks; launch_ms_event_pairs: each forward between its own "
                          "pair",
                # two warm-ups of 3, the event-pair pass, the back-to-back pass, the parity
                # forward and the per-phase passes
                "gpu_launches": (6 + 3 * launches + 1) * mlp.kernels_per_forward})
    if not parity["ok"]:
        out["value"] = None
        out["invalid"] = "the result does not match the oracle; the rate is withheld"
    return out


def bench_allreduce(torch, dist, launches=30):
    """The all-reduce kernels of the TP MLP alone: a [4096, 4096] float16 buffer in symmetric
    memory reduced in place to bfloat16 (the kernels' own barriers on), and a quarter of it;
    CUDA-event pairs around single launches, mean, max over ranks.  NCCL's all-reduce of the
    same bytes is timed beside them."""
    import ctypes
    import torch.distributed as tdist
    import torch.distributed._symmetric_memory as symm_mem
    from compiler_b200.runtime import abi
    lib = abi.lib()
    world, rank = dist.world, dist.rank
    count = MLP_M * MLP_HIDDEN
    group = tdist.group.WORLD
    buf = symm_mem.empty((MLP_M, MLP_HIDDEN), dtype=torch.float16, device="cuda")
    handle = symm_mem.rendezvous(buf, group=group)
    pad = symm_mem.empty((lib.b200_signal_pad_bytes() // 4,), dtype=torch.int32, device="cuda")
    pad.zero_()
    pad_handle = symm_mem.rendezvous(pad, group=group)
    torch.cuda.synchronize()
    pad_handle.barrier(channel=0)
    torch.cuda.synchronize()
    pointers = ctypes.c_void_p * world
    pads = pointers(*[int(p) for p in pad_handle.buffer_ptrs])
    ptrs = pointers(*[int(p) for p in handle.buffer_ptrs])
    f16, bf16 = abi.DTYPE_CODES["float16"], abi.DTYPE_CODES["bfloat16"]
    stream = torch.cuda.current_stream().cuda_stream
    epoch = [0]
    multicast = int(getattr(handle, "multicast_ptr", 0) or 0)

    def peer_loads(n):
        epoch[0] += 1
        abi.check(lib.b200_peer_allreduce(ptrs, f16, ptrs, bf16, 0, n, rank, world, pads,
                                          epoch[0], 0, stream))

    def in_switch(n):
        epoch[0] += 1
        abi.check(lib.b200_multimem_allreduce(multicast, f16, multicast, bf16, 0, n, rank, world,
                                              pads, epoch[0], 0, stream))

    out = {"protocol": "event pairs around single launches, mean of 30, max over ranks",
           "buffer": "[4096, 4096] float16 partials -> bfloat16 result, in place"}
    kernels = [("peer_loads", peer_loads)] + ([("in_switch", in_switch)] if multicast else [])
    for name, fn in kernels:
        for label, n in (("32MiB_us", count), ("8MiB_us", count // 4)):
            buf.normal_()
            torch.cuda.synchronize()
            dist.barrier()
            _, launch_ms, _ = time_event_pairs(torch, dist, lambda i: fn(n), launches, 5)
            abi.check(lib.b200_last_device_status(stream))
            out.setdefault(name, {})[label] = round(dist.max(launch_ms) * 1e3, 2)
    x = torch.randn((MLP_M, MLP_HIDDEN), device="cuda").to(torch.bfloat16)
    _, launch_ms, _ = time_event_pairs(torch, dist, lambda i: tdist.all_reduce(x), launches, 5)
    out["nccl_bf16"] = {"32MiB_us": round(dist.max(launch_ms) * 1e3, 2)}
    out["gpu_launches"] = len(kernels) * 2 * (launches + 5)
    return out


# --------------------------------------------------------------------------- siblings
def bench_siblings(torch, ops, peaks):
    """Rates of the sibling kernels at sizes well above the L2: four rotating buffer sets,
    20 launches per CUDA graph, two replays timed with CUDA events on the capturing stream;
    bytes are the algorithmic ones (every operand read once, the result written once)."""
    import ctypes
    from compiler_b200 import graph
    from compiler_b200.runtime import abi
    lib = abi.lib()
    rows, cols, sets_default, launches = 16384, 4096, 4, 20
    stream = graph.Stream()
    S = stream.handle
    records = {}

    def timed(launch, sets):
        for i in range(3):
            launch(i % sets)
        stream.synchronize()
        with graph.capture(stream) as g:
            for i in range(launches):
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
        return ms.value / (2 * launches)

    def report(name, launch, nbytes=None, flop=None, sets=sets_default):
        ms = timed(launch, sets)
        record = {"us_per_launch": round(ms * 1e3, 2)}
        if nbytes:
            rate = nbytes / ms / 1e6
            record.update({"GBps": round(rate, 1), "frac": round(rate / peaks["hbm_gbs"], 3)})
        if flop:
            rate = flop / ms / 1e9
            record.update({"TFLOPs": round(rate, 1), "frac": round(rate / peaks["bf16_tflops"], 3)})
        records[name] = record

    def rnd(shape, dtype, scale=1.0):
        return (torch.randn(shape, device="cuda") * scale).to(dtype)

    torch.manual_seed(0)
    for dtype, tag, es in ((torch.bfloat16, "bf16", 2), (torch.float32, "f32", 4)):
        n = rows * cols
        xs = [rnd((rows, cols), dtype) for _ in range(sets_default)]
        ys = [rnd((rows, cols), dtype) for _ in range(sets_default)]
        outs = [torch.empty((rows, cols), device="cuda", dtype=dtype) for _ in range(sets_default)]
        flat = lambda t: t.view(-1)  # noqa: E731
        report(f"swiglu_{tag}", lambda i: ops.swiglu(xs[i], ys[i], outs[i], stream=S), 3 * n * es)
        report(f"gelu_erf_{tag}", lambda i: ops.elementwise(
            abi.EW_GELU_ERF, flat(xs[i]), flat(outs[i]), stream=S), 2 * n * es)
        report(f"add_gelu_erf_{tag}", lambda i: ops.elementwise(
            abi.EW_ADD_GELU_ERF, flat(xs[i]), flat(outs[i]), b=flat(ys[i]), p0=1.5, stream=S),
            3 * n * es)
        report(f"geglu_tanh_{tag}", lambda i: ops.elementwise(
            abi.EW_GEGLU_TANH, flat(xs[i]), flat(outs[i]), b=flat(ys[i]), stream=S), 3 * n * es)
        bias = rnd((cols,), dtype)
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
        w = rnd((cols,), dtype)
        report(f"rmsnorm_zero_centred_gamma_{tag}", lambda i: ops.rmsnorm(
            xs[i], w, outs[i], None, eps=1e-6, gamma_offset=1.0, stream=S), 2 * n * es)
        quarter = [rnd((rows, cols // 4), dtype) for _ in range(sets_default)]
        report(f"repeat4_log_softmax_{tag}", lambda i: ops.repeat_log_softmax(
            quarter[i], outs[i], 4, stream=S), (n // 4 + n) * es)
        del xs, ys, outs, quarter
        torch.cuda.empty_cache()

    k, n = 16384, 8192
    q = [torch.randint(-128, 127, (k, n), device="cuda", dtype=torch.int8)
         for _ in range(sets_default)]
    scale = rnd((n,), torch.bfloat16)
    deq = [torch.empty((k, n), device="cuda", dtype=torch.bfloat16) for _ in range(sets_default)]
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
    wt = rnd((n, k), torch.bfloat16, 0.02)
    report("linear_weight_rows_of_k_bf16_8192x8192x4096", lambda i: ops.linear(
        xs[i], wt, outs[i], stream=S), flop=2 * m * n * k, sets=3)
    del xs, outs, w, w2, wt, scratch_w
    torch.cuda.empty_cache()
    big = 65536
    x2 = [rnd((big, 4096), torch.bfloat16) for _ in range(3)]
    wl = rnd((64, 4096), torch.bfloat16, 0.02)
    y2 = [torch.empty((big, 64), device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    report("linear_log_softmax_bf16_65536x64x4096", lambda i: ops.linear_log_softmax(
        x2[i], wl, y2[i], stream=S), (big * 4096 + big * 64 + 64 * 4096) * 2, sets=3)
    stream.synchronize()
    ops.device_status(S)
    stream.close()
    return {"protocol": "graphs of 20 launches on rotating buffer sets, two replays timed; "
                        "fractions of the measured copy rate / cuBLAS bf16 burst rate",
            "kernels": records, "gpu_launches": len(records) * (3 + 3 * launches)}


# --------------------------------------------------------------------------- CPU legs
def headline_config():
    return {"workload": "masked_softmax_fp16_16384x4000",
            "mask": "col > row % 4000 -> -inf", "io_dtype": "f16",
            "rows_per_gpu": ROWS, "sharding": "rows, no collective",
            "l2": "4 rotating buffer sets (1.05 GB) between reuses, L2 is 126 MB",
            "launching": f"native arm: one step = one replay of a CUDA graph of "
                         f"{LAUNCHES_PER_STEP} launches; reference arm: one step = one pass"}


class CpuReference:
    """The reference's CPU implementation of the headline workload: the numpy float64 oracle
    over all 16384 x 4000 elements per pass.  Rows are independent, so the rows are cut into
    blocks that a pool of threads works through (numpy releases the GIL inside its loops), the
    way the reference's own split_ref (ops/harness/opslib/case.py:591-632) runs row-independent
    oracles; the thread count is reported."""
    BLOCK = 256

    def __init__(self):
        rng = np.random.default_rng(30)
        self.x = (rng.standard_normal((ROWS, COLS), dtype=np.float32) * 2).astype(np.float16)
        self.y = np.empty_like(self.x)
        self.threads = max(1, len(os.sched_getaffinity(0)))
        self.pool = ThreadPoolExecutor(max_workers=self.threads)

    def _block(self, lo):
        from oracle import oracle
        hi = min(lo + self.BLOCK, ROWS)
        self.y[lo:hi] = oracle.masked_softmax_ref(self.x[lo:hi], lo).astype(np.float16)

    def one_pass(self) -> float:
        t0 = time.perf_counter()
        list(self.pool.map(self._block, range(0, ROWS, self.BLOCK)))
        return time.perf_counter() - t0

    def measure(self, steps, warmup):
        for _ in range(max(1, warmup)):
            self.one_pass()
        times = [self.one_pass() for _ in range(steps)]
        return float(np.mean(times)), times

    def describe(self, steps, seconds):
        return (f"numpy float64 oracle over all {ROWS} x {COLS} elements per pass, rows in "
                f"blocks of {self.BLOCK} on {self.threads} threads, mean of {steps} passes "
                f"({seconds:.3f} s each)")


def cpu_baseline():
    ref = CpuReference()
    steps = 5
    seconds, _ = ref.measure(steps, 1)
    return {"value": round(SOFTMAX_BYTES / seconds / 1e9, 4), "unit": "GB/s",
            "cores": ref.threads, "kind": "port", "sample": ref.describe(steps, seconds),
            "host_cores_available": len(os.sched_getaffinity(0))}


def reference_arm(args):
    """Reference arm: the reference's CPU implementation (numpy float64 ``ref``, restated in
    oracle/oracle.py) of the headline workload on the host cores, the whole workload per
    step, with the protocol of ``cpu_baseline``."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ref = CpuReference()
    seconds, _ = ref.measure(args.steps, max(args.warmup, 1))
    value = round(SOFTMAX_BYTES / seconds / 1e9, 4)
    line = {
        "impl": "reference", "metric": "masked_softmax_fp16_hbm_throughput", "value": value,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(seconds * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": headline_config(),
        "step": "one pass of the numpy oracle over the whole workload",
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": ref.threads, "kind": "port",
                         "sample": ref.describe(args.steps, seconds)},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- main
def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20,
                        help=f"timed steps of the headline; one step = {LAUNCHES_PER_STEP} launches")
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="native", choices=["native", "reference"])
    parser.add_argument("--ops", default="all",
                        help="comma list of extra operators: softmax_unmasked,rmsnorm,gemm,"
                             "gemm_ragged,attention,attention_decode,siblings,tp_mlp,allreduce,none,all")
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
    steps = max(1, args.steps)
    uuid = getattr(torch.cuda.get_device_properties(dist.local_rank), "uuid", None)
    sampler = ClockSampler(dist.local_rank, f"GPU-{uuid}" if uuid is not None else None)
    if dist.rank == 0:
        sampler.start()

    head = bench_softmax(torch, ops, dist, steps, warmup, peaks, source)
    strong = None
    if dist.enabled:
        strong = bench_softmax_strong(torch, ops, dist, min(steps, 20), 3, peaks, source)
    e2e = bench_softmax_e2e(dist, min(steps, 20), 3)

    wanted = args.ops.split(",")
    op_steps = max(3, min(steps, 20))   # steps of LAUNCHES_PER_STEP launches for the HBM-bound ops
    launches = 20                       # launches of the tensor-core ops' burst region
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
        extras["softmax_unmasked"] = bench_softmax_unmasked(torch, ops, dist, op_steps, 3, peaks,
                                                            source)
    if want("rmsnorm"):
        extras["rmsnorm"] = bench_rmsnorm(torch, ops, dist, op_steps, 3, peaks, source)
        if dist.enabled:
            extras["rmsnorm"]["strong"] = bench_rmsnorm(torch, ops, dist, op_steps, 3, peaks,
                                                        source, strong=True)
    if want("gemm"):
        extras["gemm"] = bench_gemm(torch, ops, dist, launches, peaks, source,
                                    (8192, 8192, 8192), "gemm_8192")
        if dist.enabled:
            extras["gemm"]["strong"] = bench_gemm(torch, ops, dist, launches, peaks, source,
                                                  (8192, 8192, 8192), "gemm_8192", strong=True)
    if want("gemm_ragged"):
        extras["gemm_ragged"] = bench_gemm(torch, ops, dist, launches, peaks, source,
                                           (4097, 11008, 4096), "gemm_ragged")
        if dist.enabled:
            extras["gemm_ragged"]["strong"] = bench_gemm(
                torch, ops, dist, launches, peaks, source, (4097, 11008, 4096), "gemm_ragged",
                strong=True)
    if want("attention"):
        extras["attention"] = bench_attention(torch, ops, dist, 10, peaks, source)
        if dist.enabled:
            extras["attention"]["strong"] = bench_attention(torch, ops, dist, 10, peaks, source,
                                                            strong=True)
    if want("attention_decode"):
        extras["attention_decode"] = bench_attention_decode(torch, ops, dist, op_steps, 3, peaks,
                                                            source)
    if want("tp_mlp"):
        if not dist.enabled:
            extras["tp_mlp"] = bench_tp_mlp(torch, ops, dist, launches, peaks, source, "nccl")
        else:
            for key, collective, options in (
                    ("tp_mlp", "nccl", {}), ("tp_mlp_peer", "peer", {}),
                    ("tp_mlp_nvls", "nvls", {"overlap_blocks": 0}),
                    ("tp_mlp_pull", "pull", {"overlap_blocks": 0}),
                    ("tp_mlp_pull_row_blocks", "pull", {"row_splits": 2, "comm_ctas": 74}),
                    ("tp_mlp_pull_beside_gemm", "pull", {"overlap_blocks": 4}),
                    ("tp_mlp_nvls_beside_gemm", "nvls", {"overlap_blocks": 4}),
                    ("tp_mlp_nvls_f32", "nvls", {"partial_dtype": torch.float32,
                                                 "overlap_blocks": 0})):
                if collective == "peer" and MLP_M % (128 * dist.world):
                    continue
                time.sleep(0.5)
                try:
                    extras[key] = bench_tp_mlp(torch, ops, dist, launches, peaks, source,
                                               collective, **options)
                except Exception as exc:  # noqa: BLE001 - symmetric memory / NVLS may be unavailable
                    extras[key] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
            valid = {k: v for k, v in extras.items() if k.startswith("tp_mlp") and
                     v.get("value") is not None and v.get("parity", {}).get("ok")}
            if valid:
                best = min(valid, key=lambda k: valid[k]["ms_per_step"])
                extras["tp_mlp_fastest"] = {
                    "variant": best, "ms_per_step": valid[best]["ms_per_step"],
                    "frac": valid[best]["frac"], "value": valid[best]["value"],
                    "unit": valid[best]["unit"],
                    "note": "the fastest of the tp_mlp* entries above whose result matched "
                            "the oracle on every rank; tp_mlp itself is the NCCL baseline"}
    if want("allreduce") and dist.enabled:
        try:
            extras["allreduce"] = bench_allreduce(torch, dist)
        except Exception as exc:  # noqa: BLE001 - symmetric memory may be unavailable
            extras["allreduce"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    if want("siblings") and not dist.enabled:
        extras["siblings"] = bench_siblings(torch, ops, peaks)

    baseline = cpu_baseline() if (dist.rank == 0 and dist.world == 1) else None

    def strip(entry):
        entry.pop("window", None)
        for sub in entry.values():
            if isinstance(sub, dict):
                sub.pop("window", None)

    if dist.rank != 0:
        for extra in extras.values():
            strip(extra)
    if dist.rank == 0:
        sampler.stop()
        clocks = sampler.summary(*head["window"])
        for extra in extras.values():  # each operator's own clock record
            if "window" in extra:
                extra["clocks"] = sampler.summary(*extra.pop("window"),
                                                  label="this operator's timed region")
            sustained = extra.get("sustained")
            if isinstance(sustained, dict) and "window" in sustained:
                sustained["clocks"] = sampler.summary(*sustained.pop("window"),
                                                      label="the sustained region")
            strip(extra)
        launch_ms = head["launch_ms"]
        value = SOFTMAX_BYTES * dist.world / (launch_ms * 1e-3) / 1e9
        roof = {k: head[k] for k in ("bound", "achieved", "peak", "unit", "frac", "peak_source",
                                     "traffic", "algorithmic_per_launch", "launch_ms",
                                     "launch_ms_event_pairs", "frac_event_pairs",
                                     "necessary_bytes_per_launch", "achieved_dram", "frac_dram",
                                     "note")}
        config = headline_config()
        line = {
            "metric": "masked_softmax_fp16_hbm_throughput", "value": round(value, 2),
            "unit": "GB/s", "n_gpus": dist.world, "steps": steps, "warmup": warmup,
            "ms_per_step": round(head["ms_per_step"], 4), "launches_per_step": LAUNCHES_PER_STEP,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config, "roofline": roof, "parity": head["parity"],
            "e2e": e2e, "gpu_launches": head["gpu_launches"], "clocks": clocks, "ops": extras,
        }
        if strong is not None:
            line["strong"] = strong
        if baseline is not None:
            line["cpu_baseline"] = baseline
        print(json.dumps(line))
    dist.finish()


if __name__ == "__main__":
    main()
