"""The benchmark lane of the operator corpus, for this backend.

The corpus times its ``suite/perf`` operators at steady-state shapes with
``harness/benchmark/run.py`` and pairs the records of a compiler device with those of
stock Triton in ``report.py``.  That runner needs, per operator, a workload entry with a
*size rule* (``harness/benchmark/size.py:41-99``); the workload file shipped with the corpus
is the correctness workload and carries none.  This module supplies

* ``lane_workload.json`` (beside this file): entries for the operator files this backend has
  native operators for, in the fields ``size.py`` and ``run.py`` read
  (``id, operator, class, family, pattern, dtype, declared_shape, scale, bytes_model,
  ref_split``);
* :func:`resolve_shape` -- the size rules, restated, so shapes can be listed and checked
  without the corpus;
* :func:`measure` / :func:`summarize` / :func:`run_entry` -- the runner's protocol for one
  staged case (``run.py:143-269``): outputs zeroed before the first launch, first launch
  timed separately as ``compile_s``, verification before timing, adaptive sampling on the
  device timer, median as the headline, the same record keys -- so a record written here
  pairs with a ``BENCH_TRITON.json`` record in ``report.py``;
* a CLI that builds the cases with the corpus's own loader when the corpus is on disk::

      python -m compiler_b200.lane --corpus /path/to/ops --out-dir evidence [--only softmax]

  (equivalent to ``harness/benchmark/run.py --device compiler_b200.device:make_device
  --workload .../lane_workload.json``; kept here because it has no Triton import.)

Nothing here computes an operator: cases arrive with their ``expected`` arrays from the
corpus (or from a test), the device launches, and verification compares.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import statistics
import sys
import time
from pathlib import Path

import numpy as np

from compiler_b200 import harness

WORKLOAD = Path(__file__).resolve().parent / "lane_workload.json"
DEFAULT_MULTIPLE = 8          # bandwidth classes: working set = 8 x last-level cache
MIN_SAMPLES_FLOOR = 10        # never summarise fewer launches than this (run.py:140)

_ITEMSIZE = {"float64": 8, "int64": 8, "float32": 4, "int32": 4, "float16": 2, "bfloat16": 2,
             "int16": 2, "int8": 1, "uint8": 1}


def itemsize(dtype) -> int:
    return _ITEMSIZE.get(str(dtype), 4)


def resolve_shape(entry: dict, llc_bytes: int, multiple: int = DEFAULT_MULTIPLE,
                  dtype: str = "float32") -> list[int]:
    """Steady-state shape of one workload entry (``benchmark/size.py:41-99``).

    Bandwidth-bound entries are sized so that their working set is ``multiple`` times the
    device's last-level cache; compute-bound entries name their shape."""
    rule, model = entry["scale"], entry.get("bytes_model", {})
    declared = [int(v) for v in entry["declared_shape"]]
    width = itemsize(entry.get("dtype", dtype))
    budget = int(llc_bytes) * int(multiple)
    kind = rule["kind"]
    if kind == "fixed":
        return [int(v) for v in rule["shape"]]
    if kind == "matmul":
        return [int(rule["size"])] * 3
    if kind == "batched_matmul":
        return [int(rule["batch"])] + [int(rule["size"])] * 3
    if kind == "linear":
        k = int(rule["k"])
        return [max(1, (budget // (width * 3)) // max(1, k)), k]
    if kind == "attention":
        return [1, int(rule["heads"]), int(rule["seq"]), int(rule["dim"])]
    if kind == "reduce":
        cols = int(rule["cols"])
        full = max(1, int(model.get("full", 1)))
        return [max(1, budget // (width * full * cols)), cols]
    if kind != "first_dim":
        raise ValueError(f"{entry.get('id')}: unknown scale kind {kind!r}")
    elements = budget // (width * max(1, int(model.get("full", 2))))
    if rule.get("quadratic"):
        side = max(1, min(int(rule.get("max", 1 << 15)), math.isqrt(elements)))
        return [side] + declared[1:]
    trailing = math.prod(declared[1:]) if len(declared) > 1 else 1
    first = max(1, elements // max(1, trailing))
    step = int(rule.get("multiple_of", 1))
    return [max(step, first // step * step)] + declared[1:]


def load_workload(path=None) -> dict:
    return json.loads(Path(path or WORKLOAD).read_text())


# --------------------------------------------------------------------------- protocol
def enough(times, *, samples=None, min_samples=50, min_time_s=0.2, max_samples=1000) -> bool:
    """Stop rule of the adaptive sampler (``run.py:143-151``): a fixed count when asked for,
    else ``min_samples`` launches or ``min_time_s`` of accumulated kernel time, whichever
    comes first, never below the floor and never above ``max_samples``."""
    count = len(times)
    if samples:
        return count >= samples
    if count >= max_samples:
        return True
    if count < MIN_SAMPLES_FLOOR:
        return False
    return count >= max(min_samples, MIN_SAMPLES_FLOOR) or sum(times) >= min_time_s


def _percentile(values, fraction):
    ordered = sorted(values)
    return ordered[min(len(ordered) - 1, round(fraction * (len(ordered) - 1)))]


def summarize(times, stat="median") -> dict:
    """The timing fields of a record (``run.py:179-195``)."""
    mean = statistics.fmean(times)
    spread = statistics.pstdev(times) if len(times) > 1 else 0.0
    cov = spread / mean if mean else 0.0
    return {"kernel_s": statistics.median(times) if stat == "median" else mean, "stat": stat,
            "median_s": statistics.median(times), "mean_s": mean,
            "p10_s": _percentile(times, 0.10), "p90_s": _percentile(times, 0.90),
            "stdev_s": spread, "cov": cov, "steady": cov < 0.05, "n_samples": len(times),
            "times_s": list(times)}


def measure(staged, device, *, warmups=3, timer=None, **stop) -> list[float]:
    """Kernel times of repeated launches of one staged case (``run.py:154-171``): device
    events when the device has a timer, else host clock between synchronisations."""
    for _ in range(warmups):
        staged.launch()
    device.synchronize()
    times: list[float] = []
    while not enough(times, **stop):
        if timer is not None:
            with timer:
                staged.launch()
            times.append(timer.seconds)
        else:
            device.synchronize()
            start = time.perf_counter()
            staged.launch()
            device.synchronize()
            times.append(time.perf_counter() - start)
    return times


# The function that uploads a case and binds its arguments: this package's stand-in, or the
# corpus's own ``opslib.device.stage_case`` once ``--corpus`` has put it on the path.
_stage_case = harness.stage_case


def stage_zeroed(case: dict, device):
    """Stage a case with every pure output buffer zeroed, so that a kernel that did not
    write shows up as a mismatch instead of passing on stale data (``run.py:105-113``)."""
    if "inputs" not in case:  # no declaration of what is read: leave every buffer as given
        return _stage_case(case, device)
    outputs, inputs = set(case.get("outputs") or ()), set(case.get("inputs") or ())
    scrubbed = dict(case)
    for key in ("args", "allocations"):
        if key in case:
            scrubbed[key] = {
                name: (np.zeros(value.shape, value.dtype)
                       if isinstance(value, np.ndarray) and name in outputs and name not in inputs
                       else value)
                for name, value in case[key].items()}
    return _stage_case(scrubbed, device)


def verify(staged, case: dict, device) -> float:
    """Compare every output with ``case["expected"]`` under the case's own policy; on the
    device when the buffer is float32 (``Device.compare``), else on the host after a
    download, as ``opslib/compare.py:253-321`` does.  Returns the largest absolute error;
    raises ``AssertionError`` on a mismatch."""
    worst = 0.0
    for name in case["outputs"]:
        policy = case["comparison"][name]
        rtol, atol = float(policy["rtol"]), float(policy["atol"])
        equal_nan = bool(policy.get("equal_nan", False))
        expected = np.asarray(case["expected"][name])
        verdict = None
        if getattr(device, "compare", None) is not None and expected.dtype == np.float32:
            verdict = device.compare(staged.buffer(name), expected,
                                     {"rtol": rtol, "atol": atol, "equal_nan": equal_nan})
        if verdict is None:
            got = np.asarray(device.download(staged.buffer(name)), dtype=np.float64)
            want = expected.astype(np.float64).reshape(got.shape)
            close = np.isclose(got, want, rtol=rtol, atol=atol, equal_nan=equal_nan)
            finite = np.isfinite(got) & np.isfinite(want)
            error = float(np.max(np.abs(got - want), where=finite, initial=0.0))
            verdict = (bool(close.all()), error)
        ok, error = verdict
        if not ok:
            raise AssertionError(f"{name}: comparison failed (max_abs_error={error:.3e})")
        worst = max(worst, float(error))
    return worst


def run_entry(record: dict, case: dict, device, *, do_verify=True, verify_only=False,
              stat="median", warmups=3, **stop) -> dict:
    """One workload entry on ``device`` (``run.py:219-269``).  ``record`` carries the
    provenance fields (id, operator, class, shape ...) and comes back with ``status``
    (PASS / LAUNCH_FAIL / MISMATCH), ``compile_s``, ``max_abs_error``, ``verified`` and the
    timing summary."""
    record = dict(record)
    staged = None
    phase = "launch"
    try:
        staged = stage_zeroed(case, device)
        start = time.perf_counter()
        staged.launch()
        device.synchronize()
        record["compile_s"] = time.perf_counter() - start
        if do_verify:
            phase = "verify"
            record["max_abs_error"] = verify(staged, case, device)
        record["verified"] = bool(do_verify)
        if not verify_only:
            phase = "measure"
            timer = device.timer() if getattr(device, "timer", None) is not None else None
            record["timer"] = "device" if timer is not None else "host"
            record.update(summarize(measure(staged, device, warmups=warmups, timer=timer,
                                            **stop), stat))
        record["status"] = "PASS"
    except Exception as exc:  # noqa: BLE001 - the record carries the failure
        message = (str(exc).splitlines() or [type(exc).__name__])[0][:200]
        record.update({"status": "MISMATCH" if phase == "verify" else "LAUNCH_FAIL",
                       "error": message})
    finally:
        release = getattr(device, "release", None)
        if staged is not None and release is not None:
            release({n: b for n, b in staged._buffers.items()})
    return record


# --------------------------------------------------------------------------- CLI
def _corpus_case(corpus: Path, entry: dict, shape, dtype, seed):
    """Build the case with the corpus's own loader and oracle (``run.py:209-221``)."""
    harness_dir = str(corpus / "harness")
    if harness_dir not in sys.path:
        sys.path.insert(0, harness_dir)
    from opslib.runner import load_operator  # the corpus's module, not part of this package
    module = load_operator(corpus / entry["operator"])
    return module.make_case(shape=tuple(shape), dtype=dtype, seed=seed)


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--corpus", help="root of the operator corpus (the directory that "
                                         "holds suite/ and harness/); without it, --list only")
    parser.add_argument("--workload", default=str(WORKLOAD))
    parser.add_argument("--list", action="store_true", help="print the resolved shapes and exit")
    parser.add_argument("--llc-bytes", type=int, default=None)
    parser.add_argument("--multiple", type=int, default=DEFAULT_MULTIPLE)
    parser.add_argument("--group", default=None, help="memory | reduction | compute")
    parser.add_argument("--only", default=None, help="comma list of entry ids")
    parser.add_argument("--seed", type=int, default=20261008)
    parser.add_argument("--no-verify", action="store_true")
    parser.add_argument("--verify-only", action="store_true")
    parser.add_argument("--samples", type=int, default=None)
    parser.add_argument("--min-samples", type=int, default=50)
    parser.add_argument("--min-time-s", type=float, default=0.2)
    parser.add_argument("--max-samples", type=int, default=1000)
    parser.add_argument("--stat", choices=("median", "mean"), default="median")
    parser.add_argument("--device-id", type=int, default=0)
    parser.add_argument("--out-dir", default="lane-results")
    args = parser.parse_args(argv)

    workload_path = Path(args.workload)
    workload = json.loads(workload_path.read_text())
    entries = [e for e in workload["entries"]
               if (not args.group or e["class"] == args.group)
               and (args.only is None or e["id"] in args.only.split(","))]
    if args.list or not args.corpus:
        llc = args.llc_bytes or (128 << 20)
        for entry in entries:
            shape = resolve_shape(entry, llc, args.multiple, workload["dtype"])
            print(f"{entry['class']:9s} {entry['id']:40s} "
                  f"{entry.get('dtype', workload['dtype']):9s} {shape}")
        return 0

    from compiler_b200.device import B200Device
    device = B200Device(args.device_id)
    props = device.properties()
    llc = args.llc_bytes or props["llc_bytes"]
    common = {"workload_sha256": hashlib.sha256(workload_path.read_bytes()).hexdigest(),
              "device_properties": props, "numpy": np.__version__, "llc_bytes": llc,
              "device": "compiler_b200.device:make_device"}
    out_dir = Path(args.out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    corpus = Path(args.corpus)
    harness_dir = str(corpus / "harness")
    if harness_dir not in sys.path:
        sys.path.insert(0, harness_dir)
    global _stage_case
    from opslib.device import stage_case as _stage_case  # the corpus's own staging and launch
    rows = []
    for entry in entries:
        dtype = entry.get("dtype", workload["dtype"])
        shape = resolve_shape(entry, llc, args.multiple, workload["dtype"])
        record = {"id": entry["id"], "operator": entry["operator"], "class": entry["class"],
                  "family": entry["family"], "dtype": dtype, "shape": shape,
                  "size_class": f"llc_x{args.multiple}", "warmups": 3,
                  "operator_sha256": hashlib.sha256(
                      (corpus / entry["operator"]).read_bytes()).hexdigest(), **common}
        try:
            case = _corpus_case(corpus, entry, shape, dtype, args.seed)
        except Exception as exc:  # noqa: BLE001
            record.update({"status": "CASE_FAIL", "error": f"{type(exc).__name__}: {exc}"[:200]})
        else:
            record = run_entry(record, case, device, do_verify=not args.no_verify,
                               verify_only=args.verify_only, stat=args.stat,
                               samples=args.samples, min_samples=args.min_samples,
                               min_time_s=args.min_time_s, max_samples=args.max_samples)
        rows.append(record)
        print(f"{record['status']:11s} {entry['class']:9s} {entry['id']:36s} "
              f"kernel={(record.get('kernel_s') or 0) * 1e3:10.4f}ms "
              f"n={record.get('n_samples', 0):4d}", flush=True)
        (out_dir / "BENCH_REPORT.json").write_text(json.dumps(
            {"schema": "tritonbench-bench-run/2", "metric": "kernel_time_s",
             "device": common["device"], "timer": "device", "llc_bytes": llc,
             "multiple": args.multiple, "seed": args.seed, "entries": rows}, indent=2) + "\n")
    passed = sum(1 for row in rows if row["status"] == "PASS")
    print(f"{passed}/{len(rows)} PASS")
    return 0 if rows and passed == len(rows) else 1


if __name__ == "__main__":
    raise SystemExit(main())
