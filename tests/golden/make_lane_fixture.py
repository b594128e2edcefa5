"""Pins ``compiler_b200/lane_workload.json`` against the reference's benchmark lane.

Run in a container that has the reference tree (imported read-only):

    python tests/golden/make_lane_fixture.py /path/to/reference

For every entry of the lane workload it records, in ``tests/golden/lane_fixture.json``,

* the shape the reference's own ``harness/benchmark/size.py: resolve_shape`` gives at three
  last-level-cache sizes (``tests/test_lane.py`` checks ``compiler_b200.lane.resolve_shape``
  against them), and
* the kernel the operator file's ``make_case`` hands out at a small resolved shape: function
  name, parameter list and autotuned constexprs (the test checks that the registry has a
  native operator for exactly that signature), with the case's outputs and comparison policy.
"""
from __future__ import annotations

import importlib.util
import inspect
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
LLC_SIZES = (1 << 20, 50 << 20, 126 << 20)


def main(reference_root: str) -> None:
    root = Path(reference_root).resolve()
    ops_root = root / "ops"
    sys.path.insert(0, str(ops_root / "harness"))
    from opslib import runner  # noqa: E402  (the reference's loader)
    spec = importlib.util.spec_from_file_location(
        "reference_size", ops_root / "harness" / "benchmark" / "size.py")
    size = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(size)

    workload = json.loads((REPO / "compiler_b200" / "lane_workload.json").read_text())
    out = {}
    for entry in workload["entries"]:
        dtype = entry.get("dtype", workload["dtype"])
        shapes = {str(llc): size.resolve_shape(entry, llc, 8, workload["dtype"])
                  for llc in LLC_SIZES}
        module = runner.load_operator(ops_root / entry["operator"])
        small = size.resolve_shape(entry, 1 << 16, 8, workload["dtype"])
        if entry["scale"]["kind"] in ("matmul", "fixed", "attention"):
            small = list(module.SHAPES[0])  # explicit shapes are too large for the host oracle
        case = module.make_case(shape=tuple(small), dtype=dtype, seed=7)
        kernel = case["kernel"]
        target = kernel
        for _ in range(8):  # Autotuner -> JITFunction -> python function
            if inspect.isfunction(target) or not hasattr(target, "fn"):
                break
            target = target.fn
        configs = getattr(kernel, "configs", None)
        out[entry["id"]] = {
            "dtype": dtype,
            "declared_dtypes": list(module.DTYPES),
            "shapes": shapes,
            "checked_shape": list(small),
            "kernel_name": target.__name__,
            "parameters": list(inspect.signature(target).parameters),
            "autotuned": sorted(configs[0].kwargs.keys()) if configs else [],
            "outputs": list(case["outputs"]),
            "comparison": {k: dict(v) for k, v in case["comparison"].items()},
        }
        print(entry["id"], shapes[str(LLC_SIZES[-1])], target.__name__)
    (HERE / "lane_fixture.json").write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
