"""Generates ``tests/golden/*.npz`` from the reference's own operator modules.

Run in a container that has the reference tree (it is imported read-only):

    python tests/golden/make_golden.py /path/to/reference [operator file ...]

(operator files as listed in ``OPERATORS``; with none, every fixture is rewritten.)

For every hot-path operator file it calls the file's own ``make_case(shape,
dtype, seed)`` for each declared shape (plus one audited mid-size shape) and each
declared dtype, and stores the case's input arrays, scalar arguments, metas and
the ``expected`` outputs computed by the file's own numpy ``ref``, together with
the comparison policy the reference attaches.  The tests then check the oracle
(``oracle/oracle.py``) and the CUDA kernels against these files; the reference
tree itself is not needed at test time.
"""
from __future__ import annotations

import inspect
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

# operator file -> extra (mid-size) shapes beyond the file's SHAPES; the mid-size
# shapes are the "source_validated_shape" entries of ops/suite/perf/workload.json
OPERATORS = {
    "perf/fast_rms_layernorm.py": [(64, 1024)],
    "perf/softmax.py": [(64, 1024)],
    "perf/matmul.py": [(256, 256, 256)],
    "perf/triton_linear_activation.py": [(256, 256, 256)],
    "perf/matmul_triton2.py": [],
    "perf/attn_fwd_causal.py": [(1, 8, 256, 64)],
    "perf/context_attn_fwd.py": [],
    "perf/swiglu_fwd.py": [(64, 1024)],
    "dev/softmax_kernel_inner.py": [],
    "dev/softmax_multi_block_forward_kernel.py": [],
    "dev/hidden__rms_norm_loop_kernel.py": [],
    # sibling kernels of the five families
    "perf/softmax_mul.py": [],
    "perf/softmax_log.py": [],
    "perf/fused_repeat_interleave_log_softmax.py": [],
    "perf/gelu.py": [],
    "perf/add_gelu.py": [],
    "perf/geglu_tanh_triton.py": [],
    "perf/swiglu_triton.py": [],
    "perf/matmul_triton_autotune.py": [],
    "perf/attention_forward_triton.py": [],
    "perf/attention_kernel.py": [],
    "dev/epilogue_kernel.py": [],
    "dev/rmsnorm_fwd_loop_kernel.py": [],
    # decode-side attention
    "perf/flash_decode.py": [(1, 8, 256, 64)],
    "dev/gqa.py": [],
    "dev/flash_varlen_fwd_kernel.py": [],
    "dev/parallel_attn_fwd_kernel.py": [],
    # GEMM with a reduction epilogue
    "perf/log_softmax_linear.py": [(64, 1024)],
    # norm folded into a GEMM
    "dev/rms_matmul_rbe.py": [],
    "perf/dequantize_matmul.py": [],
    "dev/fused_gemm_gn_min_kernel.py": [],
}
MID_DTYPES = ("bfloat16",)  # mid-size shapes are stored for one dtype to keep fixtures small


def main(reference_root: str) -> None:
    root = Path(reference_root).resolve()
    sys.path.insert(0, str(root / "ops" / "harness"))
    from opslib import runner  # noqa: E402  (the reference's loader)

    only = set(sys.argv[2:])  # optional: operator files to (re)generate, others stay as they are
    index = json.loads((HERE / "index.json").read_text()) if only else {}
    for rel, extra in OPERATORS.items():
        if only and rel not in only:
            continue
        module = runner.load_operator(root / "ops" / "suite" / rel)
        stem = Path(rel).stem
        cases = [(tuple(s), d) for s in module.SHAPES for d in module.DTYPES]
        cases += [(tuple(s), d) for s in extra for d in MID_DTYPES if d in module.DTYPES]
        for shape, dtype in cases:
            case = module.make_case(shape=shape, dtype=dtype)
            arrays, scalars = {}, {}
            for name, value in {**case.get("allocations", {}), **case["args"]}.items():
                if isinstance(value, np.ndarray):
                    arrays["arg__" + name] = value
                else:
                    scalars[name] = value.item() if isinstance(value, np.generic) else value
            for name, value in case["expected"].items():
                arrays["expected__" + name] = np.asarray(value)
            kernel = case["kernel"]
            target = kernel
            for _ in range(8):  # Autotuner -> JITFunction -> python function
                if inspect.isfunction(target) or not hasattr(target, "fn"):
                    break
                target = target.fn
            meta = {
                "operator": rel,
                "kernel_name": getattr(target, "__name__", str(target)),
                "parameters": list(inspect.signature(target).parameters),
                "autotuned": sorted(((getattr(kernel, "configs", None) or [None])[0].kwargs
                                     if getattr(kernel, "configs", None) else {}).keys()),
                "shape": list(shape),
                "dtype": dtype,
                "scalars": scalars,
                "meta": {k: (v.item() if isinstance(v, np.generic) else v)
                         for k, v in case.get("meta", {}).items()},
                "launch_meta": case.get("launch_meta", {}),
                "outputs": list(case["outputs"]),
                "pointer_dtypes": {k: str(v).rsplit(".", 1)[-1]
                                   for k, v in (case.get("pointer_dtypes") or {}).items()},
                "comparison": {k: {kk: vv for kk, vv in v.items()}
                               for k, v in case["comparison"].items()},
                "grid": (list(case["grid"]) if not callable(case["grid"]) else "callable"),
            }
            tag = f"{stem}__{'x'.join(map(str, shape))}__{dtype}"
            np.savez_compressed(HERE / f"{tag}.npz", __meta__=np.array(json.dumps(meta)), **arrays)
            index[tag] = {"operator": rel, "shape": list(shape), "dtype": dtype}
            print("wrote", tag)
    (HERE / "index.json").write_text(json.dumps(index, indent=1, sort_keys=True) + "\n")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
