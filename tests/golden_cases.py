"""Rebuilds harness case dicts from the committed golden fixtures.

Each ``tests/golden/<tag>.npz`` was written by ``tests/golden/make_golden.py`` from
the reference's own ``make_case`` / ``ref``.  A rebuilt case has the same keys a
reference case has (``args``, ``meta``, ``grid``, ``outputs``, ``expected``,
``comparison``, ``pointer_dtypes``, ``launch_meta``, ``kernel``); the kernel is
a signature-only stand-in with the reference kernel's name, parameter list and
autotuned constexprs, which is all ``bind_arguments`` and the registry look at.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"
INDEX = json.loads((GOLDEN / "index.json").read_text())


class _Config:
    def __init__(self, kwargs):
        self.kwargs = kwargs


class _Jit:
    def __init__(self, fn):
        self.fn = fn


class _Autotuner:
    def __init__(self, fn, autotuned):
        self.fn = _Jit(fn)
        self.configs = [_Config({name: 32 for name in autotuned})]


def make_handle(name, parameters, autotuned=()):
    """Signature-only stand-in for a ``@triton.jit`` kernel object."""
    namespace = {}
    exec(f"def {name}({', '.join(parameters)}):\n    pass\n", namespace)  # noqa: S102
    fn = namespace[name]
    return _Autotuner(fn, autotuned) if autotuned else _Jit(fn)


def kernel_parameters(kernel):
    """Parameter names of a stand-in kernel object."""
    import inspect
    target = kernel
    while not inspect.isfunction(target):
        target = target.fn
    return list(inspect.signature(target).parameters)


def tags(prefix=None, dtype=None):
    out = []
    for tag, info in sorted(INDEX.items()):
        if prefix is not None and not tag.startswith(prefix + "__"):
            continue
        if dtype is not None and info["dtype"] != dtype:
            continue
        out.append(tag)
    return out


def load(tag):
    """(case, meta) for one fixture."""
    data = np.load(GOLDEN / f"{tag}.npz")
    meta = json.loads(str(data["__meta__"]))
    args = dict(meta["scalars"])
    expected = {}
    for key in data.files:
        if key.startswith("arg__"):
            args[key[5:]] = np.array(data[key])
        elif key.startswith("expected__"):
            expected[key[10:]] = np.array(data[key])
    grid = meta["grid"]
    if grid == "callable":
        shape = meta["shape"]
        # the two autotuned operator files: (cdiv(M, BM), cdiv(N, BN)) and (rows, cdiv(cols, BN))
        if meta["kernel_name"] == "swiglu_fwd_kernel":
            grid = lambda m, s=shape: (s[0], -(-s[1] // m["BLOCK_N"]))  # noqa: E731
        else:
            grid = lambda m, s=shape: (-(-s[0] // m["BLOCK_M"]), -(-s[1] // m["BLOCK_N"]))  # noqa: E731
    else:
        grid = tuple(grid)
    case = {
        "args": args, "meta": meta["meta"], "grid": grid, "outputs": tuple(meta["outputs"]),
        "expected": expected, "comparison": meta["comparison"],
        "pointer_dtypes": meta["pointer_dtypes"], "launch_meta": meta["launch_meta"],
        "kernel": make_handle(meta["kernel_name"], meta["parameters"], meta["autotuned"]),
        "dtype": meta["dtype"], "shape": tuple(meta["shape"]),
    }
    return case, meta
