"""Case staging and launch for a ``Device`` -- the driver side of the protocol.

The reference's harness does this in ``ops/harness/opslib/device.py``:
``bind_arguments`` (:232-260) builds the positional / keyword lists from the
kernel signature, ``stage_case`` (:377-415) uploads every array of ``args`` /
``allocations`` once (aliased host arrays as one allocation), and
``StagedCase.launch`` (:341-349) merges buffers, metas and per-launch overrides
and calls ``device.launch(kernel, grid, positional, keywords)``.

This module is the CALLER-SIDE STAND-IN for hosts that do not have the reference tree (the
GPU box): it is not part of the operator path and nothing behind ``B200Device.launch`` uses
it.  Its users are the tests and the measuring lane (``lane.py``) when they run without the
reference's ``opslib``; a case dict that runs through the reference's ``stage_case`` runs
through this one unchanged, and ``B200Device`` works with either
(``tests/test_reference_objects.py`` drives the device with the reference's own functions
and real kernel objects and compares the two).
"""
from __future__ import annotations

import inspect

import numpy as np

from compiler_b200.registry import kernel_signature


def bind_arguments(kernel, values):
    """Positional and keyword argument lists for ``kernel`` from a name -> value map:
    autotuner-supplied constexprs are skipped, defaults fill gaps, keyword-only
    parameters become keywords (device.py:232-260)."""
    _, parameters, autotuned = kernel_signature(kernel)
    positional, keywords = [], {}
    for name, parameter in parameters.items():
        if name in values:
            value = values[name]
        elif name in autotuned:
            continue
        elif parameter.default is not inspect.Parameter.empty:
            value = parameter.default
        else:
            raise KeyError(f"missing kernel argument {name!r}")
        if parameter.kind == inspect.Parameter.KEYWORD_ONLY:
            keywords[name] = value
        else:
            positional.append(value)
    return positional, keywords


def _alias_groups(arrays: dict) -> list[list[str]]:
    names = list(arrays)
    group_of = {name: i for i, name in enumerate(names)}
    for i, left in enumerate(names):
        for right in names[i + 1:]:
            if np.shares_memory(arrays[left], arrays[right]):
                old, new = group_of[right], group_of[left]
                for name in names:
                    if group_of[name] == old:
                        group_of[name] = new
    groups: dict[int, list[str]] = {}
    for name in names:
        groups.setdefault(group_of[name], []).append(name)
    return list(groups.values())


class StagedCase:
    """Buffers on the device, arguments bound; ``launch()`` only launches."""

    def __init__(self, case, device, buffers, kernel):
        self._case, self._device, self._buffers, self._kernel = case, device, buffers, kernel
        self._bound = None  # (positional, keywords) per launch of the case, bound once

    def buffer(self, name):
        return self._buffers[name]

    def launch(self) -> None:
        """Launch the case.  Arguments are bound on the first call and kept: buffers, metas
        and overrides of a staged case do not change, and a benchmark's repeated launches
        should cost the device call, not the signature inspection."""
        case = self._case
        if self._bound is None:
            bound = []
            for overrides in case.get("launches", ({},)):
                values = {**self._buffers, **case.get("meta", {}), **overrides}
                values = {k: (v.item() if isinstance(v, np.generic) else v)
                          for k, v in values.items()}
                positional, keywords = bind_arguments(self._kernel, values)
                bound.append((positional, {**keywords, **case.get("launch_meta", {})}))
            self._bound = bound
        for positional, keywords in self._bound:
            self._device.launch(self._kernel, case["grid"], positional, keywords)

    def outputs(self) -> dict:
        return {name: self._device.download(self._buffers[name])
                for name in self._case["outputs"]}


def stage_case(case: dict, device, kernel=None) -> StagedCase:
    """Upload the case's arrays once and bind the kernel arguments (device.py:377-415)."""
    kernel = kernel if kernel is not None else case.get("kernel")
    if kernel is None:
        raise ValueError("case has no kernel")
    host = {**case.get("allocations", {}), **case.get("args", {})}
    pointer_types = case.get("pointer_dtypes", {}) or {}
    arrays = {name: value for name, value in host.items() if isinstance(value, np.ndarray)}
    buffers = {}
    for group in _alias_groups(arrays):
        if len(group) > 1:
            buffers.update(device.upload_aliased({n: arrays[n] for n in group}, pointer_types))
        else:
            name = group[0]
            buffers[name] = device.upload(arrays[name], pointer_types.get(name))
    for name, value in host.items():
        if not isinstance(value, np.ndarray):
            buffers[name] = value
    return StagedCase(case, device, buffers, kernel)


def run_case(case: dict, device, kernel=None) -> dict:
    staged = stage_case(case, device, kernel)
    staged.launch()
    return staged.outputs()
