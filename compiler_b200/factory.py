"""The a100c compile protocol with native kernels behind it.

Keeps the surface a driver of the reference uses (``a100c/factory.py:313-315``
``make_compiler()``, ``a100c/driver.py:295-328`` ``compile_case(case)`` returning
an artifact with ``identity`` / ``provenance`` / ``cache_hit`` / ``sha256`` /
``compile_ms``, and the ``compile_count`` / ``cache_hits`` counters
``driver.py:291-314``).  What changes is the artifact: instead of a RISC-V
executable it is a **compiled-kernel callable** -- ``artifact[grid](*tensor and
scalar arguments, **meta)`` enqueues the pre-built sm_100a operator.

"Compiling" a case is therefore a lookup plus validation: the kernel handle is
resolved in the registry (an unknown kernel is a located refusal, like
``PipelineError`` ``driver.py:79-87``), the library is built once per source
digest (``compiler_b200/build.py``), and the identity is the digest of (kernel
name, parameter list, pointer dtypes, scalar classes, constexpr metas, library
digest, plan options).  Shapes, grids and scalar values never enter it
(``driver.py:11-17``), so one artifact serves every shape of an operator.
"""
from __future__ import annotations

import hashlib
import json
import os
import time
from dataclasses import dataclass, field

import numpy as np

from compiler_b200 import build as _build
from compiler_b200 import registry as _registry
from compiler_b200.runtime import abi


# Environment switches of the native library that change WHICH kernel runs a launch (the
# library reads each once, at its first use in the process).
KERNEL_SWITCHES = ("B200OPS_ATTN_KERNEL", "B200OPS_ATTN_P", "B200OPS_ATTN_WAVE",
                   "B200OPS_GEMM_PAIR", "B200OPS_GEMM_GROUP_M", "B200OPS_GEMM_TAIL",
                   "B200OPS_SOFTMAX_STREAM", "B200OPS_RMSNORM_STREAM")


def _kernel_switches() -> dict:
    return {name: os.environ.get(name, "") for name in KERNEL_SWITCHES}


@dataclass
class PlanOptions:
    """Options that change which kernel runs; every one of them is part of the identity
    (``CompileOptions.identity_part``, a100c/driver.py:222-244), so two artifacts compiled
    under different kernel choices never share a cache entry.  The choices are the
    ``B200OPS_*`` switches of ``KERNEL_SWITCHES``, sampled when the options are created."""
    switches: dict = field(default_factory=_kernel_switches)
    device: int = field(default_factory=lambda: int(os.environ.get("B200OPS_DEVICE", "0")))

    @property
    def attn_p_location(self) -> str:
        return self.switches.get("B200OPS_ATTN_P") or "tmem"

    def identity_part(self) -> str:
        return json.dumps({name: self.switches.get(name, "") for name in KERNEL_SWITCHES},
                          sort_keys=True)


def _scalar_class(value) -> str:
    if isinstance(value, (bool, np.bool_)):
        return "bool"
    if isinstance(value, (int, np.integer)):
        return "int"
    if isinstance(value, (float, np.floating)):
        return "float"
    return type(value).__name__


@dataclass
class Artifact:
    """What ``compile_case`` returns (``_Artifact``, a100c/driver.py:268-277)."""
    kernel: object
    identity: str
    provenance: str
    sha256: str
    cache_hit: bool = False
    compile_ms: int = 0
    stage_stats: dict = field(default_factory=dict)
    _device: object = None

    def bind(self, device):
        self._device = device
        return self

    def __getitem__(self, grid):
        artifact = self

        def launcher(*args, **meta):
            device = artifact._device
            if device is None:
                from compiler_b200.device import B200Device
                device = artifact._device = B200Device(
                    int(os.environ.get("B200OPS_DEVICE", "0")))
            device.launch(artifact.kernel, grid, list(args), dict(meta))

        return launcher


class B200Compiler:
    """``make_compiler()`` result: ``compile_case`` + counters."""

    def __init__(self, options: PlanOptions | None = None, registry=None):
        self.options = options or PlanOptions()
        self.registry = registry or _registry.default_registry()
        self.compile_count = 0
        self.cache_hits = 0
        self._cache: dict[str, Artifact] = {}
        self._library_digest = None

    def library_digest(self) -> str:
        if self._library_digest is None:
            self._library_digest = _build.source_digest()
        return self._library_digest

    def identity(self, case: dict) -> dict:
        kernel = case.get("kernel")
        if kernel is None:
            raise _registry.UnsupportedLaunch("<none>", "case", "case has no kernel")
        name, parameters, autotuned = _registry.kernel_signature(kernel)
        args = {**case.get("allocations", {}), **case.get("args", {})}
        pointer_dtypes = dict(case.get("pointer_dtypes") or {})
        layout = []
        for pname in parameters:
            value = args.get(pname, case.get("meta", {}).get(pname))
            if isinstance(value, np.ndarray):
                layout.append((pname, "ptr", abi.dtype_name(pointer_dtypes.get(pname)
                                                            or value.dtype)))
            elif pname in case.get("meta", {}):
                layout.append((pname, "meta", repr(case["meta"][pname])))
            elif pname in autotuned:
                layout.append((pname, "autotuned", ""))
            else:
                layout.append((pname, "scalar", _scalar_class(value)))
        specialization = hashlib.sha256(json.dumps([name, layout]).encode()).hexdigest()[:16]
        key = hashlib.sha256(
            ("b200ops-artifact/1\n"
             f"specialization={specialization}\n"
             f"library={self.library_digest()}\n"
             f"options={self.options.identity_part()}\n"
             f"abi={abi.ABI_VERSION}\n").encode()).hexdigest()
        return {"key": key, "specialization": specialization, "name": name}

    def compile_case(self, case: dict) -> Artifact:
        """Resolve one case to its compiled-kernel callable; idempotent per identity."""
        started = time.monotonic()
        ident = self.identity(case)
        cached = self._cache.get(ident["key"])
        if cached is not None:
            self.cache_hits += 1
            return Artifact(kernel=case["kernel"], identity=cached.identity,
                            provenance=cached.provenance, sha256=cached.sha256, cache_hit=True,
                            stage_stats=cached.stage_stats)
        self.registry.resolve(case["kernel"])  # located refusal for unknown kernels
        path = _build.build()                  # no-op when the digest matches
        self.compile_count += 1
        artifact = Artifact(
            kernel=case["kernel"], identity=ident["specialization"],
            provenance=f"compiler_b200/{self.library_digest()[:16]}",
            sha256=hashlib.sha256(path.read_bytes()).hexdigest(),
            compile_ms=int((time.monotonic() - started) * 1000),
            stage_stats={"kernel": ident["name"], "library": str(path.name)})
        self._cache[ident["key"]] = artifact
        return artifact


def make_compiler(options: PlanOptions | None = None) -> B200Compiler:
    """Factory selected by ``A100_COMPILER_FACTORY=compiler_b200.factory:make_compiler``
    (a100_support/native_device.py:89-95)."""
    return B200Compiler(options)
