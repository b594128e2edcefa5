"""Build of the sm_100a operator library (``libb200ops.so``).

Plays the role of ``a100c/runtime/build.py:56-72`` (content-digest-keyed
compile of the runtime objects): every ``csrc/*.cu`` is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a`` and linked into one shared
library next to the package.  The digest of the sources, headers and flags is
stored beside the library, so an unchanged tree is never recompiled; nvcc
cross-compiles, so this works on a host without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
ROOT = PACKAGE.parent
CSRC = PACKAGE / "csrc"
INCLUDE = ROOT / "include"
LIB_DIR = PACKAGE / "_lib"
LIB_PATH = LIB_DIR / "libb200ops.so"
DIGEST_PATH = LIB_DIR / "libb200ops.digest"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: cannot build libb200ops.so")
    return found


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def source_digest() -> str:
    digest = hashlib.sha256()
    files = sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h")))
    for path in files:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(NVCC_FLAGS).encode())
    try:
        version = subprocess.run([nvcc_path(), "--version"], capture_output=True, text=True).stdout
    except OSError:
        version = ""
    digest.update(version.encode())
    return digest.hexdigest()


def is_current() -> bool:
    return (LIB_PATH.is_file() and DIGEST_PATH.is_file()
            and DIGEST_PATH.read_text().strip() == source_digest())


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile and link the library if the sources changed; return its path."""
    if not force and is_current():
        return LIB_PATH
    nvcc = nvcc_path()
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc, *flags, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{result.stdout}\n{result.stderr}")
        if verbose or ptxas_info:
            sys.stderr.write(result.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, sources()))
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objects), "-lcudart_static", "-ldl",
            "-lpthread", "-lrt"]
    result = subprocess.run(link, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    DIGEST_PATH.write_text(source_digest() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(path)
