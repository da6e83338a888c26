"""Builds the sm_100a kernel library in-tree with nvcc.

Every ``csrc/*.cu`` is compiled to an object (in parallel) and linked into
``areal_b200/ops/libab2_kernels.so``. The library exposes a plain C ABI that
``areal_b200.ops.lib`` loads with ctypes, so no PyTorch headers are involved and a full
rebuild takes seconds. nvcc cross-compiles without a GPU.

Usage: ``python -m areal_b200.ops.build [--force] [--verbose]``
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
LIB = HERE / "libab2_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the kernel library needs the CUDA toolkit")
    return cand


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def sources():
    return sorted(CSRC.glob("*.cu"))


def is_current() -> bool:
    stamp = BUILD / "stamp"
    if not LIB.exists() or not stamp.exists():
        return False
    return stamp.read_text().strip() == _digest(list(sources()) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles and links the library if sources changed. Returns the library path."""
    if not force and is_current():
        return LIB
    BUILD.mkdir(exist_ok=True)
    nvcc = _nvcc()
    srcs = sources()
    logs = {}

    def compile_one(src: Path):
        obj = BUILD / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, obj, r

    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(compile_one, srcs))
    objs = []
    for src, obj, r in results:
        logs[src.name] = r.stderr
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError(f"nvcc failed on {src.name}")
        if verbose:
            sys.stderr.write(f"== {src.name}\n{r.stderr}\n")
        objs.append(str(obj))
    (BUILD / "ptxas.log").write_text("\n".join(f"== {k}\n{v}" for k, v in logs.items()))
    link = [nvcc, "-shared", "-o", str(LIB), *objs, "-lcudart"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    (BUILD / "stamp").write_text(_digest(list(srcs) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))))
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
