"""Checks that an installation can run: Python dependencies, the kernel library (built for
sm_100a and loadable), a GPU if one is expected, and one numerics smoke test per kernel family.

    python -m areal_b200.tools.validate_installation [--no-gpu]

Prints one line per check and exits non-zero if a required check fails. Reference:
``areal/tools/validation_base.py`` and ``validate_docker_installation.py``."""
from __future__ import annotations

import argparse
import importlib
import sys
import traceback
from typing import Callable

REQUIRED = ["torch", "numpy", "yaml", "aiohttp"]
OPTIONAL = ["transformers", "safetensors", "uvloop", "ray", "psutil", "pynvml"]


class Report:
    def __init__(self):
        self.rows: list[tuple[str, str, str]] = []

    def run(self, name: str, fn: Callable[[], str], required: bool = True):
        try:
            self.rows.append((name, "ok", fn() or ""))
        except Exception as e:
            self.rows.append((name, "FAIL" if required else "missing", f"{type(e).__name__}: {e}"))
            if required:
                traceback.print_exc(file=sys.stderr)

    @property
    def ok(self) -> bool:
        return all(s != "FAIL" for _, s, _ in self.rows)

    def print(self):
        for n, s, d in self.rows:
            print(f"[{s:7s}] {n}: {d}")


def _import(mod: str) -> str:
    m = importlib.import_module(mod)
    return getattr(m, "__version__", "")


def _kernel_library() -> str:
    from ..ops import lib as oplib

    oplib.get_lib()
    return f"loaded {oplib._LIB_PATH} ({len(oplib._SIGS)} entry points)"


def _gpu() -> str:
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device visible")
    p = torch.cuda.get_device_properties(0)
    if (p.major, p.minor) != (10, 0):
        raise RuntimeError(f"device 0 is sm_{p.major}{p.minor}; the kernels are built for sm_100a only")
    return f"{p.name}, {p.total_memory / 2 ** 30:.0f} GiB, {p.multi_processor_count} SMs"


def _gemm_smoke() -> str:
    import torch

    from ..ops import functional as OF
    from ..ops import lib as oplib

    a = torch.randn(256, 512, device="cuda").bfloat16()
    b = torch.randn(384, 512, device="cuda").bfloat16()
    err = (OF.gemm(a, b).float() - a.float() @ b.float().t()).abs().max().item()
    if err > 0.5 or oplib.kernel_error():
        raise RuntimeError(f"GEMM mismatch (max abs err {err}, kernel error {oplib.kernel_error()})")
    return f"max abs err {err:.3f}"


def _attention_smoke() -> str:
    import torch

    from ..ops import functional as OF

    T, H, D = 256, 4, 128
    q, k, v = (torch.randn(T, H, D, device="cuda").bfloat16() for _ in range(3))
    cu = torch.tensor([0, 100, 256], device="cuda", dtype=torch.int32)
    o = OF.attention(q, k, v, cu, causal=True)
    ref = OF.attention_ref(q.float(), k.float(), v.float(), cu, True)
    err = (o.float() - ref).abs().max().item()
    if err > 0.05:
        raise RuntimeError(f"attention mismatch {err}")
    return f"max abs err {err:.4f}"


def _tiny_train_step() -> str:
    import __graft_entry__ as ge  # the repository's smoke entry

    ge.smoke()
    return "forward + backward + decode of a tiny model"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--no-gpu", action="store_true", help="skip checks that need a device")
    a = ap.parse_args(argv)
    r = Report()
    for m in REQUIRED:
        r.run(f"import {m}", lambda m=m: _import(m))
    for m in OPTIONAL:
        r.run(f"import {m}", lambda m=m: _import(m), required=False)
    r.run("import areal_b200", lambda: _import("areal_b200"))
    r.run("kernel library", _kernel_library, required=not a.no_gpu)
    if not a.no_gpu:
        r.run("gpu", _gpu)
        r.run("tcgen05 GEMM numerics", _gemm_smoke)
        r.run("flash attention numerics", _attention_smoke)
        r.run("tiny model smoke", _tiny_train_step, required=False)
    r.print()
    return 0 if r.ok else 1


if __name__ == "__main__":
    sys.exit(main())
