"""ctypes binding of the in-tree sm_100a kernel library (``libab2_kernels.so``).

The library has a plain C ABI (raw device pointers + a CUDA stream handle). It is built
by :mod:`areal_b200.ops.build`. On a machine with a GPU a missing or unloadable library is
a hard error: no op silently falls back to PyTorch on CUDA tensors.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

import torch

_LIB = None
_LOCK = threading.Lock()
_LIB_PATH = Path(__file__).resolve().parent / "libab2_kernels.so"

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float

_SIGS = {
    "ab2_kernel_error": ([], c_int),
    "ab2_runtime_init": ([], c_int),
    "ab2_kernel_error_peek": ([c_void_p, c_void_p], c_int),
    "ab2_gemm_bf16_bcast": ([c_void_p] * 4 + [c_int] * 8 + [c_void_p], c_int),
    "ab2_tp_reduce_rmsnorm": ([c_void_p, c_int, c_ll] + [c_void_p] * 4 + [c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p], c_int),
    "ab2_ppo_token_loss": ([c_void_p] * 5 + [c_ll] + [c_void_p] * 8, c_int),
    "ab2_gae_scan": ([c_void_p] * 5 + [c_float, c_int, c_int, c_void_p, c_void_p, c_void_p], c_int),
    "ab2_push_plan": ([c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p], c_int),
    "ab2_num_sms": ([], c_int),
    "ab2_gemm_bf16": ([c_void_p] * 4 + [c_int] * 10 + [c_void_p], c_int),
    "ab2_gemm_bf16_2sm": ([c_void_p] * 4 + [c_int] * 9 + [c_void_p], c_int),
    "ab2_qknorm_rope_fwd": ([c_void_p] * 8 + [c_int] * 4 + [c_ll, c_float, c_void_p], c_int),
    "ab2_qknorm_rope_bwd": ([c_void_p] * 11 + [c_int] * 4 + [c_ll, c_ll, c_void_p], c_int),
    "ab2_gemm_grouped": ([c_void_p] * 4 + [c_int] * 9 + [c_void_p], c_int),
    "ab2_gemm_grouped_rt": ([c_void_p] * 5 + [c_int] * 9 + [c_void_p], c_int),
    "ab2_moe_route_workspace": ([c_ll, c_int], c_ll),
    "ab2_moe_route": ([c_void_p] * 2 + [c_int] * 4 + [ctypes.c_float] + [c_void_p] * 10 + [c_int] + [c_void_p] * 2, c_int),
    "ab2_gemm_splitk": ([c_void_p] * 5 + [c_int] * 7 + [c_void_p], c_int),
    "ab2_gemm_fp8": ([c_void_p] * 5 + [c_int] * 8 + [c_void_p], c_int),
    "ab2_quant_fp8": ([c_void_p] * 3 + [c_int, c_int, c_ll, c_ll, c_int, c_int, c_void_p], c_int),
    "ab2_gemm_skinny": ([c_void_p] * 6 + [c_int] * 8 + [c_void_p], c_int),
    "ab2_rmsnorm_fwd": ([c_void_p] * 6 + [c_int, c_int, c_float, c_void_p], c_int),
    "ab2_rmsnorm_bwd": ([c_void_p] * 7 + [c_int, c_int, c_void_p], c_int),
    "ab2_rope": ([c_void_p] * 4 + [c_int, c_int, c_int, c_ll, c_int, c_void_p], c_int),
    "ab2_swiglu_fwd": ([c_void_p, c_void_p, c_ll, c_int, c_void_p], c_int),
    "ab2_swiglu_bwd": ([c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p], c_int),
    "ab2_embed_fwd": ([c_void_p] * 3 + [c_int] * 3 + [c_void_p], c_int),
    "ab2_embed_bwd": ([c_void_p] * 3 + [c_int] * 3 + [c_void_p], c_int),
    "ab2_sqnorm_f32": ([c_void_p, c_ll, c_void_p, c_void_p], c_int),
    "ab2_clip_coef": ([c_void_p, c_float, c_float, c_void_p], c_int),
    "ab2_adamw": ([c_void_p] * 4 + [c_int, c_void_p, c_void_p, c_ll] + [c_float] * 5 + [c_int, c_void_p], c_int),
    "ab2_logprob_fwd": ([c_void_p] * 6 + [c_int, c_int, c_ll, c_float, c_int, c_int, c_void_p], c_int),
    "ab2_logprob_bwd": ([c_void_p] * 7 + [c_int, c_int, c_ll, c_ll, c_float, c_int, c_void_p], c_int),
    "ab2_logprob_combine": ([c_void_p, c_int, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p], c_int),
    "ab2_kv_append": ([c_void_p] * 5 + [c_int, c_int, c_int, c_ll, c_ll, c_void_p], c_int),
    "ab2_paged_decode": ([c_void_p] * 8 + [c_int] * 7 + [c_float, c_void_p], c_int),
    "ab2_paged_decode_strided": ([c_void_p] * 8 + [c_int] * 7 + [c_float, c_ll, c_void_p], c_int),
    "ab2_sample": ([c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p, ctypes.c_uint, c_void_p, c_void_p, c_void_p], c_int),
    "ab2_attn_delta": ([c_void_p] * 3 + [c_int] * 3 + [c_ll, c_ll, c_void_p], c_int),
    "ab2_attn_bwd": ([c_void_p] * 11 + [c_int] * 5 + [c_ll] * 6 + [c_float, c_int, c_void_p], c_int),
    "ab2_attn_fwd": ([c_void_p] * 7 + [c_int] * 5 + [c_ll] * 4 + [c_float, c_int, c_void_p], c_int),
}


class KernelLibraryError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    """True when CUDA is usable and the kernel library can be loaded."""
    if not torch.cuda.is_available():
        return False
    try:
        get_lib()
        return True
    except KernelLibraryError:
        return False


def get_lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        if not _LIB_PATH.exists():
            try:
                from . import build as _build

                _build.build()
            except Exception as e:  # pragma: no cover - build environment specific
                raise KernelLibraryError(f"kernel library missing and build failed: {e}") from e
        try:
            lib = ctypes.CDLL(str(_LIB_PATH))
        except OSError as e:
            raise KernelLibraryError(f"cannot load {_LIB_PATH}: {e}") from e
        for name, (args, res) in _SIGS.items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                continue  # optional symbol from a newer source file; checked at call time
            fn.argtypes = args
            fn.restype = res
        _LIB = _CountingLib(lib)
    return _LIB


# Number of kernels each exported launcher enqueues (used for launch accounting).
_KERNELS_PER_CALL = {"ab2_kernel_error_peek": 0, "ab2_gemm_splitk": 2, "ab2_paged_decode": 2, "ab2_paged_decode_strided": 2, "ab2_paged_decode_noalloc": 2, "ab2_kernel_error": 0, "ab2_runtime_init": 0, "ab2_num_sms": 0}
LAUNCHES = {"count": 0}


class _CountingLib:
    """Proxy over the CDLL that counts kernel launches issued through it."""

    def __init__(self, lib):
        object.__setattr__(self, "_lib", lib)
        object.__setattr__(self, "_cache", {})

    def __getattr__(self, name):
        c = self._cache
        if name in c:
            return c[name]
        fn = getattr(self._lib, name)
        n = _KERNELS_PER_CALL.get(name, 1)
        if n == 0:
            c[name] = fn
            return fn

        def call(*a, _fn=fn, _n=n):
            LAUNCHES["count"] += _n
            return _fn(*a)
        c[name] = call
        return call


def launch_count() -> int:
    return LAUNCHES["count"]


def declare(name: str, argtypes, restype=c_int) -> None:
    """Registers the signature of an additional exported symbol."""
    _SIGS[name] = (argtypes, restype)
    if _LIB is not None and hasattr(_LIB._lib, name):
        fn = getattr(_LIB._lib, name)
        fn.argtypes, fn.restype = argtypes, restype


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelLibraryError(f"{what} failed with code {rc}")


def kernel_error() -> int:
    """Synchronises and returns (then clears) the device-side error word: 0 means every
    bounded wait completed; non-zero identifies the wait that gave up."""
    return int(get_lib().ab2_kernel_error())


KERNEL_ERROR_NAMES = {1: "a TMA stage never landed", 2: "a pipeline stage was never released", 3: "an accumulator was never filled",
                      4: "an accumulator was never drained", 5: "a peer GPU's signal never arrived", 6: "an index was out of bounds",
                      7: "a device-side wait ran out"}


class KernelWaitTimeout(KernelLibraryError):
    """A bounded device-side wait gave up: the results of the step that saw it are not to be used."""


class ErrorPoller:
    """Polls the device error word without a synchronisation of its own: ``enqueue()`` puts a copy of
    the word into a pinned host word behind the work already on the current stream, ``check()`` reads
    that host word after the caller's own synchronisation and raises if a wait gave up. Step loops
    (one optimizer step, one decode iteration) call the pair once per step."""

    def __init__(self):
        self.word = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.pending = False

    def enqueue(self) -> None:
        rc = get_lib().ab2_kernel_error_peek(self.word.data_ptr(), stream_ptr())
        check(rc, "ab2_kernel_error_peek")
        self.pending = True

    def value(self) -> int:
        """The word as of the last ``enqueue`` (valid after a synchronisation of that stream)."""
        return int(self.word[0]) if self.pending else 0

    def check(self, what: str = "step") -> None:
        v = self.value()
        self.pending = False
        if v != 0:
            kernel_error()          # clears the device word so the next step starts clean
            self.word[0] = 0
            raise KernelWaitTimeout(f"{what}: device-side wait gave up (code {v}: {KERNEL_ERROR_NAMES.get(v, 'unknown')})")
