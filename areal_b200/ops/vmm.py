"""Pausable device memory (``ops/csrc/vmm_alloc.cu``): buffers that keep their address while their
physical memory leaves the GPU and comes back.

``PausableBuffer`` owns one such range and hands out tensors that view it; ``MemoryPool`` groups
buffers under tags (``weights``, ``kv_cache``, ``optimizer`` ...) so that an engine can release
and take back whole classes of memory (``pause(tags)`` / ``resume(tags)``) -- the interface of
``torch_memory_saver`` that the reference uses for time-sliced colocation
(``areal/utils/offload.py:29-50``, ``engine.offload()`` / ``onload()`` in
``areal/engine/fsdp_engine.py:928-959``). Captured CUDA graphs and tensors stay valid across a
pause because nothing is re-allocated: only the physical pages behind the addresses change.
"""
from __future__ import annotations

import ctypes
from typing import Iterable, Optional

import torch

from . import lib as oplib

oplib.declare("ab2_vmm_available", [], ctypes.c_int)
oplib.declare("ab2_vmm_alloc", [ctypes.c_size_t], ctypes.c_void_p)
oplib.declare("ab2_vmm_pause", [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p], ctypes.c_int)
oplib.declare("ab2_vmm_resume", [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p], ctypes.c_int)
oplib.declare("ab2_vmm_is_paused", [ctypes.c_void_p], ctypes.c_int)
oplib.declare("ab2_vmm_free", [ctypes.c_void_p], ctypes.c_int)
oplib._KERNELS_PER_CALL.update({n: 0 for n in ("ab2_vmm_available", "ab2_vmm_alloc", "ab2_vmm_pause", "ab2_vmm_resume",
                                               "ab2_vmm_is_paused", "ab2_vmm_free")})

_TYPESTR = {torch.bfloat16: "<V2", torch.float16: "<f2", torch.float32: "<f4", torch.int32: "<i4", torch.int64: "<i8",
            torch.uint8: "|u1", torch.int8: "|i1", torch.float64: "<f8"}


def available() -> bool:
    return torch.cuda.is_available() and oplib.get_lib().ab2_vmm_available() == 0


class _RawView:
    """Minimal ``__cuda_array_interface__`` carrier for a raw device address."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}
        self._owner = owner


class PausableBuffer:
    def __init__(self, nbytes: int, device=None, keep_contents: bool = True):
        """``keep_contents``: a pause saves the buffer to pinned host memory and a resume restores
        it (weights, optimizer state); False discards the contents (KV cache)."""
        if device is not None and torch.device(device).index is not None:
            torch.cuda.set_device(device)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.nbytes, self.keep_contents = int(nbytes), keep_contents
        ptr = oplib.get_lib().ab2_vmm_alloc(self.nbytes)
        if not ptr:
            raise torch.cuda.OutOfMemoryError(f"pausable allocation of {nbytes / 2 ** 30:.2f} GiB failed")
        self.ptr = int(ptr)
        self._bytes = torch.as_tensor(_RawView(self.ptr, self.nbytes, self), device=self.device)
        self._host: Optional[torch.Tensor] = None

    def tensor(self, dtype, shape=None, offset_bytes: int = 0) -> torch.Tensor:
        """A tensor over (part of) the buffer; it shares the buffer's fate when paused."""
        t = self._bytes[offset_bytes:].view(dtype) if dtype != torch.uint8 else self._bytes[offset_bytes:]
        if shape is not None:
            n = 1
            for d in shape:
                n *= d
            t = t[:n].view(shape)
        return t

    @property
    def paused(self) -> bool:
        return oplib.get_lib().ab2_vmm_is_paused(self.ptr) == 1

    def pause(self) -> None:
        host = None
        if self.keep_contents:
            if self._host is None:
                self._host = torch.empty(self.nbytes, dtype=torch.uint8).pin_memory()
            host = self._host.data_ptr()
        rc = oplib.get_lib().ab2_vmm_pause(self.ptr, host, oplib.stream_ptr())
        oplib.check(rc, "ab2_vmm_pause")

    def resume(self) -> None:
        host = self._host.data_ptr() if (self.keep_contents and self._host is not None) else None
        rc = oplib.get_lib().ab2_vmm_resume(self.ptr, host, oplib.stream_ptr())
        if rc == 3:
            raise torch.cuda.OutOfMemoryError("no device memory to resume a paused buffer")
        oplib.check(rc, "ab2_vmm_resume")

    def free(self) -> None:
        if self.ptr:
            self._bytes = None
            oplib.get_lib().ab2_vmm_free(self.ptr)
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class MemoryPool:
    """Tagged pausable buffers of one process."""

    def __init__(self):
        self._by_tag: dict[str, list[PausableBuffer]] = {}

    def empty(self, shape, dtype, tag: str, keep_contents: bool = True, device=None) -> torch.Tensor:
        n = 1
        for d in (shape if isinstance(shape, (tuple, list)) else (shape,)):
            n *= d
        buf = PausableBuffer(n * torch.empty(0, dtype=dtype).element_size(), device, keep_contents)
        self._by_tag.setdefault(tag, []).append(buf)
        return buf.tensor(dtype, tuple(shape) if isinstance(shape, (tuple, list)) else (shape,))

    def _select(self, tags: Optional[Iterable[str]]):
        tags = list(self._by_tag) if tags is None else list(tags)
        return [b for t in tags for b in self._by_tag.get(t, [])]

    def pause(self, tags: Optional[Iterable[str]] = None) -> int:
        """Releases the physical memory of the tagged buffers; returns the bytes released."""
        n = 0
        for b in self._select(tags):
            if not b.paused:
                b.pause()
                n += b.nbytes
        return n

    def resume(self, tags: Optional[Iterable[str]] = None) -> int:
        n = 0
        for b in self._select(tags):
            if b.paused:
                b.resume()
                n += b.nbytes
        return n

    def bytes(self, tags: Optional[Iterable[str]] = None) -> int:
        return sum(b.nbytes for b in self._select(tags))


_POOL: Optional[MemoryPool] = None


def pool() -> MemoryPool:
    global _POOL
    if _POOL is None:
        _POOL = MemoryPool()
    return _POOL
