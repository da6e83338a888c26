"""Asynchronous Hugging Face export: parameters are copied to pinned host memory on a side
CUDA stream (``staging``; the trainer may overwrite the weights as soon as it finishes), and
a background thread writes the safetensors shards from the host copy. Staging is chunked so
the pinned pool stays under ``max_pinned_gb``. Reference: ``areal/utils/async_checkpoint.py``
and ``Saver.maybe_wait_for_staging`` (``areal/utils/saver.py``)."""
from __future__ import annotations

import threading
from typing import Callable, Iterable, Optional

import torch

from . import logging as alog

logger = alog.getLogger("async_ckpt")


class AsyncCheckpointWriter:
    def __init__(self, max_pinned_gb: float = 17.5):
        self.max_pinned_bytes = int(max_pinned_gb * 2 ** 30)
        self._staged = threading.Event()
        self._staged.set()
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None
        self._stream = None
        self.last_path: Optional[str] = None

    def _stage(self, named: Iterable[tuple[str, torch.Tensor]]) -> list[tuple[str, torch.Tensor]]:
        """Device -> pinned host copies on a side stream; returns host tensors."""
        named = list(named)
        cuda = any(t.is_cuda for _, t in named)
        out = []
        if cuda:
            if self._stream is None:
                self._stream = torch.cuda.Stream()
            self._stream.wait_stream(torch.cuda.current_stream())
            budget = 0
            with torch.cuda.stream(self._stream):
                for n, t in named:
                    nbytes = t.numel() * t.element_size()
                    pin = budget + nbytes <= self.max_pinned_bytes
                    h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=pin)
                    h.copy_(t.detach(), non_blocking=pin)
                    budget += nbytes if pin else 0
                    out.append((n, h))
            self._stream.synchronize()
        else:
            out = [(n, t.detach().clone()) for n, t in named]
        return out

    def save(self, named_tensors: Iterable[tuple[str, torch.Tensor]], write_fn: Callable[[list[tuple[str, torch.Tensor]]], None],
             path: Optional[str] = None) -> None:
        """``write_fn(host_named)`` runs in the background once staging is done. A previous
        write still in flight is waited for first (one checkpoint at a time)."""
        self.wait()
        self._staged.clear()
        self._error = None
        try:
            host = self._stage(named_tensors)
        finally:
            self._staged.set()
        self.last_path = path

        def run():
            try:
                write_fn(host)
            except BaseException as e:  # surfaced by the next wait()
                logger.error("asynchronous checkpoint write failed: %r", e)
                self._error = e
        self._thread = threading.Thread(target=run, name="async-ckpt-writer", daemon=True)
        self._thread.start()

    def wait_staging(self) -> None:
        self._staged.wait()

    def wait(self) -> None:
        """Blocks until the write in flight (if any) is on disk; re-raises its error."""
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            e, self._error = self._error, None
            raise RuntimeError("asynchronous checkpoint write failed") from e

    @property
    def busy(self) -> bool:
        return self._thread is not None and self._thread.is_alive()
