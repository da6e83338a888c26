"""Allocator snapshots of selected training steps.

``MemoryProfilerConfig(enabled, profile_steps, max_entries)``: on the listed global steps the
trainer brackets the step with ``start()`` / ``stop(dir)``; the CUDA caching allocator records
every allocation and free with its stack in between and the snapshot is written as
``memory_snapshot_step{N}_rank{R}.pickle`` (open it at pytorch.org/memory_viz). Role of
``start_memory_profile`` / ``stop_memory_profile`` in the reference
(``areal/trainer/rl_trainer.py:813-839``, ``areal/engine/megatron_engine.py:1733``). Without a
CUDA device the calls do nothing and report so.
"""
from __future__ import annotations

import os
from typing import Optional

import torch


class MemoryProfiler:
    def __init__(self, config=None, rank: int = 0):
        self.config, self.rank = config, rank
        self.enabled = bool(config is not None and getattr(config, "enabled", False))
        self.steps = frozenset(int(s) for s in (getattr(config, "profile_steps", None) or []))
        self.active_step: Optional[int] = None

    def wants(self, step: int) -> bool:
        return self.enabled and step in self.steps

    def start(self, step: int) -> bool:
        if not self.wants(step) or not torch.cuda.is_available():
            return False
        torch.cuda.memory._record_memory_history(max_entries=int(getattr(self.config, "max_entries", 100000)))
        self.active_step = step
        return True

    def stop(self, out_dir: str) -> Optional[str]:
        if self.active_step is None:
            return None
        os.makedirs(out_dir, exist_ok=True)
        path = os.path.join(out_dir, f"memory_snapshot_step{self.active_step}_rank{self.rank}.pickle")
        try:
            torch.cuda.memory._dump_snapshot(path)
        finally:
            torch.cuda.memory._record_memory_history(enabled=None)
            self.active_step = None
        return path
