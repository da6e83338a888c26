"""Asynchronous reward evaluation in a shared process pool.

Behaviour follows the reference's ``AsyncRewardWrapper`` (``areal/api/reward_api.py:62``):
reward functions run in a process pool shared by all wrappers, with a per-call timeout
(15 s), retries (3) and recovery from a broken pool; a call that never succeeds yields
reward 0.
"""
from __future__ import annotations

import asyncio
import concurrent.futures as cf
import os
import threading
from concurrent.futures.process import BrokenProcessPool
from typing import Any, Callable, Optional

from ..utils import logging as alog

logger = alog.getLogger("reward")


class AsyncRewardWrapper:
    _pool: Optional[cf.Executor] = None
    _pool_workers: int = 0
    _lock = threading.Lock()
    _instances = 0

    def __init__(self, reward_fn: Callable[..., float], timeout_seconds: float = 15.0, max_workers: Optional[int] = None,
                 max_retries: int = 3, use_threads: bool = False):
        self.reward_fn = reward_fn
        self.timeout_seconds = timeout_seconds
        self.max_retries = max_retries
        self.use_threads = use_threads
        self.max_workers = max_workers or min(8, os.cpu_count() or 1)
        with AsyncRewardWrapper._lock:
            AsyncRewardWrapper._instances += 1
        self._ensure_pool()

    def _ensure_pool(self, force: bool = False):
        with AsyncRewardWrapper._lock:
            if force and AsyncRewardWrapper._pool is not None:
                try:
                    AsyncRewardWrapper._pool.shutdown(wait=False, cancel_futures=True)
                except Exception:
                    pass
                AsyncRewardWrapper._pool = None
            if AsyncRewardWrapper._pool is None:
                if self.use_threads:
                    AsyncRewardWrapper._pool = cf.ThreadPoolExecutor(max_workers=self.max_workers)
                else:
                    import multiprocessing as mp

                    AsyncRewardWrapper._pool = cf.ProcessPoolExecutor(max_workers=self.max_workers,
                                                                      mp_context=mp.get_context("spawn"))
                AsyncRewardWrapper._pool_workers = self.max_workers
            return AsyncRewardWrapper._pool

    async def __call__(self, *args, **kwargs) -> float:
        loop = asyncio.get_running_loop()
        for attempt in range(self.max_retries):
            pool = self._ensure_pool()
            try:
                fut = loop.run_in_executor(pool, _call, self.reward_fn, args, kwargs)
                return float(await asyncio.wait_for(fut, timeout=self.timeout_seconds))
            except asyncio.TimeoutError:
                logger.warning("reward function timed out after %.1fs (attempt %d)", self.timeout_seconds, attempt + 1)
                return 0.0
            except BrokenProcessPool:
                logger.warning("reward process pool broke; rebuilding (attempt %d)", attempt + 1)
                self._ensure_pool(force=True)
            except Exception as e:  # the user's function raised
                logger.warning("reward function raised %r (attempt %d)", e, attempt + 1)
                if attempt == self.max_retries - 1:
                    return 0.0
        return 0.0

    @classmethod
    def shutdown(cls):
        with cls._lock:
            if cls._pool is not None:
                cls._pool.shutdown(wait=False, cancel_futures=True)
                cls._pool = None


def _call(fn, args, kwargs):
    return fn(*args, **kwargs)
