"""Admission control for asynchronous rollout: bounds concurrency and off-policyness.

Capacity formula (reference: ``areal/infra/staleness_manager.py:79-113``):

    capacity = min( max(1, max_concurrent) - running,
                    (max_staleness + version + 1) * max(1, consumer_bs) - (accepted + running) )

Rejected samples do not consume staleness budget. After a restart
``on_version_recovered`` re-seeds ``accepted = version * consumer_bs`` (:115-131).
"""
from __future__ import annotations

import threading
from typing import Callable, Protocol

from ..api.io_struct import RolloutStat


class VersionProvider(Protocol):
    def get_version(self) -> int: ...


class StalenessManager:
    def __init__(self, version_provider: VersionProvider, max_concurrent_rollouts: int, consumer_batch_size: int,
                 max_staleness: int):
        self.version_provider = version_provider
        self.max_concurrent_rollouts = max_concurrent_rollouts
        self.consumer_batch_size = consumer_batch_size
        self.max_staleness = max_staleness
        self._lock = threading.Lock()
        self._stat = RolloutStat()

    def get_pending_limit(self) -> int:
        return (self.max_staleness + 1) * max(1, self.consumer_batch_size)

    def get_capacity(self) -> int:
        with self._lock:
            version = self.version_provider.get_version()
            concurrency = max(1, self.max_concurrent_rollouts) - self._stat.running
            budget = (self.max_staleness + version + 1) * max(1, self.consumer_batch_size)
            staleness = budget - (self._stat.accepted + self._stat.running)
            return min(concurrency, staleness)

    def on_version_recovered(self, version: int) -> None:
        with self._lock:
            self._stat.accepted = version * max(1, self.consumer_batch_size)
            self._stat.running = 0

    def on_rollout_enqueued(self) -> None:
        with self._lock:
            self._stat.enqueued += 1

    def on_rollout_submitted(self) -> None:
        with self._lock:
            self._stat.enqueued -= 1
            self._stat.running += 1

    def on_rollout_accepted(self) -> None:
        with self._lock:
            self._stat.running -= 1
            self._stat.accepted += 1

    def on_rollout_rejected(self) -> None:
        with self._lock:
            self._stat.running -= 1
            self._stat.rejected += 1

    def get_stats(self) -> RolloutStat:
        with self._lock:
            s = self._stat
            return RolloutStat(enqueued=s.enqueued, accepted=s.accepted, running=s.running, rejected=s.rejected)
