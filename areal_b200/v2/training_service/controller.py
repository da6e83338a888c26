"""Training-service controller: the client of a set of training workers (one per data-parallel
head). Splits a batch across workers by token count, calls the same route on all of them at
once, merges tensor answers back into the caller's order. Reference:
``areal/v2/training_service/controller/controller.py`` and ``data_proxy/dispatcher.py``."""
from __future__ import annotations

import concurrent.futures as cf
from typing import Any, Optional

import torch

from ...infra.controller.train_controller import merge_results, split_batch
from ...infra.rpc.serialization import deserialize_value, serialize_value
from ..common import call


class TrainingServiceClient:
    def __init__(self, worker_addresses: list[str], group_size: int = 1, timeout: float = 7200.0):
        self.workers = list(worker_addresses)
        self.group_size = group_size
        self.timeout = timeout
        self._pool = cf.ThreadPoolExecutor(max_workers=max(4, len(self.workers)))
        self._version = 0

    def _post_all(self, path: str, bodies: list[dict]) -> list[dict]:
        futs = [self._pool.submit(call, f"http://{a}{path}", b, None, None, self.timeout) for a, b in zip(self.workers, bodies)]
        return [f.result() for f in futs]

    def _batch_call(self, path: str, batch: dict[str, Any], **kwargs):
        n = len(self.workers)
        subs, idx = split_batch(batch, n, self.group_size) if n > 1 else ([batch], [list(range(batch["attention_mask"].shape[0]))])
        res = self._post_all(path, [serialize_value({"batch": s, **kwargs}) for s in subs])
        outs = [deserialize_value(r["result"]) for r in res]
        merged = merge_results(outs, idx, seq_len=batch["attention_mask"].shape[1])
        if isinstance(merged, dict) and isinstance(merged.get("attention_mask"), torch.Tensor):
            batch.update(merged)
            return batch
        return merged

    # ---- PPO
    def compute_logp(self, batch):
        return self._batch_call("/ppo/actor/compute_logp", batch)

    def compute_advantages(self, batch, **kw):
        return self._batch_call("/ppo/actor/compute_advantages", batch, **kw)

    def ppo_update(self, batch):
        return self._batch_call("/ppo/actor/update", batch)

    def compute_values(self, batch):
        return self._batch_call("/ppo/critic/compute_values", batch)

    # ---- supervised
    def train_lm(self, batch):
        return self._batch_call("/sft/train", batch)

    def evaluate_lm(self, batch):
        return self._batch_call("/sft/eval", batch)

    def train_rw(self, batch):
        return self._batch_call("/rw/train", batch)

    def train_dpo(self, batch):
        return self._batch_call("/dpo/train", batch)

    # ---- control
    def set_version(self, version: int):
        self._version = version
        self._post_all("/set_version", [{"version": version}] * len(self.workers))

    def get_version(self) -> int:
        return self._version

    def step_lr_scheduler(self):
        self._post_all("/step_lr_scheduler", [{}] * len(self.workers))

    def save(self, meta):
        self._post_all("/save", [serialize_value({"meta": meta})] * len(self.workers))

    def load(self, meta):
        self._post_all("/load", [serialize_value({"meta": meta})] * len(self.workers))

    def export_stats(self) -> dict:
        return call(f"http://{self.workers[0]}/export_stats")["stats"]

    def health(self) -> list[dict]:
        return [call(f"http://{a}/health") for a in self.workers]
