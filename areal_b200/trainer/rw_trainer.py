"""Reward-model trainer (reference: ``areal/trainer/rw_trainer.py:76-485``). Samples carry
``chosen_ids`` / ``rejected_ids``; batches interleave chosen, rejected, chosen, ..."""
from __future__ import annotations

import torch

from ..engine.train_engine import B200RWEngine
from ..utils import data as D
from ._base import SupervisedTrainer


def pair_collate(samples):
    seqs = []
    for s in samples:
        for key in ("chosen_ids", "rejected_ids"):
            ids = torch.as_tensor(s[key])
            seqs.append(dict(input_ids=ids, loss_mask=torch.ones_like(ids, dtype=torch.int32)))
    return D.pad_sequences_to_tensors(seqs)


class RWTrainer(SupervisedTrainer):
    engine_cls = B200RWEngine

    def __init__(self, config, train_dataset, valid_dataset=None, **kw):
        kw.setdefault("collate_fn", pair_collate)
        super().__init__(config, train_dataset, valid_dataset, **kw)

    def _shard_for_dp(self, batch):
        dp = getattr(self.engine, "dp_size", 1)
        if dp <= 1:
            return batch
        n_pairs = batch["attention_mask"].shape[0] // 2
        mine = [i for i in range(n_pairs) if i % dp == self.engine.dp_rank]
        return D.select_batch(batch, [j for i in mine for j in (2 * i, 2 * i + 1)])

    def train_step(self, batch):
        return self.engine.train_rw(batch)

    def eval_step(self, batch):
        return self.engine.evaluate_rw(batch)
