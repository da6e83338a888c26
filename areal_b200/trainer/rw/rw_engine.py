"""Reward-model training: Bradley-Terry loss on the terminal-token scores of
(chosen, rejected) pairs laid out alternately in the batch
(reference: ``areal/trainer/rw/rw_engine.py``)."""
from __future__ import annotations

import torch

from ...algo.functional import rw_loss_fn
from ...utils import stats_tracker


def compute_rw_loss(values: torch.Tensor, input_data: dict) -> torch.Tensor:
    cu = input_data["cu_seqlens"].long()
    n_seqs = cu.numel() - 1
    n_pairs = n_seqs // 2 * 2
    last = (cu[1:n_pairs + 1] - 1).clamp(min=0)
    scores = values[last]
    loss, stat = rw_loss_fn(scores)
    stats_tracker.scalar(acc=float(stat["acc"]), margin=float(stat["margin"]))
    return loss


class RWEngine:
    def __init__(self, engine):
        self.engine = engine

    def train_rw(self, data: dict):
        self.engine.train()
        with stats_tracker.scope("rw"):
            st = self.engine.train_batch(data, loss_fn=compute_rw_loss,
                                         loss_weight_fn=lambda x: torch.tensor(max(1, (x["cu_seqlens"].numel() - 1) // 2)))
            stats_tracker.scalar(**st)
        return st

    def evaluate_rw(self, data: dict):
        self.engine.eval()
        with stats_tracker.scope("rw-eval"):
            return self.engine.eval_batch(data, loss_fn=compute_rw_loss,
                                          loss_weight_fn=lambda x: torch.tensor(max(1, (x["cu_seqlens"].numel() - 1) // 2)))
