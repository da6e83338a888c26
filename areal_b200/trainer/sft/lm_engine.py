"""Supervised fine-tuning on packed sequences: token-mean negative log-likelihood over
``loss_mask`` (reference: ``areal/trainer/sft/lm_engine.py:83``)."""
from __future__ import annotations

import torch

from ...algo.functional import sft_loss_fn
from ...utils import stats_tracker


def compute_packed_sft_loss(logprobs: torch.Tensor, entropy: torch.Tensor, input_data: dict) -> torch.Tensor:
    # next-token convention: position t predicts token t+1, so the mask is shifted left
    loss_mask = torch.roll(input_data["loss_mask"].bool(), shifts=-1, dims=0)
    cu = input_data.get("cu_seqlens")
    if cu is not None and cu.numel() > 1:
        ends = (cu[1:].long() - 1).clamp(min=0)
        ends = ends[ends < loss_mask.shape[0]]
        loss_mask = loss_mask.clone()
        loss_mask[ends] = False  # the last token of a sequence predicts nothing
    loss = sft_loss_fn(logprobs, loss_mask)
    with torch.no_grad():
        stats_tracker.denominator(n_valid_tokens=loss_mask)
        stats_tracker.stat(nll=-logprobs.detach(), denominator="n_valid_tokens")
    return loss


class LMEngine:
    def __init__(self, engine):
        self.engine = engine

    def train_lm(self, data: dict):
        self.engine.train()
        with stats_tracker.scope("sft"):
            st = self.engine.train_batch(data, loss_fn=compute_packed_sft_loss,
                                         loss_weight_fn=lambda x: x["loss_mask"].count_nonzero())
            stats_tracker.scalar(**st)
        return st

    def evaluate_lm(self, data: dict):
        self.engine.eval()
        with stats_tracker.scope("sft-eval"):
            return self.engine.eval_batch(data, loss_fn=compute_packed_sft_loss,
                                          loss_weight_fn=lambda x: x["loss_mask"].count_nonzero())
