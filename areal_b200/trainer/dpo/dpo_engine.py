"""Direct preference optimisation (sigmoid / IPO) on alternating (chosen, rejected) packed
sequences with reference log-probs supplied in the batch as ``ref_logp``
(reference: ``areal/trainer/dpo/dpo_engine.py``; loss math ``functional.py:796-857``)."""
from __future__ import annotations

import functools

import torch

from ...algo import functional as AF
from ...utils import stats_tracker


def compute_dpo_loss(logprobs: torch.Tensor, entropy: torch.Tensor, input_data: dict, beta: float,
                     loss_type: str) -> torch.Tensor:
    loss_mask = torch.roll(input_data["loss_mask"].bool(), shifts=-1, dims=0)
    cu = input_data["cu_seqlens"]
    n_real = int(cu[-1]) if cu.numel() else 0
    pc, pr, rc, rr, lc, lr_ = AF.dpo_pair_logratios(logprobs, input_data["ref_logp"], loss_mask, cu)
    n_pairs = min(pc.numel(), pr.numel())
    loss, stat = AF.dpo_preference_loss(pc[:n_pairs], pr[:n_pairs], rc[:n_pairs], rr[:n_pairs], beta, loss_type,
                                        lc[:n_pairs], lr_[:n_pairs])
    stats_tracker.scalar(dpo_acc=float(stat["accuracy"].mean()), reward_chosen=float(stat["reward_chosen"].mean()),
                         reward_rejected=float(stat["reward_rejected"].mean()))
    return loss


class DPOEngine:
    def __init__(self, engine, beta: float = 0.1, loss_type: str = "sigmoid"):
        self.engine, self.beta, self.loss_type = engine, beta, loss_type

    def _fns(self):
        return (functools.partial(compute_dpo_loss, beta=self.beta, loss_type=self.loss_type),
                lambda x: torch.tensor(max(1, (x["cu_seqlens"].numel() - 1) // 2)))

    @torch.no_grad()
    def compute_ref_logp(self, ref_engine, data: dict) -> torch.Tensor:
        return ref_engine.forward_batch(data, output="logprobs")

    def train_dpo(self, data: dict):
        self.engine.train()
        loss_fn, w = self._fns()
        with stats_tracker.scope("dpo"):
            st = self.engine.train_batch(data, loss_fn=loss_fn, loss_weight_fn=w)
            stats_tracker.scalar(**st)
        return st

    def evaluate_dpo(self, data: dict):
        self.engine.eval()
        loss_fn, w = self._fns()
        with stats_tracker.scope("dpo-eval"):
            return self.engine.eval_batch(data, loss_fn=loss_fn, loss_weight_fn=w)
