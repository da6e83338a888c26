"""PPO critic: value forward and clipped value loss
(reference: ``areal/trainer/ppo/critic.py:24,115``)."""
from __future__ import annotations

import functools
from typing import Any

import torch

from ...algo import functional as AF
from ...utils import data as D
from ...utils import stats_tracker


class PPOCritic:
    def __init__(self, config, engine):
        self.config, self.engine = config, engine

    @torch.no_grad()
    def compute_values(self, data: dict[str, Any]) -> torch.Tensor:
        self.engine.eval()
        return self.engine.forward_batch(data, output="values")

    def ppo_update(self, data: dict[str, Any]) -> list[dict[str, float]]:
        cfg = self.config
        self.engine.train()
        B = data["attention_mask"].shape[0]
        from ...utils.seqpack import balanced_greedy_partition

        lens = data["attention_mask"].sum(-1).tolist()
        groups = [g for g in balanced_greedy_partition(lens, min(max(1, cfg.ppo_n_minibatches), B)) if g]
        loss_fn = functools.partial(critic_loss_fn, eps_clip=cfg.eps_clip,
                                    loss_type=getattr(cfg, "value_loss_type", "mse"))
        out = []
        for g in groups:
            mb = D.select_batch(data, g)
            with stats_tracker.scope("ppo_critic"):
                st = self.engine.train_batch(mb, loss_fn=loss_fn, loss_weight_fn=lambda x: x["loss_mask"].count_nonzero())
                stats_tracker.scalar(**st)
            out.append(st)
        return out


def critic_loss_fn(values: torch.Tensor, input_data: dict, eps_clip: float, loss_type: str = "mse") -> torch.Tensor:
    loss_mask = input_data["loss_mask"].bool()
    loss, stat = AF.ppo_critic_loss_fn(values.float(), input_data["values"].float(), input_data["returns"].float(),
                                       eps_clip, loss_mask, loss_type)
    stats_tracker.denominator(n_valid_tokens=loss_mask)
    stats_tracker.stat(value_loss=stat["loss"], value_clip_ratio=stat["clip_mask"].float(),
                       new_values=values.detach().float(), denominator="n_valid_tokens")
    return loss
