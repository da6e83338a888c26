"""Sharded AdamW over a :class:`FlatParamStore` plus learning-rate schedules.

Step protocol (reference: ``areal/engine/fsdp_engine.py:696-727`` and
``fsdp_utils/grad.py:112-232``): global L2 grad norm over all shards -> clip coefficient ->
non-finite norm skips the update (``update_successful = 0``) -> fused AdamW on the local
shard (fp32 master, bf16 compute copy refreshed in the same kernel). The clip coefficient
and the skip flag stay on the device, so a step issues no host synchronisation until the
caller reads the returned statistics.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import functional as OF
from .flat_params import FlatParamStore


def lr_lambda(step: int, total_steps: int, warmup_steps: int, kind: str, min_lr_ratio: float) -> float:
    """Multiplier of the base LR at ``step`` (0-based): linear warm-up, then constant /
    linear / cosine decay to ``min_lr_ratio``."""
    if warmup_steps > 0 and step < warmup_steps:
        return float(step + 1) / float(warmup_steps)
    if kind == "constant":
        return 1.0
    span = max(1, total_steps - warmup_steps)
    prog = min(1.0, max(0.0, (step - warmup_steps) / span))
    if kind == "linear":
        return min_lr_ratio + (1.0 - min_lr_ratio) * (1.0 - prog)
    if kind == "cosine":
        return min_lr_ratio + (1.0 - min_lr_ratio) * 0.5 * (1.0 + math.cos(math.pi * prog))
    raise ValueError(f"unknown lr scheduler {kind}")


class ShardedAdamW:
    def __init__(self, store: FlatParamStore, cfg, total_steps: int = 1, group=None, optimizer_dtype=torch.float32):
        self.store, self.cfg, self.group = store, cfg, group
        n, dev = store.shard_numel, store.device
        self.master = store.param_shard.detach().to(torch.float32).clone()
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        self.state = torch.zeros(4, dtype=torch.float32, device=dev)
        self.step_count = 0
        self.sched_step = 0
        self.total_steps = max(1, total_steps)
        ws = cfg.warmup_steps
        self.warmup_steps = ws if ws is not None else int(math.ceil(cfg.warmup_steps_proportion * self.total_steps))
        self.sgd = cfg.type == "sgd"

    # ------------------------------------------------------------------ lr
    def current_lr(self) -> float:
        return self.cfg.lr * lr_lambda(self.sched_step, self.total_steps, self.warmup_steps,
                                       self.cfg.lr_scheduler_type, self.cfg.min_lr_ratio)

    def lr_scheduler_step(self) -> None:
        self.sched_step += 1

    # ------------------------------------------------------------------ step
    def step(self, grad_shard: torch.Tensor, inv_scale: float = 1.0, norm_already_global: bool = False,
             precomputed_sumsq: Optional[torch.Tensor] = None) -> dict:
        """``grad_shard``: reduced fp32 gradient of this rank's shard. Returns the statistics
        tensor (device): [sumsq, coef, finite, norm]. ``precomputed_sumsq``: global squared norm
        worked out by the caller (tensor parallelism de-duplicates replicated parameters)."""
        st = self.state
        st.zero_()
        if precomputed_sumsq is not None:
            st[0:1].copy_(precomputed_sumsq.to(st.dtype))
        else:
            OF.sqnorm_accumulate_(grad_shard, st)
            if not norm_already_global and self.group is not None and dist.is_initialized() and dist.get_world_size(self.group) > 1:
                dist.all_reduce(st[0:1], group=self.group)
        OF.clip_coef_(st, float(self.cfg.gradient_clipping or 0.0), inv_scale)
        self.step_count += 1
        lr = self.current_lr()
        if self.sgd:
            ok = st[2]
            self.master.add_(grad_shard * st[1] * ok, alpha=-lr)
            self.store.param_shard.copy_(self.master.to(self.store.dtype))
        else:
            OF.adamw_step_(self.master, self.exp_avg, self.exp_avg_sq, grad_shard, self.store.param_shard, st, lr,
                           self.cfg.beta1, self.cfg.beta2, self.cfg.eps, self.cfg.weight_decay, self.step_count)
        return {"state": st, "lr": lr}

    # ------------------------------------------------------------------ (de)serialisation
    def state_dict(self) -> dict:
        return dict(master=self.master.cpu(), exp_avg=self.exp_avg.cpu(), exp_avg_sq=self.exp_avg_sq.cpu(),
                    step_count=self.step_count, sched_step=self.sched_step, shard_range=self.store.shard_range,
                    world_size=self.store.world_size)

    def load_state_dict(self, sd: dict) -> None:
        if tuple(sd["shard_range"]) != tuple(self.store.shard_range) or sd["world_size"] != self.store.world_size:
            raise ValueError("optimizer state was saved with a different sharding")
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.step_count, self.sched_step = int(sd["step_count"]), int(sd["sched_step"])

    def resync_master(self) -> None:
        """Re-reads the master copy from the compute weights (after loading a checkpoint)."""
        self.master.copy_(self.store.param_shard.to(torch.float32))
