"""Rollout data plumbing for SPMD trainers with model parallelism.

* :func:`redistribute_trajectories`: all-gathers the trajectories every data-parallel rank
  collected and deals them out again balanced by token count (FFD / KK), so no rank trains on
  a much longer batch than the others.
* :class:`DistRolloutCoordinator`: only the head of each data-parallel replica talks to the
  rollout engine; its batch is broadcast to the context- and tensor-parallel peers, which must
  feed identical tokens.

Reference: ``areal/infra/dist_rollout.py`` (``redistribute_trajectories`` :29-94, coordinator
:97-271)."""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist

from ..utils import data as D
from ..utils.seqpack import balanced_greedy_partition


def redistribute_trajectories(batch: dict[str, Any], group, granularity: int = 1) -> dict[str, Any]:
    """Balanced re-deal of padded batches over ``group`` (units of ``granularity`` consecutive
    samples, e.g. a GRPO group, stay together)."""
    if group is None or dist.get_world_size(group) == 1:
        return batch
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    gathered = D.all_gather_tensor_container(batch, group=group)
    merged = D.concat_padded_tensors(gathered)
    B = D.batch_size_of(merged)
    g = granularity if granularity > 0 and B % granularity == 0 and B // granularity >= world else 1
    lens = merged["attention_mask"].sum(1).view(B // g, g).sum(1).tolist()
    parts = balanced_greedy_partition(lens, world, equal_count=True)
    mine = [u * g + j for u in parts[rank] for j in range(g)]
    out = D.select_batch(merged, mine)
    L = int(out["attention_mask"].sum(1).max().item()) if mine else 0
    full_L = merged["attention_mask"].shape[1]
    return {k: (v[:, :L].contiguous() if torch.is_tensor(v) and v.dim() >= 2 and v.shape[1] == full_L else v) for k, v in out.items()}


class DistRolloutCoordinator:
    def __init__(self, rollout_engine, train_engine, redistribute: bool = True, granularity: int = 1):
        self.rollout, self.train = rollout_engine, train_engine
        self.redistribute = redistribute
        self.granularity = granularity

    def _share(self, batch: Optional[dict]) -> dict:
        te = self.train
        if self.redistribute and te.is_data_parallel_head() and te.data_parallel_world_size > 1:
            batch = redistribute_trajectories(batch, te.data_parallel_group, self.granularity)
        g = te.context_and_model_parallel_group
        if g is not None and dist.get_world_size(g) > 1:
            # the batch stays a host batch on every rank (the engine stages micro-batches itself); an NCCL
            # group only carries the pickled bytes through device memory
            batch = D.broadcast_tensor_container(batch, src=te.current_data_parallel_head(), group=g)
        return batch

    def rollout_batch(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None) -> dict:
        b = None
        if self.train.is_data_parallel_head():
            b = self.rollout.rollout_batch(data, workflow=workflow, workflow_kwargs=workflow_kwargs, should_accept_fn=should_accept_fn)
        return self._share(b)

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None, dynamic_bs: bool = False) -> dict:
        b = None
        if self.train.is_data_parallel_head():
            b = self.rollout.prepare_batch(dataloader, workflow=workflow, workflow_kwargs=workflow_kwargs,
                                           should_accept_fn=should_accept_fn, dynamic_bs=dynamic_bs)
        return self._share(b)
