"""Controller-side proxy of a distributed train engine.

One controller process drives N engine workers (one per GPU) over RPC. Every public engine
method is forwarded to all workers at once (they enter the same collectives); a batch
argument is split across the data-parallel ranks with token balancing, replicated to the
sequence-parallel peers of each rank, and tensor results are merged back in the caller's
sample order. Reference: ``areal/infra/controller/train_controller.py`` (``_dispatch_tensors``
:76, ``_merge_tensors`` :154, worker environment :336-350, ``_call_workers`` :558-589,
``connect_engine`` :600, ordered teardown :403-469).
"""
from __future__ import annotations

import concurrent.futures as cf
import dataclasses
from typing import Any, Optional

import torch

from ...api.alloc_mode import ModelAllocation
from ...api.cli_args import SchedulingSpec, SchedulingStrategy, TrainEngineConfig
from ...api.io_struct import FinetuneSpec, SaveLoadMeta, WeightUpdateMeta
from ...api.scheduler_api import Job, Scheduler, Worker
from ...utils import logging as alog
from ...utils.data import concat_padded_tensors
from ...utils.network import find_free_ports
from ...utils.seqpack import balanced_greedy_partition
from ..rpc.rtensor import RTensor

logger = alog.getLogger("train_controller")


def _is_batch(x) -> bool:
    return isinstance(x, dict) and isinstance(x.get("attention_mask"), torch.Tensor)


def split_batch(batch: dict[str, Any], n_parts: int, group_size: int = 1) -> tuple[list[dict[str, Any]], list[list[int]]]:
    """Token-balanced split of a padded batch into ``n_parts`` sample subsets. Samples move in
    units of ``group_size`` consecutive rows (a GRPO group stays on one rank so group
    statistics need no communication)."""
    am = batch["attention_mask"]
    B = am.shape[0]
    g = group_size if group_size > 0 and B % group_size == 0 else 1
    n_units = B // g
    if n_units < n_parts:
        g, n_units = 1, B
    if n_units < n_parts:
        raise ValueError(f"cannot split {B} samples over {n_parts} data-parallel ranks")
    lens = am.sum(1).view(n_units, g).sum(1).tolist()
    parts = balanced_greedy_partition(lens, n_parts, equal_count=True)
    index_lists = [[u * g + j for u in units for j in range(g)] for units in parts]
    out = []
    for idx in index_lists:
        it = torch.tensor(idx, dtype=torch.long)
        sub = {}
        for k, v in batch.items():
            if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.shape[0] == B:
                sub[k] = v.index_select(0, it)
            else:
                sub[k] = v
        # trim the padding this subset no longer needs
        L = int(sub["attention_mask"].sum(1).max().item()) if len(idx) else 0
        for k, v in sub.items():
            if isinstance(v, torch.Tensor) and v.dim() >= 2 and v.shape[1] == am.shape[1]:
                sub[k] = v[:, :L].contiguous()
        out.append(sub)
    return out, index_lists


def merge_results(results: list[Any], index_lists: list[list[int]], seq_len: Optional[int] = None) -> Any:
    """Inverse of :func:`split_batch` for what the data-parallel heads returned."""
    first = results[0]
    if first is None:
        return None
    if isinstance(first, torch.Tensor):
        B = sum(len(i) for i in index_lists)
        if first.dim() == 0 or first.shape[0] != len(index_lists[0]):
            return first
        L = max([r.shape[1] for r in results if r.dim() >= 2] + ([seq_len] if seq_len else [])) if first.dim() >= 2 else None
        shape = (B,) + ((L,) + tuple(first.shape[2:]) if L is not None else ())
        out = torch.zeros(shape, dtype=first.dtype)
        for r, idx in zip(results, index_lists):
            it = torch.tensor(idx, dtype=torch.long)
            if L is not None:
                out[it, : r.shape[1]] = r
            else:
                out[it] = r
        return out
    if _is_batch(first):
        keys = first.keys()
        return {k: merge_results([r[k] for r in results], index_lists, seq_len) for k in keys}
    if isinstance(first, dict):
        # scalar statistics: workers already reduced them over the group; rank 0's copy stands
        return first
    if isinstance(first, list) and first and isinstance(first[0], dict):
        return first
    return first


class TrainController:
    """Mirrors the ``TrainEngine`` API (and the algorithm mix-ins' methods through
    ``__getattr__``) over a :class:`Scheduler`."""

    def __init__(self, engine_cls: str, config: TrainEngineConfig, scheduler: Scheduler, role: str = "actor"):
        if not isinstance(engine_cls, str):
            engine_cls = f"{engine_cls.__module__}.{engine_cls.__qualname__}"
        self.engine_cls = engine_cls
        self.config = config
        self.scheduler = scheduler
        self.role = role
        self.workers: list[Worker] = []
        self.parallel = None
        self.dp_size = self.sp_size = 1
        self.group_size = 1
        self._version = 0
        self.rollout = None
        self.weight_update_meta: Optional[WeightUpdateMeta] = None
        self._pool: Optional[cf.ThreadPoolExecutor] = None
        self._own_workers = False

    # ------------------------------------------------------------------ lifecycle
    def initialize(self, ft_spec: Optional[FinetuneSpec] = None, model_config=None, seed: int = 1, n_workers: Optional[int] = None,
                   gpus_per_worker: Optional[int] = None, group_size: int = 1, colocate_with: Optional[str] = None, **kwargs):
        cfg = self.config
        alloc = ModelAllocation.from_str(cfg.backend).parallel if cfg.backend else None
        n = n_workers or (alloc.world_size if alloc is not None else 1)
        self.group_size = group_size
        spec = dataclasses.replace(cfg.scheduling_spec[0]) if getattr(cfg, "scheduling_spec", None) else SchedulingSpec()
        if gpus_per_worker is not None:
            spec.gpu = gpus_per_worker
        strat = SchedulingStrategy(type="colocation", target=colocate_with) if colocate_with else SchedulingStrategy()
        self.scheduler.create_workers(Job(replicas=n, tasks=[spec], scheduling_strategy=strat, role=self.role))
        self._own_workers = True
        self.workers = self.scheduler.get_workers(self.role)
        self._pool = cf.ThreadPoolExecutor(max_workers=max(4, 2 * n), thread_name_prefix=f"{self.role}-rpc")
        port = find_free_ports(1)[0]
        for r, w in enumerate(self.workers):
            self.scheduler.set_worker_env(w.id, {"RANK": r, "WORLD_SIZE": n, "LOCAL_RANK": 0, "MASTER_ADDR": self.workers[0].ip,
                                                 "MASTER_PORT": port, "LOCAL_WORLD_SIZE": 1})
        self._each(lambda w: self.scheduler.create_engine(w.id, self.engine_cls, cfg, name=self.role))
        self._call_all("create_process_group", None)
        self._call_all("initialize", None, ft_spec, model_config, seed=seed, **kwargs)
        dp = self._call_all("data_parallel_world_size")
        self.dp_size = int(dp[0])
        self.sp_size = n // self.dp_size
        self.dp_ranks = [int(x) for x in self._call_all("data_parallel_rank")]
        logger.info("train controller '%s': %d workers (dp=%d, sp=%d)", self.role, n, self.dp_size, self.sp_size)
        return self

    def destroy(self):
        if self._pool is None:
            return
        try:
            self._call_all("destroy")
        except Exception as e:  # workers may already be gone
            logger.warning("destroy on workers failed: %r", e)
        if self._own_workers:
            self.scheduler.delete_workers(self.role)
        self._pool.shutdown(wait=False)
        self._pool = None

    # ------------------------------------------------------------------ RPC plumbing
    def _each(self, fn):
        futs = [self._pool.submit(fn, w) for w in self.workers]
        return [f.result() for f in futs]

    def _call_all(self, method: str, *args, **kwargs):
        return self._each(lambda w: self.scheduler.call_engine(w.id, method, *args, engine_name=self.role, **kwargs))

    def _call_one(self, rank: int, method: str, *args, **kwargs):
        return self.scheduler.call_engine(self.workers[rank].id, method, *args, engine_name=self.role, **kwargs)

    def _call_per_worker(self, method: str, per_worker_args: list[tuple], kwargs: dict):
        futs = [self._pool.submit(self.scheduler.call_engine, w.id, method, *a, engine_name=self.role, **kwargs)
                for w, a in zip(self.workers, per_worker_args)]
        return [f.result() for f in futs]

    def _custom_function_call(self, method: str, *args, **kwargs):
        """Forwards ``method``; the first batch-shaped argument is split over data-parallel
        ranks, tensor results are merged back into the caller's order."""
        pos = next((i for i, a in enumerate(args) if _is_batch(a) or isinstance(a, RTensor)), None)
        if pos is None:
            res = self._call_all(method, *args, **kwargs)
            return res[0]
        batch = args[pos]
        if isinstance(batch, RTensor):
            # shards stay where they are; each data-parallel rank fetches its share itself
            lens = [sum(s.seqlens) for s in batch.shards]
            parts = balanced_greedy_partition(lens, self.dp_size, equal_count=True)
            subs = [RTensor([batch.shards[i] for i in p]) for p in parts]
            index_lists = None
        else:
            subs, index_lists = split_batch(batch, self.dp_size, self.group_size)
        per_worker = [tuple(args[:pos]) + (subs[self.dp_ranks[r]],) + tuple(args[pos + 1:]) for r in range(len(self.workers))]
        res = self._call_per_worker(method, per_worker, kwargs)
        heads = {}
        for r, out in enumerate(res):
            heads.setdefault(self.dp_ranks[r], out)
        ordered = [heads[d] for d in range(self.dp_size)]
        if index_lists is None:
            return ordered[0] if not isinstance(ordered[0], torch.Tensor) else torch.cat(ordered, 0)
        merged = merge_results(ordered, index_lists, seq_len=batch["attention_mask"].shape[1])
        if _is_batch(merged):
            batch.update(merged)
            return batch
        return merged

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)

        def call(*args, **kwargs):
            return self._custom_function_call(name, *args, **kwargs)
        call.__name__ = name
        return call

    # ------------------------------------------------------------------ TrainEngine surface
    @property
    def data_parallel_world_size(self) -> int:
        return self.dp_size

    @property
    def data_parallel_rank(self) -> int:
        return 0

    @property
    def rank(self) -> int:
        return 0

    def is_data_parallel_head(self) -> bool:
        return True

    def train(self, mode: bool = True):
        self._call_all("train", mode)
        return self

    def eval(self):
        return self.train(False)

    def set_version(self, version: int):
        self._version = version
        self._call_all("set_version", version)

    def get_version(self) -> int:
        return self._version

    def step_lr_scheduler(self):
        self._call_all("step_lr_scheduler")

    def save(self, meta: SaveLoadMeta):
        self._call_all("save", meta)

    def load(self, meta: SaveLoadMeta):
        self._call_all("load", meta)

    def export_stats(self) -> dict[str, float]:
        return self._call_all("export_stats")[0]

    def clear_batches(self, *batches):
        """Frees the shards behind remote-tensor handles once a step no longer needs them."""
        by_node: dict[str, list[str]] = {}
        for b in batches:
            if isinstance(b, RTensor):
                for s in b.shards:
                    by_node.setdefault(s.node_addr, []).append(s.shard_id)
        from ..scheduler.local import http_json

        for addr, ids in by_node.items():
            try:
                http_json(f"http://{addr}/data/clear", {"shard_ids": ids}, timeout=30)
            except Exception as e:
                logger.warning("clearing shards on %s failed: %r", addr, e)

    # ------------------------------------------------------------------ rollout coupling
    def connect_engine(self, rollout, meta: WeightUpdateMeta):
        self.rollout = rollout
        self.weight_update_meta = meta

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None, dynamic_bs: bool = False):
        return self.rollout.prepare_batch(dataloader, workflow=workflow, workflow_kwargs=workflow_kwargs,
                                          should_accept_fn=should_accept_fn, dynamic_bs=dynamic_bs)

    def rollout_batch(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None):
        return self.rollout.rollout_batch(data, workflow=workflow, workflow_kwargs=workflow_kwargs,
                                          should_accept_fn=should_accept_fn)

    def update_weights(self, meta: Optional[WeightUpdateMeta] = None):
        """Weights travel trainer workers -> rollout workers. ``disk``: the trainer writes a
        checkpoint, rollout workers load it. ``http``: rollout workers pull the tensors of
        trainer rank 0 through the shard store (small models / CPU)."""
        meta = meta or self.weight_update_meta
        if self.rollout is None:
            return
        if meta.type == "disk":
            self._call_all("save", SaveLoadMeta(path=meta.path, weight_format="hf", with_optim=False))
            self.rollout.update_weights_from_disk(meta)
        else:
            # parameters are replicated on every trainer rank: rank 0 alone exports them
            handle = self._call_one(0, "export_weights", return_rtensor=True)
            self.rollout.update_weights_from_handle(handle, meta)
            self.clear_batches(handle)
