"""Trainer -> rollout weight update service.

Modes (``WeightUpdateMeta.type``):

* ``shared`` / in-process: trainer and rollout engine live in one process (colocated, one
  GPU); the engine's parameters are refreshed by a device copy of the trainer's flat buffer;
* ``disk``: HF safetensors written to ``meta.path`` (``weight_update_v{N}``) and loaded by the
  engine (reference ``areal/engine/fsdp_engine.py:1695-1785``);
* ``xccl``: bucketed ``dist.broadcast`` from the trainer head to every rollout rank -- the
  reference's path (``fsdp_engine.py:1596-1692``), kept as the measured baseline;
* ``p2p``: every trainer rank pushes its own shard of the flat bf16 parameter buffer straight
  into every rollout replica's buffer over NVLink peer memory with an in-kernel reshard /
  cast (see ``areal_b200.parallel.weight_push``); no gather to rank 0.

Protocol around a push (reference ``fsdp_engine.py:1596-1692``): pause generation (abort
in-flight requests, they resume under the new weights), push, bump the version, continue.
"""
from __future__ import annotations

import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from ..api.io_struct import ParamSpec, WeightUpdateMeta
from ..models import hf_io
from ..utils import logging as alog

logger = alog.getLogger("wsync")


class GatheredPusher:
    """Pipeline- or expert-parallel trainer + engine in the same process: the ranks exchange the
    tensors they own and every rank loads the full set into its engine."""

    def __init__(self, train_engine, infer_engine):
        self.train, self.infer = train_engine, infer_engine
        self.last_ms = 0.0

    def push(self, meta: Optional[WeightUpdateMeta] = None):
        t0 = time.perf_counter()
        weights = self.train.export_weights()
        self.infer.pause_generation()
        try:
            self.infer.update_weights_from_tensors(iter(weights.items()), meta)
        finally:
            self.infer.continue_generation()
        self.last_ms = (time.perf_counter() - t0) * 1e3
        return self.last_ms


class InProcessPusher:
    """Trainer and engine share the process: copy parameters tensor by tensor (device copy)."""

    def __init__(self, train_engine, infer_engine):
        self.train, self.infer = train_engine, infer_engine
        self.last_ms = 0.0

    def push(self, meta: Optional[WeightUpdateMeta] = None):
        t0 = time.perf_counter()
        self.infer.pause_generation()
        try:
            if self.infer.model is not self.train.model:
                src = dict(self.train.model.named_parameters())
                self.infer.update_weights_from_tensors(((n, p.data) for n, p in src.items()), meta)
            elif meta is not None and meta.version is not None:
                self.infer.set_version(meta.version)
        finally:
            self.infer.continue_generation()
        self.last_ms = (time.perf_counter() - t0) * 1e3
        return self.last_ms


class DiskPusher:
    def __init__(self, train_engine, infer_engine):
        self.train, self.infer = train_engine, infer_engine
        self.last_ms = 0.0

    def push(self, meta: WeightUpdateMeta):
        t0 = time.perf_counter()
        path = meta.path
        if getattr(self.train, "pp_size", 1) * getattr(self.train, "tp_size", 1) * getattr(self.train, "ep_size", 1) > 1:
            from ..api.io_struct import SaveLoadMeta

            self.train.save(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))   # collective: gathers slices / stages
        elif self.train.local_index <= 0:
            hf_io.save_model_hf(self.train.model, path)
        if self.train.cpu_group is not None:
            dist.barrier(group=self.train.cpu_group)
        self.infer.pause_generation()
        try:
            self.infer.update_weights_from_disk(meta).result()
        finally:
            self.infer.continue_generation()
        if meta.clear_checkpoint_after_load and self.train.local_index <= 0:
            import shutil

            shutil.rmtree(path, ignore_errors=True)
        self.last_ms = (time.perf_counter() - t0) * 1e3
        return self.last_ms


def make_weight_pusher(train_engine, infer_engine, meta: WeightUpdateMeta):
    if meta.type == "disk":
        return DiskPusher(train_engine, infer_engine)
    if getattr(train_engine, "_z3", None) is not None:
        # sharded parameters: the full tensors are gathered unit by unit and handed over (or written to disk above)
        if hasattr(infer_engine, "remote_ranks"):
            raise NotImplementedError("fsdp.shard_parameters with rollout ranks in other processes: use actor.weight_update_mode=disk "
                                      "(the peer-memory and broadcast paths read a replicated parameter buffer)")
        return GatheredPusher(train_engine, infer_engine)
    if meta.type in ("p2p", "xccl", "awex") and hasattr(infer_engine, "remote_ranks"):
        from ..parallel.weight_push import BroadcastWeightPusher, DistributedWeightPusher, TPWeightPusher

        symmetric = train_engine.store.flat_param.data_ptr() in train_engine._symm_handles
        if meta.type == "xccl" or not symmetric:
            return BroadcastWeightPusher(train_engine, infer_engine, infer_engine.wu_group,
                                         bucket_mb=meta.weight_chunked_mem_mb)
        rollout_tp = getattr(infer_engine.split, "rollout_tp", 1)
        if rollout_tp > 1:
            return TPWeightPusher(train_engine, infer_engine, meta, rollout_tp)
        return DistributedWeightPusher(train_engine, infer_engine, meta)
    if any(getattr(train_engine, a, 1) > 1 for a in ("pp_size", "ep_size", "tp_size")):
        return GatheredPusher(train_engine, infer_engine)
    return InProcessPusher(train_engine, infer_engine)


def param_specs_of(model, chunk_mb: int = 1024) -> list[list[ParamSpec]]:
    """HF-named parameter specs grouped into buckets of at most ``chunk_mb`` MiB."""
    named = [(n, p.detach()) for n, p in model.named_parameters()]
    buckets, cur, size = [], [], 0
    for name, t in hf_io.native_to_hf_tensors(model.cfg, named):
        spec = ParamSpec(name=name, shape=tuple(t.shape), dtype=str(t.dtype).replace("torch.", ""))
        if cur and size + spec.size > chunk_mb * 1024 * 1024:
            buckets.append(cur)
            cur, size = [], 0
        cur.append(spec)
        size += spec.size
    if cur:
        buckets.append(cur)
    return buckets


def receive_broadcast(infer_engine, meta: WeightUpdateMeta, param_specs: list[ParamSpec]):
    """Rollout-rank side of the ``xccl`` baseline: receives one bucket of HF-named tensors."""
    group = getattr(infer_engine, "weight_update_group", None)
    src = getattr(infer_engine, "weight_update_src", 0)
    dev = infer_engine.device
    tensors = []
    for spec in param_specs:
        t = torch.empty(spec.shape, dtype=getattr(torch, spec.dtype), device=dev)
        dist.broadcast(t, src=src, group=group)
        tensors.append((spec.name, t))
    params = {n: p.data for n, p in infer_engine.model.named_parameters()}
    hf_io.load_hf_tensors_into(infer_engine.model.cfg, params, tensors, strict=False)
