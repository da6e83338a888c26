"""Single-node SPMD deployment: one process per GPU in one ``torch.distributed`` world, split
into trainer ranks and rollout ranks.

* trainer ranks ``[0, n_train)`` run the train engine (ZeRO data parallel [+ Ulysses SP]);
* rollout ranks ``[n_train, world)`` each run a rollout engine replica with its own workflow
  executor and dataset shard and stream finished training batches to their trainer;
* control messages and trajectories travel over a ``TCPStore`` message bus (host side);
  weights travel GPU to GPU over NVLink peer memory (:mod:`areal_b200.parallel.weight_push`).

This is the role of the reference's legacy SPMD launcher + remote inference engine
(``areal/infra/launcher/local.py:268-452``, ``areal/infra/dist_rollout.py:97-271``,
``areal/infra/remote_inf_engine.py``) with the HTTP servers replaced by in-world ranks.
"""
from __future__ import annotations

import io
import os
import pickle
import threading
import time
from concurrent.futures import Future
from datetime import timedelta
from typing import Any, Optional

import torch
import torch.distributed as dist

from ..api.engine_api import InferenceEngine
from ..utils import logging as alog

logger = alog.getLogger("spmd")


class SplitWorld:
    """Rank bookkeeping of a trainer / rollout split."""

    def __init__(self, n_train: int, n_rollout: int, rank: Optional[int] = None):
        self.n_train, self.n_rollout = n_train, n_rollout
        self.world = n_train + n_rollout
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.train_ranks = list(range(n_train))
        self.rollout_ranks = list(range(n_train, self.world))

    @property
    def is_trainer(self) -> bool:
        return self.rank < self.n_train

    def rollout_peers_of(self, train_rank: int) -> list[int]:
        """Rollout ranks that feed ``train_rank`` (round-robin pairing)."""
        return [r for i, r in enumerate(self.rollout_ranks) if i % self.n_train == train_rank]

    def trainer_of(self, rollout_rank: int) -> int:
        return (rollout_rank - self.n_train) % self.n_train


def build_split_groups(split: SplitWorld, sp_size: int = 1, use_cuda: bool = True) -> dict:
    """Creates, collectively on every rank of the world, the process groups of the trainer
    side (``dist.new_group`` must be entered by all ranks in the same order). Returns the
    groups this rank belongs to: ``shard`` (all trainers), ``cpu`` (gloo mirror), ``dp`` and
    ``sp`` (this trainer's data- / sequence-parallel group) and ``world_cpu`` (gloo, all ranks)."""
    tr = split.train_ranks
    n = len(tr)
    out: dict = {"shard": None, "cpu": None, "dp": None, "sp": None}
    out["world_cpu"] = dist.new_group(list(range(split.world)), backend="gloo")
    if n > 1:
        out["shard"] = dist.new_group(tr)
        out["cpu"] = dist.new_group(tr, backend="gloo") if use_cuda else out["shard"]
    # weight-update broadcast group (baseline / CPU path): trainer head + every rollout rank
    out["wu"] = dist.new_group([tr[0]] + split.rollout_ranks)
    dp_size = n // sp_size
    me = split.rank
    for d in range(dp_size):
        ranks = [tr[d * sp_size + s] for s in range(sp_size)]
        if sp_size > 1:
            g = dist.new_group(ranks)
            if me in ranks:
                out["sp"] = g
    for s_ in range(sp_size):
        ranks = [tr[d * sp_size + s_] for d in range(dp_size)]
        if dp_size > 1:
            g = dist.new_group(ranks)
            if me in ranks:
                out["dp"] = g
    return out


class MessageBus:
    """Small key/value message bus on a dedicated TCPStore (rank 0 hosts it)."""

    def __init__(self, rank: int, world: int, host: Optional[str] = None, port: Optional[int] = None, timeout_s: float = 1800):
        host = host or os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = port or (int(os.environ.get("MASTER_PORT", "29500")) + 17)
        self.store = dist.TCPStore(host, port, world_size=world, is_master=(rank == 0), timeout=timedelta(seconds=timeout_s),
                                   wait_for_workers=False)
        self.rank = rank

    def put(self, key: str, obj: Any) -> None:
        buf = io.BytesIO()
        pickle.dump(obj, buf, protocol=pickle.HIGHEST_PROTOCOL)
        self.store.set(key, buf.getvalue())

    def get(self, key: str, timeout_s: Optional[float] = None) -> Any:
        if timeout_s is not None:
            self.store.wait([key], timedelta(seconds=timeout_s))
        else:
            self.store.wait([key])
        return pickle.loads(self.store.get(key))

    def poll(self, key: str) -> Optional[Any]:
        try:
            if self.store.check([key]):
                return pickle.loads(self.store.get(key))
        except Exception:
            return None
        return None

    def delete(self, key: str) -> None:
        try:
            self.store.delete_key(key)
        except Exception:
            pass

    def add(self, key: str, n: int = 1) -> int:
        return self.store.add(key, n)


class RemoteRolloutClient(InferenceEngine):
    """Trainer-side handle of the rollout ranks: receives ready-made training batches and
    drives the weight-update handshake."""

    def __init__(self, bus: MessageBus, split: SplitWorld, train_rank: int, wu_group=None):
        self.bus, self.split, self.train_rank = bus, split, train_rank
        self.wu_group = wu_group
        self.remote_ranks = split.rollout_ranks
        self.my_rollout_ranks = split.rollout_peers_of(train_rank)
        self._seq = {r: 0 for r in self.my_rollout_ranks}
        self._version = 0
        self.device = None

    def prepare_batch(self, dataloader=None, workflow=None, workflow_kwargs=None, should_accept_fn=None, dynamic_bs=False):
        from ..utils.data import concat_padded_tensors

        parts = []
        for r in self.my_rollout_ranks:
            key = f"traj/{r}/{self._seq[r]}"
            parts.append(self.bus.get(key))
            self.bus.delete(key)
            self._seq[r] += 1
        return concat_padded_tensors(parts) if len(parts) > 1 else parts[0]

    def rollout_batch(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None):
        return self.prepare_batch()

    def set_version(self, version: int) -> None:
        self._version = version

    def get_version(self) -> int:
        return self._version

    def pause(self):
        pass

    def resume(self):
        pass

    def pause_generation(self):
        pass

    def continue_generation(self):
        pass

    def destroy(self):
        pass

    def export_stats(self) -> dict[str, float]:
        return {}


class RolloutWorker:
    """Main loop of a rollout rank."""

    def __init__(self, engine, bus: MessageBus, split: SplitWorld, dataloader, workflow, workflow_kwargs=None,
                 flat_param: Optional[torch.Tensor] = None, wu_group=None):
        self.engine, self.bus, self.split = engine, bus, split
        self.flat_param, self.wu_group = flat_param, wu_group
        self.dataloader, self.workflow, self.workflow_kwargs = dataloader, workflow, workflow_kwargs
        self.rank = split.rank
        self._stop = threading.Event()
        self._ctl = threading.Thread(target=self._control_loop, name="rollout-control", daemon=True)
        self.push_seq = 0
        self.produced = 0

    def _control_loop(self):
        while not self._stop.is_set():
            cmd = self.bus.poll(f"wu/{self.push_seq}/pause")
            if cmd is None:
                if self.bus.poll("exit") is not None:
                    self._stop.set()
                    break
                time.sleep(0.002)
                continue
            self.engine.pause_generation()
            if self.engine.device.type == "cuda":
                torch.cuda.synchronize(self.engine.device)
            self.bus.put(f"wu/{self.push_seq}/ack/{self.rank}", 1)
            if isinstance(cmd, dict) and cmd.get("mode") == "broadcast":
                flat = self.flat_param
                for a in range(0, flat.numel(), cmd["bucket"]):
                    dist.broadcast(flat[a:a + cmd["bucket"]], src=cmd["src"], group=self.wu_group)
            done = self.bus.get(f"wu/{self.push_seq}/done")
            if self.engine.device.type == "cuda":
                torch.cuda.synchronize(self.engine.device)
            self.engine.set_version(int(done["version"]))
            self.engine.continue_generation()
            self.push_seq += 1

    def run(self, max_batches: Optional[int] = None):
        self._ctl.start()
        try:
            while not self._stop.is_set() and (max_batches is None or self.produced < max_batches):
                batch = self._next_batch()
                if batch is None:
                    break
                self.bus.put(f"traj/{self.rank}/{self.produced}", batch)
                self.produced += 1
        finally:
            self._stop.set()

    def _next_batch(self):
        ex = self.engine.workflow_executor
        holder: dict = {}

        def work():
            try:
                holder["b"] = self.engine.prepare_batch(self.dataloader, workflow=self.workflow,
                                                        workflow_kwargs=self.workflow_kwargs)
            except BaseException as e:
                holder["e"] = e

        t = threading.Thread(target=work, daemon=True)
        t.start()
        while t.is_alive():
            t.join(timeout=0.05)
            if self._stop.is_set():
                return None
        if "e" in holder:
            raise holder["e"]
        return holder["b"]


# --------------------------------------------------------------------------- launch helpers
def init_split_world(n_train: int, device: Optional[torch.device] = None):
    """Initialises ``torch.distributed`` (NCCL on CUDA, gloo on CPU) from the torchrun-style
    environment and returns ``(split, groups, bus)``."""
    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    use_cuda = device is not None and device.type == "cuda"
    if not dist.is_initialized():
        to = timedelta(seconds=float(os.environ.get("AREAL_DIST_TIMEOUT_S", "600")))
        if use_cuda:
            # No ``device_id`` here: binding the default group to a device makes every later
            # ``new_group`` call an NCCL communicator split on the NON-member ranks, also for gloo
            # sub-groups whose members never join that split; with trainer-only gloo groups
            # (2+ trainer ranks) the rollout ranks then wait in the split forever.
            dist.init_process_group("nccl", timeout=to)
        else:
            dist.init_process_group("gloo", timeout=to)
    split = SplitWorld(n_train, world - n_train, rank)
    groups = build_split_groups(split, sp_size=1, use_cuda=use_cuda)
    logger.info("rank %d: process groups ready", rank)
    bus = MessageBus(rank, world)
    logger.info("rank %d: message bus connected", rank)
    return split, groups, bus


def make_split_trainer(cfg, model_cfg, split: SplitWorld, groups: dict, bus: MessageBus, dataset, seed: int = 1,
                       symmetric: bool = True):
    """Trainer-rank side: builds the actor engine on the trainer sub-world, the remote rollout
    client and the :class:`PPOTrainer`, and pushes the initial weights."""
    from ..api.io_struct import FinetuneSpec
    from ..engine.train_engine import B200PPOActor
    from ..trainer.rl_trainer import PPOTrainer

    actor = B200PPOActor(cfg.actor)
    actor.set_train_ranks(split.train_ranks, groups)
    actor.create_process_group()
    kw = {}
    if symmetric and actor.device.type == "cuda":
        kw = dict(param_symm_group=dist.group.WORLD, param_symm_ranks=list(range(split.world)))
    ft = FinetuneSpec(cfg.total_train_epochs, len(dataset), cfg.train_dataset.batch_size)
    actor.initialize(ft_spec=ft, model_config=model_cfg, seed=seed, **kw)
    client = RemoteRolloutClient(bus, split, split.rank, wu_group=groups.get("wu"))
    trainer = PPOTrainer(cfg, dataset, model_config=model_cfg, rollout_engine=client, actor_engine=actor)
    actor.update_weights(trainer.weight_update_meta.with_version(0))
    return trainer


def run_rollout_rank(cfg, model_cfg, split: SplitWorld, groups: dict, bus: MessageBus, dataset, workflow,
                     device: torch.device, seed: int = 1, symmetric: bool = True, eos_token_id=None,
                     max_batches: Optional[int] = None):
    """Rollout-rank side: builds the engine over a flat parameter buffer laid out like the
    trainer's (peer-mapped when ``symmetric``), then produces batches until told to exit."""
    from torch.utils.data import DataLoader

    from ..engine.flat_params import FlatParamStore
    from ..engine.infer_engine import NativeInferenceEngine
    from ..models.decoder import build_model

    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    logger.info("rollout rank %d: building the model", split.rank)
    model = build_model(model_cfg, dtype=dtype, device=device, seed=seed)
    logger.info("rollout rank %d: model built, mapping the parameter buffer", split.rank)
    alloc = None
    if symmetric and device.type == "cuda":
        from ..parallel.symm import symm_empty

        def alloc(n, dt, d):
            t, _ = symm_empty(n, dt, d, dist.group.WORLD)
            t.zero_()
            return t
    n_shards = split.n_train if split.n_train > 1 else 1
    store = FlatParamStore(model, n_shards, 0, alloc_param=alloc, with_grads=False)
    logger.info("rollout rank %d: parameter buffer ready (%d elements)", split.rank, store.padded)
    engine = NativeInferenceEngine(cfg.rollout, cfg.native_infer, model=model, eos_token_id=eos_token_id)
    engine.initialize(device=device, seed=seed)
    dl = DataLoader(dataset, batch_size=cfg.train_dataset.batch_size, shuffle=True, drop_last=True, collate_fn=list,
                    generator=torch.Generator().manual_seed(seed + split.rank))
    worker = RolloutWorker(engine, bus, split, dl, workflow, flat_param=store.flat_param, wu_group=groups.get("wu"))
    try:
        worker.run(max_batches=max_batches)
    finally:
        engine.destroy()
    return worker
