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

    def __init__(self, bus: MessageBus, split: SplitWorld, train_rank: int):
        self.bus, self.split, self.train_rank = bus, split, train_rank
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

    def __init__(self, engine, bus: MessageBus, split: SplitWorld, dataloader, workflow, workflow_kwargs=None):
        self.engine, self.bus, self.split = engine, bus, split
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
