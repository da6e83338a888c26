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
    """Rank bookkeeping of a trainer / rollout split.

    Trainer ranks ``[0, n_train)`` form ``dp = n_train / sp`` data-parallel replicas of ``sp``
    sequence-parallel ranks each (rank ``d * sp + s``); the first rank of a replica is its head.
    Rollout ranks ``[n_train, world)`` form ``n_rollout / rollout_tp`` tensor-parallel engine
    replicas of consecutive ranks; the first rank of a replica is its leader (the only one that
    takes requests and produces batches). Leaders feed trainer heads round-robin: with more
    leaders than heads a head merges several leaders' batches, with fewer a leader deals its
    batches to several heads in turn."""

    def __init__(self, n_train: int, n_rollout: int, rank: Optional[int] = None, sp: int = 1, rollout_tp: int = 1):
        if n_train % max(1, sp) or n_rollout % max(1, rollout_tp):
            raise ValueError(f"sp={sp} must divide the {n_train} trainer ranks and rollout_tp={rollout_tp} the {n_rollout} rollout ranks")
        self.n_train, self.n_rollout = n_train, n_rollout
        self.sp, self.rollout_tp = max(1, sp), max(1, rollout_tp)
        self.dp = n_train // self.sp
        self.n_replicas = n_rollout // self.rollout_tp
        self.world = n_train + n_rollout
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.train_ranks = list(range(n_train))
        self.rollout_ranks = list(range(n_train, self.world))
        self.heads = [d * self.sp for d in range(self.dp)]
        self.leaders = [n_train + k * self.rollout_tp for k in range(self.n_replicas)]
        if self.n_replicas >= self.dp:
            if self.n_replicas % self.dp:
                raise ValueError(f"{self.n_replicas} rollout replicas cannot be dealt evenly to {self.dp} trainer replicas")
        elif self.dp % self.n_replicas:
            raise ValueError(f"{self.dp} trainer replicas cannot share {self.n_replicas} rollout replicas evenly")

    @property
    def is_trainer(self) -> bool:
        return self.rank < self.n_train

    # ---- rollout side
    def replica_of(self, rollout_rank: int) -> int:
        return (rollout_rank - self.n_train) // self.rollout_tp

    def tp_rank_of(self, rollout_rank: int) -> int:
        return (rollout_rank - self.n_train) % self.rollout_tp

    def replica_ranks(self, k: int) -> list[int]:
        return [self.n_train + k * self.rollout_tp + j for j in range(self.rollout_tp)]

    def is_leader(self, rank: Optional[int] = None) -> bool:
        return (self.rank if rank is None else rank) in self.leaders

    def consumers_of(self, leader: int) -> list[int]:
        """Trainer heads that a rollout leader produces batches for."""
        k = self.leaders.index(leader)
        if self.n_replicas >= self.dp:
            return [self.heads[k % self.dp]]
        return [h for i, h in enumerate(self.heads) if i % self.n_replicas == k]

    # ---- trainer side
    def rollout_peers_of(self, train_rank: int) -> list[int]:
        """Rollout leaders whose batches ``train_rank`` consumes (empty unless it is a head)."""
        if train_rank not in self.heads:
            return []
        return [l for l in self.leaders if train_rank in self.consumers_of(l)]

    def trainer_of(self, rollout_rank: int) -> int:
        return self.consumers_of(self.leaders[self.replica_of(rollout_rank)])[0]


def build_split_groups(split: SplitWorld, sp_size: Optional[int] = None, use_cuda: bool = True) -> dict:
    """Creates, collectively on every rank of the world, all process groups of the deployment
    (``dist.new_group`` must be entered by all ranks in the same order). Returns the groups this
    rank belongs to: ``shard`` (all trainers), ``cpu`` (its gloo mirror), ``dp`` / ``sp`` (this
    trainer's data- / sequence-parallel group), ``wu`` (trainer head + every rollout rank: the
    broadcast baseline of the weight update), ``rtp`` / ``rtp_cpu`` (this rollout rank's
    tensor-parallel replica: data plane and gloo control plane) and ``world_cpu`` (gloo, all ranks)."""
    sp_size = split.sp if sp_size is None else sp_size
    tr = split.train_ranks
    n = len(tr)
    out: dict = {"shard": None, "cpu": None, "dp": None, "sp": None, "rtp": None, "rtp_cpu": None}
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
    out["stats"] = None
    if sp_size > 1 and dp_size > 1:
        g = dist.new_group([tr[h] for h in split.heads], backend="gloo")
        if me in split.heads:
            out["stats"] = g
    if split.rollout_tp > 1:
        for k in range(split.n_replicas):
            ranks = split.replica_ranks(k)
            g = dist.new_group(ranks)
            gc = dist.new_group(ranks, backend="gloo") if use_cuda else dist.new_group(ranks)
            if me in ranks:
                out["rtp"], out["rtp_cpu"] = g, gc
    return out


class MessageBus:
    """Small key/value message bus on a dedicated TCPStore (rank 0 hosts it)."""

    def __init__(self, rank: int, world: int, host: Optional[str] = None, port: Optional[int] = None, timeout_s: float = 1800):
        host = host or os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = port or (int(os.environ.get("MASTER_PORT", "29500")) + 17)
        self.store = dist.TCPStore(host, port, world_size=world, is_master=(rank == 0), timeout=timedelta(seconds=timeout_s),
                                   wait_for_workers=False)
        self.rank = rank

    # The store refuses values above a few MB (its server closes the connection), and a training batch
    # of long sequences is larger: values travel in pieces, announced by a small header under the key.
    CHUNK = 2 << 20

    def put(self, key: str, obj: Any) -> None:
        buf = io.BytesIO()
        pickle.dump(obj, buf, protocol=pickle.HIGHEST_PROTOCOL)
        data = buf.getvalue()
        if len(data) <= self.CHUNK:
            self.store.set(key, b"\x00" + data)
            return
        n = (len(data) + self.CHUNK - 1) // self.CHUNK
        for i in range(n):
            self.store.set(f"{key}#{i}", data[i * self.CHUNK:(i + 1) * self.CHUNK])
        self.store.set(key, b"\x01" + str(n).encode())          # the header goes last: readers wait on it

    def _read(self, key: str) -> Any:
        head = self.store.get(key)
        if head[:1] == b"\x00":
            return pickle.loads(head[1:])
        n = int(head[1:].decode())
        return pickle.loads(b"".join(self.store.get(f"{key}#{i}") for i in range(n)))

    def get(self, key: str, timeout_s: Optional[float] = None) -> Any:
        if timeout_s is not None:
            self.store.wait([key], timedelta(seconds=timeout_s))
        else:
            self.store.wait([key])
        return self._read(key)

    def poll(self, key: str) -> Optional[Any]:
        try:
            if self.store.check([key]):
                return self._read(key)
        except Exception:
            return None
        return None

    def delete(self, key: str) -> None:
        try:
            head = self.store.get(key) if self.store.check([key]) else b""
            if head[:1] == b"\x01":
                for i in range(int(head[1:].decode())):
                    self.store.delete_key(f"{key}#{i}")
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
            key = f"traj/{r}/{self.train_rank}/{self._seq[r]}"
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
    """Main loop of a rollout rank. A replica leader produces batches and deals them to the trainer
    heads it feeds; the other ranks of a tensor-parallel replica only take part in weight updates
    (their engine follows the leader's schedule in lock-step). ``staging``: a full flat parameter
    buffer in the trainer's layout for the broadcast path of a tensor-parallel replica (every rank
    receives the whole buffer and keeps its slices)."""

    def __init__(self, engine, bus: MessageBus, split: SplitWorld, dataloader, workflow, workflow_kwargs=None,
                 flat_param: Optional[torch.Tensor] = None, wu_group=None, staging=None):
        self.engine, self.bus, self.split = engine, bus, split
        self.flat_param, self.wu_group, self.staging = flat_param, wu_group, staging
        self.dataloader, self.workflow, self.workflow_kwargs = dataloader, workflow, workflow_kwargs
        self.rank = split.rank
        self.consumers = split.consumers_of(self.rank) if split.is_leader(self.rank) else []
        self._stop = threading.Event()
        self._ctl = threading.Thread(target=self._control_loop, name="rollout-control", daemon=True)
        self._ctl_exc: Optional[BaseException] = None
        self.push_seq = 0
        self.produced = 0

    def _control_loop(self):
        try:
            self._control_loop_inner()
        except BaseException as e:          # surfaced by run()
            self._ctl_exc = e
            self._stop.set()

    def _control_loop_inner(self):
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
                if self.staging is not None and self.staging.get("flat") is None:     # allocated on first use
                    self.staging["flat"] = torch.zeros(self.staging["padded"], dtype=self.flat_param.dtype, device=self.flat_param.device)
                flat = self.staging["flat"] if self.staging is not None else self.flat_param
                if cmd.get("sparse") is not None:
                    # delta push: (index, value) pairs of the elements that changed since the last push
                    k = int(cmd["sparse"])
                    idx = torch.empty(k, dtype=getattr(torch, cmd.get("index_dtype", "int32")), device=flat.device)
                    vals = torch.empty(k, dtype=flat.dtype, device=flat.device)
                    for a in range(0, k, cmd["bucket"]):
                        dist.broadcast(idx[a:a + cmd["bucket"]], src=cmd["src"], group=self.wu_group)
                        dist.broadcast(vals[a:a + cmd["bucket"]], src=cmd["src"], group=self.wu_group)
                    flat[idx.long()] = vals
                    self.delta_pushes = getattr(self, "delta_pushes", 0) + 1
                else:
                    for a in range(0, flat.numel(), cmd["bucket"]):
                        dist.broadcast(flat[a:a + cmd["bucket"]], src=cmd["src"], group=self.wu_group)
                if self.staging is not None:
                    self._reshard_from_staging()
            done = self.bus.get(f"wu/{self.push_seq}/done")
            if self.engine.device.type == "cuda":
                torch.cuda.synchronize(self.engine.device)
            self.engine.set_version(int(done["version"]))
            self.engine.continue_generation()
            self.push_seq += 1

    @torch.no_grad()
    def _reshard_from_staging(self):
        """Broadcast path of a tensor-parallel replica: slices of the full tensors -> local parameters."""
        from ..parallel import tp as TP

        st, eng = self.staging, self.engine
        params = dict(eng.model.named_parameters())
        for name, off, shape in zip(st["names"], st["offsets"], st["shapes"]):
            n = 1
            for d in shape:
                n *= d
            full = st["flat"][off:off + n].view(shape)
            params[name].data.copy_(TP.shard_tensor(st["cfg"], name, full, eng.tp_size, eng.tp_rank))

    def run(self, max_batches: Optional[int] = None):
        self._ctl.start()
        try:
            if not self.consumers:                       # follower of a tensor-parallel replica
                while not self._stop.is_set():
                    time.sleep(0.01)
            seqs = {c: 0 for c in self.consumers}
            while self.consumers and not self._stop.is_set() and (max_batches is None or self.produced < max_batches):
                for c in self.consumers:
                    batch = self._next_batch()
                    if batch is None:
                        break
                    self.bus.put(f"traj/{self.rank}/{c}/{seqs[c]}", batch)
                    seqs[c] += 1
                    self.produced += 1
                else:
                    continue
                break
        finally:
            self._stop.set()
        if self._ctl_exc is not None:
            raise RuntimeError("rollout control loop failed") from self._ctl_exc

    def _next_batch(self):
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
def init_split_world(n_train: int, device: Optional[torch.device] = None, sp: int = 1, rollout_tp: int = 1):
    """Initialises ``torch.distributed`` (NCCL on CUDA, gloo on CPU) from the torchrun-style
    environment and returns ``(split, groups, bus)``. ``sp``: Ulysses sequence-parallel degree of
    the trainers; ``rollout_tp``: tensor-parallel degree of a rollout replica."""
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
    split = SplitWorld(n_train, world - n_train, rank, sp=sp, rollout_tp=rollout_tp)
    groups = build_split_groups(split, use_cuda=use_cuda)
    logger.info("rank %d: process groups ready", rank)
    bus = MessageBus(rank, world)
    logger.info("rank %d: message bus connected", rank)
    return split, groups, bus


def make_split_trainer(cfg, model_cfg, split: SplitWorld, groups: dict, bus: MessageBus, dataset, seed: int = 1,
                       symmetric: bool = True):
    """Trainer-rank side: builds the actor engine on the trainer sub-world, the remote rollout
    client and the :class:`PPOTrainer`, and pushes the initial weights."""
    from ..api.alloc_mode import FSDPParallelStrategy
    from ..api.io_struct import FinetuneSpec
    from ..engine.train_engine import B200PPOActor
    from ..trainer.rl_trainer import PPOTrainer

    actor = B200PPOActor(cfg.actor)
    actor.set_train_ranks(split.train_ranks, groups)
    actor.create_process_group(FSDPParallelStrategy(data_parallel_size=split.dp, context_parallel_size=split.sp)
                               if split.sp > 1 else None)
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
    """Rollout-rank side: builds the engine over a flat parameter buffer (peer-mapped when
    ``symmetric``; laid out like the trainer's for a single-GPU replica, like the rank-local
    tensor-parallel slice otherwise), then produces batches until told to exit."""
    import copy

    from torch.utils.data import DataLoader

    from ..engine.flat_params import FlatParamStore, flat_layout
    from ..engine.infer_engine import NativeInferenceEngine
    from ..models.decoder import build_model

    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    tp = split.rollout_tp
    tp_rank = split.tp_rank_of(split.rank)
    n_shards = split.n_train if split.n_train > 1 else 1
    # size of the trainers' flat buffer: symmetric allocations of one group must agree on it
    meta_full = build_model(model_cfg, dtype=dtype, device="meta")
    full_names = [n for n, _ in meta_full.named_parameters()]
    full_shapes = [tuple(p.shape) for _, p in meta_full.named_parameters()]
    full_offsets, full_padded = flat_layout([p.numel() for _, p in meta_full.named_parameters()], n_shards)
    logger.info("rollout rank %d: building the model (tp %d/%d)", split.rank, tp_rank, tp)
    if tp > 1:
        from ..parallel import tp as TP

        local_cfg = TP.local_config(model_cfg, tp)
        model = build_model(local_cfg, dtype=dtype, device=device, seed=seed)
        TP.install_tp(model, groups["rtp"], tp, tp_rank)
    else:
        local_cfg = model_cfg
        model = build_model(model_cfg, dtype=dtype, device=device, seed=seed)
    alloc = None
    if symmetric and device.type == "cuda":
        from ..parallel.symm import symm_empty

        def alloc(n, dt, d):
            t, _ = symm_empty(max(n, full_padded), dt, d, dist.group.WORLD)
            t.zero_()
            return t[:n]
    store = FlatParamStore(model, n_shards if tp == 1 else 1, 0, alloc_param=alloc, with_grads=False)
    logger.info("rollout rank %d: parameter buffer ready (%d elements)", split.rank, store.padded)
    staging = None
    if tp > 1:
        # broadcast path: the whole buffer arrives in the trainer's layout and is sliced locally
        # (the buffer itself is allocated when the first broadcast update arrives)
        staging = dict(flat=None, padded=full_padded, names=full_names, shapes=full_shapes, offsets=full_offsets, cfg=model_cfg)
    rcfg = cfg.rollout
    is_leader = split.is_leader(split.rank)
    consumers = split.consumers_of(split.rank) if is_leader else []
    if len(consumers) > 1:
        # one version step consumes a batch for each of the heads this leader feeds
        rcfg = copy.copy(rcfg)
        rcfg.consumer_batch_size = cfg.rollout.consumer_batch_size * len(consumers)
        if rcfg.max_concurrent_rollouts:
            rcfg.max_concurrent_rollouts = rcfg.max_concurrent_rollouts * len(consumers)
    engine = NativeInferenceEngine(rcfg, cfg.native_infer, model_config=local_cfg, model=model, eos_token_id=eos_token_id,
                                   tp_group=groups.get("rtp") if tp > 1 else None,
                                   tp_control_group=groups.get("rtp_cpu") if tp > 1 else None)
    if tp > 1:
        engine.full_model_config = model_cfg
    engine.initialize(device=device, seed=seed, start_executor=is_leader)
    dl = DataLoader(dataset, batch_size=cfg.train_dataset.batch_size, shuffle=True, drop_last=True, collate_fn=list,
                    generator=torch.Generator().manual_seed(seed + split.rank))
    worker = RolloutWorker(engine, bus, split, dl, workflow, flat_param=store.flat_param, wu_group=groups.get("wu"), staging=staging)
    try:
        worker.run(max_batches=max_batches)
    finally:
        engine.destroy()
    return worker
