"""PPO / GRPO trainer: builds engines, couples the actor to the rollout engine, and runs the
asynchronous RL step loop.

Step loop (reference ``areal/trainer/rl_trainer.py:640-966``):

    prepare_batch (staleness-gated async rollout) -> critic values -> ref logp -> teacher logp
    -> recomputed (proximal) logp -> advantages -> actor update -> lr step -> critic update
    -> pause rollout -> push weights (version+1) -> set versions -> save / recover dump
    -> evaluate -> stats commit -> resume rollout

Rollout keeps generating while the trainer computes; only weight swaps interrupt it.

Two deployment shapes share this class:
* colocated (one process, one GPU or CPU): the rollout engine lives in the trainer process;
* SPMD split (``torchrun``): trainer ranks and rollout ranks are different processes of one
  ``torch.distributed`` world; see :mod:`areal_b200.infra.spmd`.
"""
from __future__ import annotations

import os
import time
from typing import Any, Callable, Optional

import torch
from torch.utils.data import DataLoader

from ..api.alloc_mode import AllocationMode, ModelAllocation
from ..api.cli_args import GRPOConfig, PPOConfig
from ..api.io_struct import FinetuneSpec, StepInfo, WeightUpdateMeta
from ..utils import data as D
from ..utils import logging as alog
from ..utils import perf_tracer, stats_tracker
from ..utils.evaluator import Evaluator
from ..utils.recover import RecoverHandler
from ..utils.saver import Saver
from ..utils.stats_logger import StatsLogger

logger = alog.getLogger("rl_trainer")


def _collate_list(batch):
    return list(batch)


class PPOTrainer:
    def __init__(self, config: PPOConfig, train_dataset, valid_dataset=None, tokenizer=None, rollout_engine=None,
                 actor_engine=None, model_config=None):
        self.config = config
        self.tokenizer = tokenizer
        self.train_dataset, self.valid_dataset = train_dataset, valid_dataset
        self._validate_cfg()
        self.train_dataloader = self._make_dataloader(train_dataset, config.train_dataset)
        self.valid_dataloader = self._make_dataloader(valid_dataset, config.valid_dataset) if valid_dataset is not None and config.valid_dataset else None
        bs = config.train_dataset.batch_size
        self.ft_spec = FinetuneSpec(total_train_epochs=config.total_train_epochs, dataset_size=len(train_dataset),
                                    train_batch_size=bs)
        self.model_config = model_config
        # Single-controller mode (the reference's default, areal/trainer/rl_trainer.py:131-141 and
        # :1123-1177): with ``scheduler.type`` set and no torchrun environment this process only
        # orchestrates; engines live in worker processes that a scheduler starts and are driven
        # through TrainController / RolloutController over RPC.
        self._scheduler = None
        self._owned_controllers: list = []
        if actor_engine is None and rollout_engine is None and self._wants_single_controller():
            actor_engine, rollout_engine = self._init_single_controller()
        self.actor = actor_engine or self._create_train_engine(config.actor, "actor")
        self.critic = self._create_train_engine(config.critic, "critic") if config.critic is not None else None
        self.ref = None
        if config.ref is not None and config.actor.kl_ctl > 0:
            self.ref = self._create_train_engine(config.ref, "ref")
        self.teacher = self._create_train_engine(config.teacher, "teacher") if config.teacher is not None else None
        # resumable loader; data-parallel ranks draw disjoint prompts (model-parallel peers share their head's batch)
        dp_rank = int(getattr(self.actor, "data_parallel_rank", 0) or 0)
        dp_world = int(getattr(self.actor, "data_parallel_world_size", 1) or 1)
        self.train_dataloader = self._make_dataloader(train_dataset, config.train_dataset, dp_rank, dp_world)
        self.rollout = rollout_engine or self._init_rollout()
        self.eval_rollout = None
        self.weight_update_meta = self._choose_weight_update_meta()
        self.actor.connect_engine(self.rollout, self.weight_update_meta)
        self.saver = Saver(config.saver, self.ft_spec)
        self.evaluator = Evaluator(config.evaluator, self.ft_spec)
        self.recover_handler = RecoverHandler(config.recover, self.ft_spec)
        self.stats_logger = StatsLogger(config.stats_logger, self.ft_spec, rank=getattr(self.actor, "rank", 0))
        if getattr(self.actor, "rank", 0) == 0 and config.stats_logger.fileroot:
            from ..infra.utils.exp_metadata import save_experiment_metadata

            # which source state produced this run, kept beside its logs
            save_experiment_metadata(config.stats_logger.fileroot, config.stats_logger.experiment_name or "exp", config.stats_logger.trial_name or "trial",
                                     {"allocation_mode": getattr(config, "allocation_mode", None)})
        if config.perf_tracer is not None:
            perf_tracer.configure(config.perf_tracer, rank=getattr(self.actor, "rank", 0), role="trainer")
        from ..utils.memory_profiler import MemoryProfiler

        self.memory_profiler = MemoryProfiler(getattr(config, "memory_profiler", None), rank=getattr(self.actor, "rank", 0))
        self.start_step = 0
        info = self.recover_handler.load(self._engines(), self.saver, self.evaluator, self.stats_logger,
                                         self.train_dataloader, self.rollout, self.weight_update_meta)
        if info is not None:
            self.start_step = info.last_step_info.global_step + 1
        self.step_times: list[float] = []

    # ------------------------------------------------------------------ construction helpers
    def _validate_cfg(self):
        c = self.config
        if c.actor.use_decoupled_loss and not c.actor.recompute_logprob and c.actor.prox_logp_method == "recompute":
            raise ValueError("use_decoupled_loss with prox_logp_method='recompute' needs recompute_logprob=true")
        if c.rollout.max_head_offpolicyness < 0:
            raise ValueError("max_head_offpolicyness must be >= 0")
        if c.gconfig.n_samples < 1:
            raise ValueError("gconfig.n_samples must be >= 1")

    def _wants_single_controller(self) -> bool:
        from ..utils.environ import is_single_controller

        sc = getattr(self.config, "scheduler", None)
        return sc is not None and getattr(sc, "type", None) in ("local", "ray", "slurm") and is_single_controller()

    def _init_single_controller(self):
        """Scheduler -> worker processes -> engines created over RPC. Worker counts come from the
        allocation strings (``actor.backend`` e.g. ``native:d2``, ``rollout.backend`` e.g.
        ``native:d2t1``); a worker gets a GPU when the node has one per worker."""
        import torch

        from ..api.alloc_mode import ModelAllocation
        from ..infra.controller import RolloutController, TrainController

        c = self.config
        kind = c.scheduler.type
        if kind == "local":
            from ..infra.scheduler import LocalScheduler

            n_gpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
            sched = LocalScheduler(gpu_devices=None if n_gpu else [])
        elif kind == "ray":
            from ..infra.scheduler import RayScheduler

            sched = RayScheduler()
        else:
            from ..infra.scheduler import SlurmScheduler

            sched = SlurmScheduler()
        self._scheduler = sched
        n_train = ModelAllocation.from_str(c.actor.backend).parallel.world_size if c.actor.backend else 1
        ra = ModelAllocation.from_str(c.rollout.backend).parallel if c.rollout.backend else None
        n_roll = ra.dp_size if ra is not None else 1
        use_gpu = bool(torch.cuda.is_available() and torch.cuda.device_count() >= n_train + n_roll)
        gpw = 1 if use_gpu else 0
        actor = TrainController("areal_b200.engine.train_engine.B200PPOActor", c.actor, sched, role="actor")
        rollout = RolloutController("areal_b200.engine.infer_engine.NativeInferenceEngine", c.rollout, sched, role="rollout")
        self._owned_controllers = [rollout, actor]
        mc = self.model_config
        actor.initialize(ft_spec=self.ft_spec, model_config=mc, seed=c.seed, n_workers=n_train, gpus_per_worker=gpw,
                         group_size=c.gconfig.n_samples)
        if mc is None:
            mc = actor.model_config() if hasattr(actor, "model_config") and callable(actor.model_config) else None
        rollout.initialize(n_workers=n_roll, gpus_per_worker=gpw,
                           engine_kwargs={"model_config": mc, "infer_config": c.native_infer} if mc is not None else {"infer_config": c.native_infer},
                           init_kwargs={"seed": c.seed, **({"model_path": c.actor.path} if mc is None else {})})
        return actor, rollout

    def _make_dataloader(self, dataset, dcfg, rank: int = 0, world: int = 1):
        if dataset is None or dcfg is None:
            return None
        from ..utils.dataloader import StatefulDataLoader

        # every rank hands ``batch_size`` prompts per call to its own rollout executor
        return StatefulDataLoader(dataset, dcfg.batch_size, shuffle=dcfg.shuffle, drop_last=dcfg.drop_last, collate_fn=_collate_list,
                                  seed=self.config.seed, rank=rank, world_size=world)

    def _create_train_engine(self, ecfg, role: str):
        from ..engine.train_engine import B200PPOActor, B200PPOCritic

        ecfg.experiment_name = ecfg.experiment_name or self.config.experiment_name
        ecfg.trial_name = ecfg.trial_name or self.config.trial_name
        if role == "critic":
            eng = B200PPOCritic(ecfg)
        else:
            if role in ("ref", "teacher"):
                ecfg.optimizer = None
            eng = B200PPOActor(ecfg)
        eng.create_process_group()
        eng.initialize(ft_spec=self.ft_spec, model_config=self.model_config, seed=self.config.seed)
        return eng

    def _init_rollout(self):
        from ..engine.infer_engine import NativeInferenceEngine

        c = self.config
        eos = getattr(self.tokenizer, "eos_token_id", None)
        # a trainer rank that holds only part of the model (pipeline stage, expert or tensor slice)
        # cannot lend its parameters to the engine: the engine keeps a full copy, fed by gathers
        partial = any(getattr(self.actor, a, 1) > 1 for a in ("pp_size", "ep_size", "tp_size")) or getattr(self.actor, "_z3", None) is not None
        share = self.actor.device.type == "cuda" and getattr(c.native_infer, "share_trainer_weights", True) and not partial
        if share:
            # colocated on one GPU: the rollout engine reads the trainer's bf16 parameters in
            # place (no second copy in HBM); generation is interrupted while the optimizer
            # rewrites them and resumes, re-prefilling, under the new version.
            eng = NativeInferenceEngine(c.rollout, c.native_infer, model=self.actor.model, eos_token_id=eos)
            eng.initialize(device=self.actor.device, seed=c.seed, shared_model=True,
                           train_data_parallel_size=self.actor.data_parallel_world_size)
            self.actor.before_optimizer_step = eng.pause_generation
            return eng
        eng = NativeInferenceEngine(c.rollout, c.native_infer, model_config=self.actor.model_config, eos_token_id=eos)
        eng.initialize(device=self.actor.device, seed=c.seed, train_data_parallel_size=self.actor.data_parallel_world_size)
        # start from the trainer's weights
        if partial:
            eng.update_weights_from_tensors(iter(self.actor.export_weights().items()))
        else:
            eng.update_weights_from_tensors(((n, p.data) for n, p in self.actor.model.named_parameters()))
        return eng

    def _choose_weight_update_meta(self) -> WeightUpdateMeta:
        mode = self.config.actor.weight_update_mode
        c = self.config
        if mode == "disk":
            return WeightUpdateMeta.from_disk(c.experiment_name, c.trial_name, c.cluster.fileroot)
        if hasattr(self.rollout, "remote_ranks"):
            return WeightUpdateMeta(type="xccl" if mode == "xccl" else "p2p")
        return WeightUpdateMeta(type="shared")

    def _engines(self) -> dict:
        d = {"actor": self.actor}
        if self.critic is not None:
            d["critic"] = self.critic
        return d

    # ------------------------------------------------------------------ main loop
    def train(self, workflow=None, workflow_kwargs: Optional[dict] = None, eval_workflow=None,
              eval_workflow_kwargs: Optional[dict] = None, should_accept_fn: Optional[Callable] = None,
              max_steps: Optional[int] = None) -> list[dict]:
        cfg = self.config
        steps_per_epoch = self.ft_spec.steps_per_epoch
        total = cfg.total_train_steps or self.ft_spec.total_train_steps
        if max_steps is not None:
            total = min(total, self.start_step + max_steps)
        history = []
        if self.start_step == 0 and self.valid_dataloader is not None and eval_workflow is not None:
            # ``evaluator.eval_before_train``: the initial policy's score, before any update
            self.evaluator.evaluate(lambda: self._evaluate(eval_workflow, eval_workflow_kwargs), 0, -1, -1)
        for global_step in range(self.start_step, total):
            t_step = time.perf_counter()
            epoch, step = divmod(global_step, steps_per_epoch)
            si = StepInfo(epoch=epoch, epoch_step=step, global_step=global_step, steps_per_epoch=steps_per_epoch)
            perf_tracer.set_step(global_step)
            self.memory_profiler.start(global_step)
            with stats_tracker.record_timing("rollout"), perf_tracer.trace_scope("train.rollout", category="scheduler"):
                batch = self.actor.prepare_batch(self.train_dataloader, workflow=workflow, workflow_kwargs=workflow_kwargs,
                                                 should_accept_fn=should_accept_fn, dynamic_bs=cfg.dynamic_bs)
            group_sizes = None
            if self.critic is not None:
                with stats_tracker.record_timing("critic_values"), perf_tracer.trace_scope("train.critic_values"):
                    batch["values"] = self.critic.compute_values(batch)
            if self.ref is not None:
                with stats_tracker.record_timing("ref_logp"), perf_tracer.trace_scope("train.ref_logp"):
                    batch["ref_logp"] = self.ref.compute_logp(batch) if self.ref.config.recompute_logprob or True else None
                    if batch["ref_logp"] is None:
                        batch["ref_logp"] = self.ref.forward_batch(batch, output="logprobs")
            if self.teacher is not None:
                with stats_tracker.record_timing("teacher_logp"):
                    batch["teacher_logp"] = self.teacher.forward_batch(batch, output="logprobs")
                    batch["rl_loss_weight"] = cfg.teacher.rl_loss_weight
                    batch["distill_loss_weight"] = cfg.teacher.distill_loss_weight
            with stats_tracker.record_timing("recompute_logp"), perf_tracer.trace_scope("train.recompute_logp"):
                prox = self.actor.compute_logp(batch)
                if prox is not None:
                    batch["prox_logp"] = prox
            with stats_tracker.record_timing("compute_advantage"), perf_tracer.trace_scope("train.compute_advantage"):
                self.actor.compute_advantages(batch, group_sizes=group_sizes)
            self.saver.maybe_wait_for_staging()
            with stats_tracker.record_timing("train_step"), perf_tracer.profile_scope("train.ppo_update"):
                self.actor.ppo_update(batch)      # on the steps listed in perf_tracer.profile_steps every kernel of the update is traced
                self.actor.step_lr_scheduler()
            if self.critic is not None:
                with stats_tracker.record_timing("critic_train_step"), perf_tracer.trace_scope("train.critic_update"):
                    self.critic.ppo_update(batch)
                    self.critic.step_lr_scheduler()
            self.rollout.pause()
            with stats_tracker.record_timing("update_weights"), perf_tracer.trace_scope("train.update_weights", category="comm"):
                new_version = global_step + 1
                self.actor.update_weights(self.weight_update_meta.with_version(new_version))
                self.actor.set_version(new_version)
                if self.critic is not None:
                    self.critic.set_version(new_version)
                self.rollout.set_version(new_version)
                if self.eval_rollout is not None:
                    self.eval_rollout.set_version(new_version)
            with stats_tracker.record_timing("save"), perf_tracer.trace_scope("train.save", category="io"):
                self.saver.save(self.actor, epoch, step, global_step, tokenizer=self.tokenizer)
                self.recover_handler.dump(self._engines(), si, self.saver, self.evaluator, self.stats_logger,
                                          self.train_dataloader, self.rollout)
            if self.valid_dataloader is not None and eval_workflow is not None:
                with stats_tracker.record_timing("eval"):
                    self.evaluator.evaluate(lambda: self._evaluate(eval_workflow, eval_workflow_kwargs), epoch, step, global_step)
            self.actor.clear_batches(batch)
            if self.memory_profiler.active_step is not None:
                self.memory_profiler.stop(os.path.join(cfg.cluster.fileroot or "/tmp/areal", "logs", cfg.experiment_name or "exp",
                                                       cfg.trial_name or "trial", "memory_snapshots"))
            stats = self._export_stats()
            stats["timeperf/step"] = time.perf_counter() - t_step
            self.step_times.append(stats["timeperf/step"])
            self.stats_logger.commit(epoch, step, global_step, stats)
            history.append(stats)
            self.rollout.resume()
            perf_tracer.save(step=global_step)
        return history

    def _evaluate(self, eval_workflow, eval_workflow_kwargs):
        eng = self.eval_rollout or self.rollout
        rewards = []
        for items in self.valid_dataloader:
            b = eng.rollout_batch(items, workflow=eval_workflow, workflow_kwargs=eval_workflow_kwargs)
            rewards.append(b["rewards"].float())
        if rewards:
            r = torch.cat(rewards)
            stats_tracker.get("eval").scalar(reward=float(r.mean()), n=float(r.numel()))

    def _export_stats(self) -> dict[str, float]:
        stats = self.actor.export_stats()
        if hasattr(self.rollout, "export_stats"):
            try:
                stats.update(self.rollout.export_stats())
            except Exception:
                pass
        return stats

    def close(self):
        try:
            self.saver.wait()
        except Exception as e:  # an export that failed must not mask the shutdown
            import logging as _l

            _l.getLogger("areal_b200.trainer").error("pending checkpoint export failed: %r", e)
        for e in (self.rollout, self.eval_rollout):
            if e is not None:
                e.destroy()
        self.stats_logger.close()
        for e in (self.actor, self.critic, self.ref, self.teacher):
            if e is not None:
                e.destroy()
        if self._scheduler is not None:
            try:
                self._scheduler.delete_workers()
            except Exception:
                pass
            self._scheduler = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


GRPOTrainer = PPOTrainer
