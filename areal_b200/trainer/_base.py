"""Shared skeleton of the supervised trainers (SFT / RW / DPO): dataloader -> padded batch ->
``train_batch`` through an algorithm engine -> save / recover / evaluate / stats. Mirrors the
structure the reference repeats in ``areal/trainer/{sft,rw,dpo}_trainer.py``."""
from __future__ import annotations

import time
from typing import Any, Callable, Optional

import torch
from torch.utils.data import DataLoader

from ..api.io_struct import FinetuneSpec, StepInfo
from ..utils import data as D
from ..utils import logging as alog
from ..utils import stats_tracker
from ..utils.evaluator import Evaluator
from ..utils.recover import RecoverHandler
from ..utils.saver import Saver
from ..utils.stats_logger import StatsLogger

logger = alog.getLogger("trainer")


def pad_collate(samples: list[dict[str, Any]]) -> dict[str, Any]:
    return D.pad_sequences_to_tensors(samples)


class SupervisedTrainer:
    engine_cls = None
    role = "actor"

    def __init__(self, config, train_dataset, valid_dataset=None, tokenizer=None, model_config=None, collate_fn=None,
                 engine=None):
        self.config, self.tokenizer = config, tokenizer
        self.collate_fn = collate_fn or pad_collate
        g = torch.Generator().manual_seed(config.seed)
        dc = config.train_dataset
        # ``train_dataset.num_workers``: worker processes that tokenise / collate ahead of the training loop (0: in the loop)
        self.train_dataloader = DataLoader(train_dataset, batch_size=dc.batch_size, shuffle=dc.shuffle, drop_last=dc.drop_last,
                                           collate_fn=self.collate_fn, generator=g, num_workers=max(0, int(getattr(dc, "num_workers", 0) or 0)))
        self.valid_dataloader = None
        if valid_dataset is not None:
            vb = config.valid_dataset.batch_size if config.valid_dataset else dc.batch_size
            self.valid_dataloader = DataLoader(valid_dataset, batch_size=vb, shuffle=False, collate_fn=self.collate_fn)
        self.ft_spec = FinetuneSpec(config.total_train_epochs, len(train_dataset), dc.batch_size)
        ecfg = config.actor if getattr(config, "model", None) is None else config.model
        self.engine = engine or self._build_engine(ecfg, model_config)
        self.saver = Saver(config.saver, self.ft_spec)
        self.evaluator = Evaluator(config.evaluator, self.ft_spec)
        self.recover_handler = RecoverHandler(config.recover, self.ft_spec)
        self.stats_logger = StatsLogger(config.stats_logger, self.ft_spec, rank=getattr(self.engine, "rank", 0))
        if getattr(self.engine, "rank", 0) == 0 and config.stats_logger.fileroot:
            from ..infra.utils.exp_metadata import save_experiment_metadata

            # which source state produced this run, kept beside its logs
            save_experiment_metadata(config.stats_logger.fileroot, config.stats_logger.experiment_name or "exp", config.stats_logger.trial_name or "trial",
                                     {"allocation_mode": getattr(config, "allocation_mode", None)})
        self.start_step = 0
        info = self.recover_handler.load({self.role: self.engine}, self.saver, self.evaluator, self.stats_logger,
                                         self.train_dataloader)
        if info is not None:
            self.start_step = info.last_step_info.global_step + 1

    def _build_engine(self, ecfg, model_config):
        eng = self.engine_cls(ecfg)
        eng.create_process_group()
        eng.initialize(ft_spec=self.ft_spec, model_config=model_config, seed=self.config.seed)
        return eng

    # to be provided by subclasses
    def train_step(self, batch: dict[str, Any]) -> dict[str, float]:
        raise NotImplementedError

    def eval_step(self, batch: dict[str, Any]):
        raise NotImplementedError

    def _shard_for_dp(self, batch: dict[str, Any]) -> dict[str, Any]:
        """Every DP rank loads the same global batch and keeps a token-balanced slice."""
        dp = getattr(self.engine, "dp_size", 1)
        if dp <= 1:
            return batch
        from ..utils.seqpack import balanced_greedy_partition

        lens = batch["attention_mask"].sum(1).tolist()
        groups = balanced_greedy_partition(lens, dp)
        return D.select_batch(batch, groups[self.engine.dp_rank])

    def train(self, max_steps: Optional[int] = None) -> list[dict]:
        cfg = self.config
        spe = self.ft_spec.steps_per_epoch
        total = cfg.total_train_steps or self.ft_spec.total_train_steps
        if max_steps is not None:
            total = min(total, self.start_step + max_steps)
        gen = D.cycle_dataloader(self.train_dataloader)
        for _ in range(self.start_step % max(1, spe)):
            next(gen)
        history = []
        for global_step in range(self.start_step, total):
            t0 = time.perf_counter()
            epoch, step = divmod(global_step, spe)
            batch = self._shard_for_dp(next(gen))
            with stats_tracker.record_timing("train_step"):
                self.train_step(batch)
                self.engine.step_lr_scheduler()
            self.engine.set_version(global_step + 1)
            with stats_tracker.record_timing("save"):
                self.saver.save(self.engine, epoch, step, global_step, tokenizer=self.tokenizer)
                self.recover_handler.dump({self.role: self.engine}, StepInfo(epoch, step, global_step, spe), self.saver,
                                          self.evaluator, self.stats_logger, self.train_dataloader)
            if self.valid_dataloader is not None:
                with stats_tracker.record_timing("eval"):
                    self.evaluator.evaluate(self.evaluate, epoch, step, global_step)
            stats = self.engine.export_stats()
            stats["timeperf/step"] = time.perf_counter() - t0
            self.stats_logger.commit(epoch, step, global_step, stats)
            history.append(stats)
        return history

    def evaluate(self):
        losses = []
        for batch in self.valid_dataloader:
            out = self.eval_step(self._shard_for_dp(batch))
            if out is not None:
                losses.append(float(out))
        if losses:
            stats_tracker.get("eval").scalar(loss=sum(losses) / len(losses))

    def close(self):
        self.stats_logger.close()
        self.engine.destroy()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False
