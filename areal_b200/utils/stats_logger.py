"""Per-step metric sink: always a local JSONL + console table; tensorboard / wandb /
swanlab when configured and importable (reference: ``areal/utils/stats_logger.py``)."""
from __future__ import annotations

import getpass
import json
import os
import time
from typing import Optional

from . import logging as alog

logger = alog.getLogger("stats")


class StatsLogger:
    def __init__(self, config, ft_spec=None, rank: int = 0, exp_config=None):
        self.config, self.ft_spec, self.rank = config, ft_spec, rank
        self.start = time.perf_counter()
        self._last_commit_step = -1
        self._tb = None
        self._wandb = None
        self._fh = None
        if rank == 0:
            self._init(exp_config)

    @staticmethod
    def get_log_path(config) -> str:
        return os.path.join(config.fileroot or "/tmp/areal", "logs", getpass.getuser(), config.experiment_name or "exp",
                            config.trial_name or "trial")

    def _init(self, exp_config):
        c = self.config
        d = self.get_log_path(c)
        os.makedirs(d, exist_ok=True)
        if getattr(c, "jsonl", True):
            self._fh = open(os.path.join(d, "stats.jsonl"), "a")
        if c.tensorboard.path:
            try:
                from torch.utils.tensorboard import SummaryWriter

                self._tb = SummaryWriter(log_dir=c.tensorboard.path)
            except Exception as e:  # pragma: no cover
                logger.warning("tensorboard unavailable: %r", e)
        if c.wandb.mode != "disabled":
            try:
                import wandb

                w = c.wandb
                if w.wandb_base_url:
                    os.environ["WANDB_BASE_URL"] = w.wandb_base_url
                if w.wandb_api_key:
                    os.environ["WANDB_API_KEY"] = w.wandb_api_key
                cfg = {**(w.config or {}), **(exp_config if isinstance(exp_config, dict) else {})} or exp_config
                # a stable run id (experiment, trial, suffix): a recovered run resumes its own curves
                run_id = f"{c.experiment_name}_{c.trial_name}_{w.id_suffix}" if w.id_suffix else None
                wandb.init(mode=w.mode, entity=w.entity, project=w.project or c.experiment_name, name=w.name or c.trial_name, job_type=w.job_type,
                           group=w.group or f"{c.experiment_name}_{c.trial_name}", notes=w.notes, tags=w.tags, config=cfg, dir=d, id=run_id,
                           resume="allow", force=True)
                self._wandb = wandb
            except Exception as e:  # pragma: no cover
                logger.warning("wandb unavailable: %r", e)

        # swanlab and trackio share wandb's call shape: init(project, name, config) / log(dict, step) / finish()
        self._trackers = []
        sw = c.swanlab
        if (sw.mode or "disabled") != "disabled":
            self._open_tracker("swanlab", project=sw.project or c.experiment_name, experiment_name=sw.name or c.trial_name,
                               config={**(sw.config or {}), **(exp_config if isinstance(exp_config, dict) else {})} or None,
                               logdir=sw.logdir or os.path.join(d, "swanlab"), mode=sw.mode)
        tk = c.trackio
        if tk.mode != "disabled":
            self._open_tracker("trackio", project=tk.project or c.experiment_name, name=tk.name or c.trial_name,
                               config=exp_config if isinstance(exp_config, dict) else None, space_id=tk.space_id)

    def _open_tracker(self, module: str, **init_kw):
        try:
            import importlib

            m = importlib.import_module(module)
            m.init(**{k: v for k, v in init_kw.items() if v is not None})
            self._trackers.append(m)
        except Exception as e:
            logger.warning("%s unavailable: %r", module, e)

    def commit(self, epoch: int, step: int, global_step: int, data):
        if self.rank != 0:
            return
        items = data if isinstance(data, list) else [data]
        merged = {}
        for d in items:
            merged.update(d)
        total = self.ft_spec.total_train_steps if self.ft_spec is not None else 0
        logger.info("epoch %d step %d (global %d/%d) %.1fs since start", epoch + 1, step + 1, global_step + 1, total,
                    time.perf_counter() - self.start)
        keys = sorted(merged)
        show = [k for k in keys if k.startswith("timeperf/")] + \
               [k for k in keys if not k.endswith(("/min", "/max")) and not k.startswith("timeperf/")][:40]
        logger.info("stats: " + ", ".join(f"{k}={merged[k]:.4g}" for k in show))
        if self._fh:
            self._fh.write(json.dumps(dict(epoch=epoch, step=step, global_step=global_step, **merged)) + "\n")
            self._fh.flush()
        if self._tb:
            for k, v in merged.items():
                self._tb.add_scalar(k, v, global_step)
        if self._wandb:
            self._wandb.log(merged, step=global_step)
        for m in getattr(self, "_trackers", ()):
            m.log(merged, step=global_step)
        self._last_commit_step = global_step

    def close(self):
        if self._fh:
            self._fh.close()
        if self._tb:
            self._tb.close()
        if self._wandb:
            self._wandb.finish()
        for m in getattr(self, "_trackers", ()):
            m.finish()

    def state_dict(self):
        return {"last_commit_step": self._last_commit_step}

    def load_state_dict(self, sd):
        self._last_commit_step = sd.get("last_commit_step", -1)
