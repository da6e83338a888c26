"""Checkpoint-based recovery of a whole training run.

``RecoverInfo`` carries the step position plus the state of the saver / evaluator / stats
logger / dataloader; ``RecoverHandler.dump`` writes a sharded engine checkpoint (weights +
optimizer) and the info file, ``load`` restores them and tells the caller which weight
version must be re-pushed to the rollout engines (``global_step + 1``). Reference:
``areal/utils/recover.py`` (RecoverInfo :41-149, dump :266, load :318-408,
check_if_recover :511).
"""
from __future__ import annotations

import getpass
import json
import os
import pickle
from dataclasses import asdict, dataclass, field
from typing import Any, Optional

from ..api.io_struct import SaveLoadMeta, StepInfo
from . import logging as alog
from .timeutil import EpochStepTimeFreqCtl

logger = alog.getLogger("recover")


@dataclass
class RecoverInfo:
    last_step_info: StepInfo
    saver_info: dict = field(default_factory=dict)
    evaluator_info: dict = field(default_factory=dict)
    stats_logger_info: dict = field(default_factory=dict)
    dataloader_info: Any = None
    checkpoint_info: dict = field(default_factory=dict)
    rollout_stat: dict = field(default_factory=dict)

    def dump(self, path: str):
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "step_info.json"), "w") as f:
            json.dump(asdict(self.last_step_info), f)
        with open(os.path.join(path, "recover_info.pkl"), "wb") as f:
            pickle.dump(dict(saver_info=self.saver_info, evaluator_info=self.evaluator_info,
                             stats_logger_info=self.stats_logger_info, dataloader_info=self.dataloader_info,
                             checkpoint_info=self.checkpoint_info, rollout_stat=self.rollout_stat), f)

    @classmethod
    def load(cls, path: str) -> "RecoverInfo":
        with open(os.path.join(path, "step_info.json")) as f:
            si = StepInfo(**json.load(f))
        with open(os.path.join(path, "recover_info.pkl"), "rb") as f:
            d = pickle.load(f)
        return cls(last_step_info=si, **d)


def check_if_recover(config, run_id: int = 0) -> bool:
    """``on``/``auto``: recover when a checkpoint exists (``on`` insists on one for
    ``run_id > 0``); ``off``/``disabled``: never."""
    mode = config.mode
    if mode in ("off", "disabled"):
        return False
    exists = os.path.exists(os.path.join(RecoverHandler.recover_root(config), "step_info.json"))
    if mode == "on" and run_id > 0 and not exists:
        raise FileNotFoundError("recover.mode=on but no recover checkpoint was found")
    return exists


class RecoverHandler:
    def __init__(self, config, ft_spec=None):
        self.config, self.ft_spec = config, ft_spec
        self.freq_ctl = EpochStepTimeFreqCtl(config.freq_epochs, config.freq_steps, config.freq_secs)

    @staticmethod
    def recover_root(config) -> str:
        return os.path.join(config.fileroot or "/tmp/areal", "checkpoints", getpass.getuser(), config.experiment_name,
                            config.trial_name, "recover_checkpoint")

    def dump(self, engines: dict, step_info: StepInfo, saver=None, evaluator=None, stats_logger=None, dataloader=None,
             rollout=None, force: bool = False) -> Optional[str]:
        if self.config.mode == "disabled":
            return None
        steps_per_epoch = self.ft_spec.steps_per_epoch if self.ft_spec is not None else 1 << 30
        if not force and not self.freq_ctl.check(epochs=int(step_info.epoch_step == steps_per_epoch - 1), steps=1):
            return None
        root = self.recover_root(self.config)
        for name, eng in engines.items():
            eng.save(SaveLoadMeta(path=os.path.join(root, name), weight_format="sharded",
                                  with_optim=not self.config.no_save_optim))
        dl_state = dataloader.state_dict() if dataloader is not None and hasattr(dataloader, "state_dict") else None
        info = RecoverInfo(
            last_step_info=step_info, saver_info=saver.state_dict() if saver else {},
            evaluator_info=evaluator.state_dict() if evaluator else {},
            stats_logger_info=stats_logger.state_dict() if stats_logger else {}, dataloader_info=dl_state,
            rollout_stat=asdict(rollout.workflow_executor.staleness.get_stats()) if rollout is not None and
            getattr(rollout, "workflow_executor", None) is not None else {})
        rank0 = all(getattr(e, "local_index", 0) <= 0 for e in engines.values())
        if rank0:
            info.dump(root)
        logger.info("recover checkpoint written at global step %d", step_info.global_step)
        return root

    def load(self, engines: dict, saver=None, evaluator=None, stats_logger=None, dataloader=None, rollout=None,
             weight_update_meta=None) -> Optional[RecoverInfo]:
        if not check_if_recover(self.config, run_id=int(os.environ.get("AREAL_RECOVER_RUN", "0"))):
            return None
        root = self.recover_root(self.config)
        info = RecoverInfo.load(root)
        for name, eng in engines.items():
            eng.load(SaveLoadMeta(path=os.path.join(root, name), weight_format="sharded",
                                  with_optim=not self.config.no_load_optim))
        if saver:
            saver.load_state_dict(info.saver_info)
        if evaluator:
            evaluator.load_state_dict(info.evaluator_info)
        if stats_logger:
            stats_logger.load_state_dict(info.stats_logger_info)
        if dataloader is not None and info.dataloader_info is not None and hasattr(dataloader, "load_state_dict"):
            dataloader.load_state_dict(info.dataloader_info)
        version = info.last_step_info.global_step + 1
        for eng in engines.values():
            eng.set_version(version)
        if rollout is not None:
            actor = engines.get("actor") or next(iter(engines.values()))
            if weight_update_meta is not None and getattr(actor, "_weight_pusher", None) is not None:
                actor.update_weights(weight_update_meta.with_version(version))
            rollout.set_version(version)
            ex = getattr(rollout, "workflow_executor", None)
            if ex is not None:
                ex.staleness.on_version_recovered(version)
        logger.info("recovered from global step %d (weight version %d)", info.last_step_info.global_step, version)
        return info
