"""Periodic model export (reference: ``areal/utils/saver.py:34-191``). Paths:
``{fileroot}/checkpoints/{user}/{experiment}/{trial}/{name}/epoch{e}epochstep{s}globalstep{g}``."""
from __future__ import annotations

import getpass
import os
from typing import Optional

from ..api.io_struct import SaveLoadMeta
from .timeutil import EpochStepTimeFreqCtl


class Saver:
    def __init__(self, config, ft_spec=None, for_recover: bool = False):
        self.config, self.ft_spec, self.for_recover = config, ft_spec, for_recover
        self.freq_ctl = EpochStepTimeFreqCtl(config.freq_epochs, config.freq_steps, config.freq_secs)
        self._async = None

    @staticmethod
    def get_save_root(experiment_name: str, trial_name: str, fileroot: str) -> str:
        return os.path.join(fileroot, "checkpoints", getpass.getuser(), experiment_name, trial_name)

    @staticmethod
    def get_model_save_root(experiment_name: str, trial_name: str, fileroot: str, name: str = "default") -> str:
        return os.path.join(Saver.get_save_root(experiment_name, trial_name, fileroot), name)

    @staticmethod
    def get_model_save_path(experiment_name, trial_name, fileroot, epoch: int, step: int, globalstep: int,
                            name: str = "default") -> str:
        return os.path.join(Saver.get_model_save_root(experiment_name, trial_name, fileroot, name),
                            f"epoch{epoch}epochstep{step}globalstep{globalstep}")

    def save(self, engine, epoch: int, step: int, global_step: int, name: str = "default", tokenizer=None,
             processor=None, base_model_path: Optional[str] = None, force: bool = False) -> Optional[str]:
        steps_per_epoch = self.ft_spec.steps_per_epoch if self.ft_spec is not None else 1 << 30
        epochs = int(step == steps_per_epoch - 1)
        if not force and not self.freq_ctl.check(epochs=epochs, steps=1):
            return None
        c = self.config
        path = self.get_model_save_path(c.experiment_name, c.trial_name, c.fileroot, epoch, step, global_step, name)
        fmt = "sharded" if self.for_recover else "hf"
        mode = getattr(c, "mode", "auto")
        use_async = (mode == "async" or (mode == "auto" and getattr(getattr(engine, "device", None), "type", "cpu") == "cuda")) \
            and not self.for_recover and hasattr(engine, "model") and getattr(engine, "tp_size", 1) == 1 \
            and not getattr(engine, "use_lora", False) and getattr(engine, "local_index", 0) <= 0
        if use_async:
            from ..models import hf_io
            from .async_checkpoint import AsyncCheckpointWriter

            if self._async is None:
                self._async = AsyncCheckpointWriter(getattr(c, "max_pinned_gb", 17.5))
            cfg_m = engine.model.cfg
            named = [(n, p.detach()) for n, p in engine.model.named_parameters()]

            def write(host_named, path=path, cfg_m=cfg_m, tokenizer=tokenizer):
                hf_io.save_hf_sharded(path, cfg_m, hf_io.native_to_hf_tensors(cfg_m, host_named))
                if tokenizer is not None and hasattr(tokenizer, "save_pretrained"):
                    tokenizer.save_pretrained(path)
            self._async.save(named, write, path)
            return path
        engine.save(SaveLoadMeta(path=path, weight_format=fmt, with_optim=self.for_recover, tokenizer=tokenizer,
                                 processor=processor, base_model_path=base_model_path))
        return path

    def maybe_wait_for_staging(self):
        """Called before the optimizer rewrites the weights: the device->host copy of an
        asynchronous export must be complete by then."""
        if self._async is not None:
            self._async.wait_staging()

    def wait(self):
        """Blocks until an export in flight is on disk (end of training, before loading it)."""
        if self._async is not None:
            self._async.wait()

    def state_dict(self):
        return self.freq_ctl.state_dict()

    def load_state_dict(self, sd):
        self.freq_ctl.load_state_dict(sd)
