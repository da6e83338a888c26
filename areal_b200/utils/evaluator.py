"""Frequency-gated evaluation hook (reference: ``areal/utils/evaluator.py``)."""
from __future__ import annotations

from typing import Callable

from .timeutil import EpochStepTimeFreqCtl


class Evaluator:
    def __init__(self, config, ft_spec=None):
        self.config, self.ft_spec = config, ft_spec
        self.freq_ctl = EpochStepTimeFreqCtl(config.freq_epochs, config.freq_steps, config.freq_secs)

    def evaluate(self, evaluate_fn: Callable, epoch: int, step: int, global_step: int):
        if global_step < 0:
            # the call before the first training step: only with ``eval_before_train`` (a baseline of the initial policy)
            return evaluate_fn() if getattr(self.config, "eval_before_train", False) else None
        steps_per_epoch = self.ft_spec.steps_per_epoch if self.ft_spec is not None else 1 << 30
        if not self.freq_ctl.check(epochs=int(step == steps_per_epoch - 1), steps=1):
            return None
        return evaluate_fn()

    def state_dict(self):
        return self.freq_ctl.state_dict()

    def load_state_dict(self, sd):
        self.freq_ctl.load_state_dict(sd)
