"""Frequency control by epochs / steps / seconds and simple value schedules
(reference: ``areal/utils/timeutil.py`` FrequencyControl :17, EpochStepTimeFreqCtl :145,
schedulers :184-285)."""
from __future__ import annotations

import math
import time
from typing import Optional


class FrequencyControl:
    """Fires when ``frequency_steps`` calls or ``frequency_seconds`` seconds have passed."""

    def __init__(self, frequency_seconds: Optional[float] = None, frequency_steps: Optional[int] = None,
                 initial_value: bool = False):
        self.frequency_seconds, self.frequency_steps = frequency_seconds, frequency_steps
        self._last_time = time.monotonic()
        self._steps = 0
        self._initial = initial_value
        self.total_checks = 0

    def check(self, steps: int = 1) -> bool:
        self.total_checks += 1
        if self._initial:
            self._initial = False
            self._last_time = time.monotonic()
            return True
        self._steps += steps
        fire = False
        if self.frequency_steps is not None and self._steps >= self.frequency_steps:
            fire = True
        if self.frequency_seconds is not None and time.monotonic() - self._last_time >= self.frequency_seconds:
            fire = True
        if fire:
            self._steps = 0
            self._last_time = time.monotonic()
        return fire

    def state_dict(self):
        return dict(steps=self._steps, elapsed=time.monotonic() - self._last_time, total_checks=self.total_checks)

    def load_state_dict(self, sd):
        self._steps = sd["steps"]
        self._last_time = time.monotonic() - sd.get("elapsed", 0.0)
        self.total_checks = sd.get("total_checks", 0)


class EpochStepTimeFreqCtl:
    def __init__(self, freq_epoch: Optional[int] = None, freq_step: Optional[int] = None, freq_sec: Optional[float] = None):
        self.epoch_ctl = FrequencyControl(frequency_steps=freq_epoch)
        self.step_ctl = FrequencyControl(frequency_steps=freq_step)
        self.time_ctl = FrequencyControl(frequency_seconds=freq_sec)
        self.freq_epoch, self.freq_step, self.freq_sec = freq_epoch, freq_step, freq_sec

    def check(self, epochs: int, steps: int) -> bool:
        a = self.epoch_ctl.check(steps=epochs) if self.freq_epoch is not None and epochs > 0 else False
        b = self.step_ctl.check(steps=steps) if self.freq_step is not None else False
        c = self.time_ctl.check() if self.freq_sec is not None else False
        if a or b or c:
            for ctl in (self.epoch_ctl, self.step_ctl, self.time_ctl):
                ctl._steps = 0
                ctl._last_time = time.monotonic()
            return True
        return False

    def state_dict(self):
        return dict(epoch=self.epoch_ctl.state_dict(), step=self.step_ctl.state_dict(), time=self.time_ctl.state_dict())

    def load_state_dict(self, sd):
        self.epoch_ctl.load_state_dict(sd["epoch"])
        self.step_ctl.load_state_dict(sd["step"])
        self.time_ctl.load_state_dict(sd["time"])


class ValueScheduler:
    """constant | linear | exponential | cosine schedules between two values."""

    def __init__(self, kind: str, init_value: float, total_iters: int, end_value: Optional[float] = None):
        self.kind, self.init, self.total = kind, init_value, max(1, total_iters)
        self.end = init_value if end_value is None else end_value

    def get(self, step: int) -> float:
        p = min(1.0, max(0.0, step / self.total))
        if self.kind == "constant":
            return self.init
        if self.kind == "linear":
            return self.init + (self.end - self.init) * p
        if self.kind == "exponential":
            return self.init * (self.end / self.init) ** p if self.init > 0 and self.end > 0 else self.init
        if self.kind == "cosine":
            return self.end + (self.init - self.end) * 0.5 * (1 + math.cos(math.pi * p))
        raise ValueError(f"unknown scheduler {self.kind}")


class ChainedValueScheduler:
    """Several schedules one after another: each runs for its own ``total`` steps from where the previous one ended in
    time (values need not be continuous). Reference: ``areal/utils/timeutil.py`` (``ChainedScheduler``)."""

    def __init__(self, schedulers: list[ValueScheduler]):
        if not schedulers:
            raise ValueError("a chained schedule needs at least one part")
        self.parts = list(schedulers)

    @property
    def total_iters(self) -> int:
        return sum(p.total for p in self.parts)

    @property
    def init_value(self) -> float:
        return self.parts[0].init

    @property
    def final_value(self) -> float:
        return self.parts[-1].get(self.parts[-1].total)

    def get(self, step: int) -> float:
        if step < 0:
            raise ValueError("step must be non-negative")
        for p in self.parts:
            if step < p.total:
                return p.get(step)
            step -= p.total
        return self.final_value
