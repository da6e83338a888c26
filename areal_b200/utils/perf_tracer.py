"""Per-rank performance tracing in Chrome-trace format plus per-rollout-session lifecycle
records.

``trace_scope`` / ``atrace_scope`` / ``instant`` / ``trace_perf`` emit complete ("X") events
into ``perf_tracer/traces-r{rank}.jsonl``; with a CUDA device each scope can also be timed
on the device with CUDA events (``device=True``), which is how multi-GPU numbers are taken
(max over ranks). ``SessionTracer`` records submit -> generate -> reward -> accepted/rejected
per rollout session into ``sessions.jsonl``. Reference: ``areal/utils/perf_tracer.py``
(PerfTracer :1272, SessionTracer :923, trace_perf :1924, categories :63).
"""
from __future__ import annotations

import asyncio
import functools
import getpass
import json
import os
import threading
import time
from contextlib import asynccontextmanager, contextmanager
from typing import Any, Optional

CATEGORIES = ("compute", "comm", "io", "scheduler", "instr", "misc")


class PerfTracer:
    def __init__(self, config=None, rank: int = 0, role: str = "worker"):
        self.config, self.rank, self.role = config, rank, role
        self.enabled = bool(config is not None and getattr(config, "enabled", False))
        ranks = os.environ.get("AREAL_PERF_TRACER_RANKS")
        if ranks and str(rank) not in ranks.split(","):
            self.enabled = False
        self._events: list[dict] = []
        self._lock = threading.Lock()
        self._t0 = time.perf_counter()
        self._device_events: list[tuple] = []
        self.session_tracer = SessionTracer(config, rank) if self.enabled and getattr(config, "session_tracer", None) and \
            config.session_tracer.enabled else None
        self._save_interval = max(1, getattr(config, "save_interval", 1)) if config is not None else 1

    def _out_dir(self) -> str:
        c = self.config
        return os.path.join(c.fileroot or "/tmp/areal", "logs", getpass.getuser(), c.experiment_name or "exp",
                            c.trial_name or "trial", "perf_tracer")

    def _now_us(self) -> float:
        return (time.perf_counter() - self._t0) * 1e6

    def add_complete(self, name: str, cat: str, ts_us: float, dur_us: float, args: Optional[dict] = None):
        if not self.enabled:
            return
        ev = dict(name=name, cat=cat, ph="X", ts=ts_us, dur=dur_us, pid=self.rank, tid=threading.get_ident() % 100000,
                  args=args or {})
        with self._lock:
            self._events.append(ev)

    def instant(self, name: str, category: str = "misc", args: Optional[dict] = None):
        if not self.enabled:
            return
        ev = dict(name=name, cat=category, ph="i", ts=self._now_us(), pid=self.rank, tid=threading.get_ident() % 100000,
                  s="t", args=args or {})
        with self._lock:
            self._events.append(ev)

    @contextmanager
    def trace_scope(self, name: str, category: str = "compute", args: Optional[dict] = None, device: bool = False):
        if not self.enabled:
            yield
            return
        start = self._now_us()
        ev0 = ev1 = None
        if device:
            try:
                import torch

                if torch.cuda.is_available():
                    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    ev0.record()
            except Exception:
                ev0 = ev1 = None
        try:
            yield
        finally:
            if ev0 is not None:
                ev1.record()
                self._device_events.append((name, category, start, ev0, ev1, args))
            self.add_complete(name, category, start, self._now_us() - start, args)

    @asynccontextmanager
    async def atrace_scope(self, name: str, category: str = "compute", args: Optional[dict] = None):
        start = self._now_us()
        try:
            yield
        finally:
            self.add_complete(name, category, start, self._now_us() - start, args)

    def _flush_device_events(self):
        if not self._device_events:
            return
        import torch

        torch.cuda.synchronize()
        for name, cat, start, e0, e1, args in self._device_events:
            self.add_complete(name + "[device]", cat, start, e0.elapsed_time(e1) * 1e3, args)
        self._device_events.clear()

    def save(self, step: Optional[int] = None, force: bool = False):
        if not self.enabled:
            return
        if not force and step is not None and (step + 1) % self._save_interval != 0:
            return
        self._flush_device_events()
        d = self._out_dir()
        os.makedirs(d, exist_ok=True)
        with self._lock:
            evs, self._events = self._events, []
        with open(os.path.join(d, f"traces-r{self.rank}.jsonl"), "a") as f:
            for e in evs:
                f.write(json.dumps(e) + "\n")
        if self.session_tracer is not None:
            self.session_tracer.flush(d)


class SessionTracer:
    """Lifecycle of rollout sessions: phases with wall-clock stamps and a final status."""

    def __init__(self, config=None, rank: int = 0):
        self.rank = rank
        self._sessions: dict[Any, dict] = {}
        self._done: list[dict] = []
        self._lock = threading.Lock()
        self._next = 0

    def register(self, task_id=None) -> int:
        with self._lock:
            self._next += 1
            sid = self._next
            self._sessions[sid] = dict(session_id=sid, task_id=task_id, rank=self.rank, submit_ts=time.time(), phases=[])
            return sid

    def phase(self, sid: int, name: str, start: float, end: float):
        with self._lock:
            s = self._sessions.get(sid)
            if s is not None:
                s["phases"].append(dict(name=name, start=start, end=end))

    def finish(self, sid: int, status: str):
        with self._lock:
            s = self._sessions.pop(sid, None)
            if s is not None:
                s["status"], s["end_ts"] = status, time.time()
                self._done.append(s)

    def flush(self, out_dir: str):
        with self._lock:
            done, self._done = self._done, []
        if done:
            with open(os.path.join(out_dir, "sessions.jsonl"), "a") as f:
                for s in done:
                    f.write(json.dumps(s) + "\n")


_GLOBAL = PerfTracer()


def configure(config, rank: int = 0, role: str = "worker") -> PerfTracer:
    global _GLOBAL
    _GLOBAL = PerfTracer(config, rank, role)
    return _GLOBAL


def get_tracer() -> PerfTracer:
    return _GLOBAL


def trace_scope(name: str, category: str = "compute", args: Optional[dict] = None, device: bool = False):
    return _GLOBAL.trace_scope(name, category, args, device)


def atrace_scope(name: str, category: str = "compute", args: Optional[dict] = None):
    return _GLOBAL.atrace_scope(name, category, args)


def instant(name: str, category: str = "misc", args: Optional[dict] = None):
    _GLOBAL.instant(name, category, args)


def save(step: Optional[int] = None, force: bool = False):
    _GLOBAL.save(step, force)


def trace_perf(name: Optional[str] = None, category: str = "compute"):
    """Decorator: traces every call of a (sync or async) function."""
    def deco(fn):
        label = name or fn.__qualname__
        if asyncio.iscoroutinefunction(fn):
            @functools.wraps(fn)
            async def aw(*a, **k):
                async with atrace_scope(label, category):
                    return await fn(*a, **k)
            return aw

        @functools.wraps(fn)
        def w(*a, **k):
            with trace_scope(label, category):
                return fn(*a, **k)
        return w
    return deco


@asynccontextmanager
async def atrace_session_phase(sid: Optional[int], phase: str):
    st = _GLOBAL.session_tracer
    t0 = time.time()
    try:
        yield
    finally:
        if st is not None and sid is not None:
            st.phase(sid, phase, t0, time.time())
