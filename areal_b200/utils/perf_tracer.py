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
        self.session_tracer = None
        if self.enabled and getattr(config, "session_tracer", None) and config.session_tracer.enabled:
            d = self._out_dir()
            os.makedirs(d, exist_ok=True)
            self.session_tracer = SessionTracer(config.session_tracer, rank, out_dir=d)
        self._save_interval = max(1, getattr(config, "save_interval", 1)) if config is not None else 1
        self.profile_steps = self._normalize_profile_steps(getattr(config, "profile_steps", None) if config is not None else None)
        self.current_step: Optional[int] = None
        self._virtual_tids: dict = {}
        self._profiling = False

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

    # ------------------------------------------------------------------ kernel-level traces
    @staticmethod
    def _normalize_profile_steps(steps) -> frozenset:
        out = set()
        for raw in steps or ():
            try:
                out.add(int(raw))
            except (TypeError, ValueError):
                continue
        return frozenset(out)

    def set_step(self, step: Optional[int]) -> None:
        """The trainer's current global step: scopes opened with ``profile=True`` run under the
        PyTorch profiler when this step is listed in ``profile_steps``."""
        self.current_step = step

    def should_profile(self, requested: bool = True) -> bool:
        return bool(self.enabled and requested and self.profile_steps and self.current_step is not None
                    and self.current_step in self.profile_steps and not self._profiling)

    @contextmanager
    def profile_scope(self, name: str, category: str = "compute"):
        """``trace_scope`` that additionally records every CPU op and GPU kernel inside it with
        ``torch.profiler`` on the steps listed in ``profile_steps`` and merges those events into
        this rank's trace (reference: areal/utils/perf_tracer.py:1454 merge_profiler_trace)."""
        if not self.should_profile():
            with self.trace_scope(name, category):
                yield
            return
        import tempfile

        import torch
        from torch.profiler import ProfilerActivity, profile

        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        self._profiling = True
        base_us = self._now_us()
        try:
            with profile(activities=acts) as prof, self.trace_scope(name, category, args={"profiled": True}):
                yield
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            with tempfile.NamedTemporaryFile(suffix=".json", delete=False) as f:
                path = f.name
            try:
                prof.export_chrome_trace(path)
                with open(path) as fh:
                    self.merge_profiler_trace(json.load(fh), base_us)
            finally:
                try:
                    os.unlink(path)
                except OSError:
                    pass
        finally:
            self._profiling = False

    def merge_profiler_trace(self, profiler_trace: dict, base_us: float) -> int:
        """Merges a PyTorch-profiler Chrome trace (the loaded JSON) into this rank's event stream:
        timestamps are shifted so the earliest profiler event lands at ``base_us`` on this tracer's
        clock, every event is attributed to this rank's process id, and each (profiler pid, tid)
        pair (CPU threads, ``GPU d stream s`` lanes) gets its own virtual, negative thread id with a
        ``thread_name`` record, so kernels show up as extra lanes under the rank's own scopes.
        Returns the number of events merged."""
        if not self.enabled:
            return 0
        events = profiler_trace.get("traceEvents") or []
        stamps = [e["ts"] for e in events if "ts" in e and e.get("ph") != "M"]
        if not stamps:
            return 0
        shift = base_us - min(stamps)
        names = {}
        for e in events:
            if e.get("ph") == "M" and e.get("name") == "thread_name":
                names[(str(e.get("pid")), str(e.get("tid")))] = (e.get("args") or {}).get("name")
        ignored_meta = {"process_name", "process_sort_index", "process_labels", "thread_name", "thread_sort_index"}
        ignored_pids = {"Spans", "Traces", ""}
        merged = []
        for e in events:
            if e.get("ph") == "M" and e.get("name") in ignored_meta:
                continue
            if str(e.get("pid")) in ignored_pids or "ts" not in e:
                continue
            key = (str(e.get("pid")), str(e.get("tid")))
            vt = self._virtual_tids.get(key)
            if vt is None:
                vt = self._virtual_tids[key] = -(len(self._virtual_tids) + 1)
                label = names.get(key) or (f"GPU {e.get('pid')} stream {e.get('tid')}" if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset")
                                           else f"profiler thread {e.get('tid')}")
                merged.append(dict(name="thread_name", ph="M", pid=self.rank, tid=vt, args={"name": label}))
            ev = dict(e)
            ev["ts"] = e["ts"] + shift
            ev["pid"], ev["tid"] = self.rank, vt
            merged.append(ev)
        with self._lock:
            self._events.extend(merged)
        return sum(1 for m in merged if m.get("ph") != "M")

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

    def __init__(self, config=None, rank: int = 0, out_dir: Optional[str] = None):
        self.rank = rank
        # finished sessions are written out once this many are waiting (``session_tracer.flush_threshold``), not only at
        # the periodic save: a long run keeps a bounded list in memory
        self.flush_threshold = max(1, int(getattr(config, "flush_threshold", 256) or 256))
        self.out_dir = out_dir
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
            pending = len(self._done)
        if self.out_dir is not None and pending >= self.flush_threshold:
            self.flush(self.out_dir)

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


def set_step(step: Optional[int]) -> None:
    get_tracer().set_step(step)


def profile_scope(name: str, category: str = "compute"):
    return get_tracer().profile_scope(name, category)


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
