"""Scoped, distributed statistics tracker.

Semantics follow the reference's ``areal/utils/stats_tracker.py``: nested ``scope`` names,
boolean ``denominator`` masks, ``stat`` tensors reduced against a denominator as
AVG_MIN_MAX / AVG / SUM / MIN / MAX, ``scalar`` values averaged over records,
``record_timing`` -> ``timeperf/<name>``, and ``export`` that (optionally) all-reduces over a
process group after synchronising the key set. Named trackers via ``get(name)``.
"""
from __future__ import annotations

import enum
import time
from collections import defaultdict
from contextlib import contextmanager
from typing import Optional

import torch
import torch.distributed as dist


class ReduceType(enum.Enum):
    AVG_MIN_MAX = "avg_min_max"
    AVG = "avg"
    SUM = "sum"
    MIN = "min"
    MAX = "max"
    SCALAR = "scalar"


class DistributedStatsTracker:
    def __init__(self, name: str = ""):
        self.name = name
        self._scopes: list[str] = [name] if name else []
        self._denoms: dict[str, list[torch.Tensor]] = defaultdict(list)
        self._stats: dict[str, list[torch.Tensor]] = defaultdict(list)
        self._stat_denom: dict[str, str] = {}
        self._reduce: dict[str, ReduceType] = {}
        self._scalars: dict[str, list[float]] = defaultdict(list)

    # ------------------------------------------------------------------ recording
    def _key(self, k: str) -> str:
        return "/".join(self._scopes + [k])

    @contextmanager
    def scope(self, name: str):
        self._scopes.append(name)
        try:
            yield
        finally:
            self._scopes.pop()

    def denominator(self, **kwargs):
        for k, v in kwargs.items():
            if v.dtype != torch.bool:
                raise ValueError(f"denominator '{k}' must be a bool tensor")
            self._denoms[self._key(k)].append(v.detach().clone())
            self._reduce.setdefault(self._key(k), ReduceType.SUM)

    def stat(self, denominator: str, reduce_type: Optional[ReduceType] = None, **kwargs):
        dk = self._key(denominator)
        if dk not in self._denoms:
            raise ValueError(f"denominator '{denominator}' was not recorded in this scope")
        for k, v in kwargs.items():
            key = self._key(k)
            if v.shape != self._denoms[dk][-1].shape:
                raise ValueError(f"stat '{k}' shape {tuple(v.shape)} != denominator shape")
            self._stats[key].append(v.detach().float().clone())
            self._stat_denom[key] = dk
            self._reduce[key] = reduce_type or ReduceType.AVG_MIN_MAX

    def scalar(self, **kwargs):
        for k, v in kwargs.items():
            self._scalars[self._key(k)].append(float(v))
            self._reduce[self._key(k)] = ReduceType.SCALAR

    @contextmanager
    def record_timing(self, key: str):
        t0 = time.perf_counter()
        try:
            yield
        finally:
            name = "/".join(["timeperf", key])
            self._scalars[name].append(time.perf_counter() - t0)
            self._reduce[name] = ReduceType.SCALAR

    # ------------------------------------------------------------------ export
    def export(self, key: Optional[str] = None, reduce_group=None, reset: bool = True,
               distributed: Optional[bool] = None) -> dict[str, float]:
        """``distributed``: force (True) or forbid (False) the cross-rank reduction; by default
        statistics are reduced over ``reduce_group`` (the default group when None) whenever
        ``torch.distributed`` is initialised with more than one rank."""
        out: dict[str, float] = {}
        use_dist = dist.is_initialized() and (reduce_group is not None or dist.get_world_size() > 1)
        if distributed is not None:
            use_dist = bool(distributed) and dist.is_initialized()
        keys = sorted(set(self._denoms) | set(self._stats) | set(self._scalars))
        if use_dist:
            gathered = [None] * dist.get_world_size(reduce_group)
            dist.all_gather_object(gathered, [(k, self._reduce[k].value, self._stat_denom.get(k)) for k in keys],
                                   group=reduce_group)
            merged = {}
            for lst in gathered:
                for k, rt, dk in lst:
                    merged[k] = (rt, dk)
            keys = sorted(merged)
            for k, (rt, dk) in merged.items():
                self._reduce.setdefault(k, ReduceType(rt))
                if dk is not None:
                    self._stat_denom.setdefault(k, dk)
        for k in keys:
            if key is not None and not k.startswith(key):
                continue
            rt = self._reduce[k]
            if rt == ReduceType.SCALAR:
                vals = self._scalars.get(k, [])
                s, n = float(sum(vals)), float(len(vals))
                if use_dist:
                    t = torch.tensor([s, n], dtype=torch.float64)
                    t = self._all_reduce(t, dist.ReduceOp.SUM, reduce_group)
                    s, n = t.tolist()
                if n > 0:
                    out[k] = s / n
            elif k in self._denoms or (k not in self._stats and k not in self._stat_denom):
                tot = float(sum(int(d.sum()) for d in self._denoms.get(k, [])))
                if use_dist:
                    tot = float(self._all_reduce(torch.tensor([tot], dtype=torch.float64), dist.ReduceOp.SUM,
                                                 reduce_group)[0])
                out[k] = tot
            else:
                self._export_stat(k, rt, out, use_dist, reduce_group)
        if reset:
            self._denoms.clear(); self._stats.clear(); self._scalars.clear()
            self._stat_denom.clear(); self._reduce.clear()
        return out

    def _export_stat(self, k, rt, out, use_dist, group):
        dk = self._stat_denom.get(k)
        xs = self._stats.get(k, [])
        ds = self._denoms.get(dk, []) if dk else []
        s = n = 0.0
        mn, mx = float("inf"), float("-inf")
        for x, d in zip(xs, ds):
            d = d.to(x.device)
            if d.any():
                sel = x[d]
                s += float(sel.sum())
                n += float(d.sum())
                mn = min(mn, float(sel.min()))
                mx = max(mx, float(sel.max()))
        if use_dist:
            t = self._all_reduce(torch.tensor([s, n], dtype=torch.float64), dist.ReduceOp.SUM, group)
            s, n = t.tolist()
            mn = float(self._all_reduce(torch.tensor([mn], dtype=torch.float64), dist.ReduceOp.MIN, group)[0])
            mx = float(self._all_reduce(torch.tensor([mx], dtype=torch.float64), dist.ReduceOp.MAX, group)[0])
        if n == 0:
            return
        if rt == ReduceType.AVG_MIN_MAX:
            out[f"{k}/avg"], out[f"{k}/min"], out[f"{k}/max"] = s / n, mn, mx
        elif rt == ReduceType.AVG:
            out[k] = s / n
        elif rt == ReduceType.SUM:
            out[k] = s
        elif rt == ReduceType.MIN:
            out[k] = mn
        elif rt == ReduceType.MAX:
            out[k] = mx

    @staticmethod
    def _all_reduce(t, op, group):
        backend = dist.get_backend(group)
        if backend == "nccl" and torch.cuda.is_available():
            t = t.cuda()
        dist.all_reduce(t, op=op, group=group)
        return t.cpu()


DEFAULT_TRACKER = DistributedStatsTracker()
_TRACKERS: dict[str, DistributedStatsTracker] = {}

scope = DEFAULT_TRACKER.scope
denominator = DEFAULT_TRACKER.denominator
stat = DEFAULT_TRACKER.stat
scalar = DEFAULT_TRACKER.scalar
record_timing = DEFAULT_TRACKER.record_timing
export = DEFAULT_TRACKER.export


def get(name: str = "") -> DistributedStatsTracker:
    if not name:
        return DEFAULT_TRACKER
    if name not in _TRACKERS:
        _TRACKERS[name] = DistributedStatsTracker(name)
    return _TRACKERS[name]


def export_all(reduce_group=None, reset: bool = True, distributed: Optional[bool] = None) -> dict[str, float]:
    out = DEFAULT_TRACKER.export(reduce_group=reduce_group, reset=reset, distributed=distributed)
    for name in sorted(_TRACKERS):
        out.update(_TRACKERS[name].export(reduce_group=reduce_group, reset=reset, distributed=distributed))
    return out
