"""Streaming rollout executor: staleness-gated admission of workflow episodes, asynchronous
execution, ordered collection of finished trajectories into training batches.

Semantics follow the reference's ``areal/infra/workflow_executor.py`` (BatchTaskDispatcher
:284-770: producer admits tasks only while ``not paused and capacity > 0``; ``wait`` drains
all finished results, orders them by creation time (task id in deterministic mode), returns
the first ``count`` shuffled and keeps the rest; ``pause/resume`` gate admission only.
WorkflowExecutor :772-1492: workflow resolution, accept filter, trajectory format check,
``submit`` :1277, ``wait`` :1307, ``rollout_batch`` :1358, ``prepare_batch`` :1393).
"""
from __future__ import annotations

import collections
import inspect
import json
import os
import random
import threading
import time
from typing import Any, Callable, Optional

import torch

from ..api.cli_args import InferenceEngineConfig
from ..api.workflow_api import AgentWorkflow, RolloutWorkflow
from ..utils import data as D
from ..utils import logging as alog
from ..utils.dynamic_import import import_from_string
from .staleness import StalenessManager
from .task_runner import AsyncTaskRunner, TaskQueueFullError, TaskResult

logger = alog.getLogger("rollout_executor")

ROLLOUT_POLL_S = 0.05
# ``wait`` / ``wait_for_task`` without a timeout still end: a week, like the reference's
# ``_DEFAULT_WAIT_TIMEOUT_SECONDS`` (areal/infra/workflow_executor.py:252)
DEFAULT_WAIT_TIMEOUT_S = float(7 * 24 * 3600)
REQUIRED_KEYS = ("input_ids", "attention_mask")


def check_trajectory_format(traj: Any, expected_keys: Optional[set] = None) -> bool:
    """Validates a trajectory: dict of tensors with a shared ``[n, L]`` leading shape,
    ``input_ids`` and ``attention_mask`` present. Raises ``ValueError`` on mismatch."""
    if traj is None:
        return True
    if not isinstance(traj, dict):
        raise ValueError(f"trajectory must be a dict or None, got {type(traj).__name__}")
    for k in REQUIRED_KEYS:
        if k not in traj:
            raise ValueError(f"trajectory lacks required key '{k}'")
    ids = traj["input_ids"]
    if not torch.is_tensor(ids) or ids.dim() != 2:
        raise ValueError("input_ids must be a 2-D tensor [n, L]")
    n, L = ids.shape
    for k, v in traj.items():
        if torch.is_tensor(v):
            if v.shape[0] != n:
                raise ValueError(f"'{k}' batch dim {v.shape[0]} != {n}")
            if v.dim() >= 2 and v.shape[1] != L and k not in ("rewards",):
                raise ValueError(f"'{k}' sequence dim {v.shape[1]} != {L}")
    if expected_keys is not None and set(traj.keys()) != expected_keys:
        raise ValueError(f"trajectory keys {sorted(traj)} differ from the first trajectory's {sorted(expected_keys)}")
    return True


class WorkflowExecutor:
    def __init__(self, config: InferenceEngineConfig, inference_engine, staleness_manager: Optional[StalenessManager] = None,
                 dp_world_size: int = 1):
        self.config = config
        self.engine = inference_engine
        self.dp_world_size = max(1, dp_world_size)
        mc = config.max_concurrent_rollouts or config.consumer_batch_size
        self.max_concurrent = max(1, mc // self.dp_world_size)
        self.consumer_bs = max(1, config.consumer_batch_size // self.dp_world_size)
        qsize = config.queue_size or self.max_concurrent * 16
        self.staleness = staleness_manager or StalenessManager(inference_engine, self.max_concurrent, self.consumer_bs,
                                                               config.max_head_offpolicyness)
        self.runner = AsyncTaskRunner(max_queue_size=qsize)
        self._pending: collections.deque = collections.deque()
        self._pending_lock = threading.Lock()
        self._results: list[TaskResult] = []
        self._results_lock = threading.Lock()
        self._task_results: dict[int, Any] = {}    # only for task ids somebody asked to wait on (``_tracked``)
        self._tracked: set[int] = set()
        self._start_version: dict[int, int] = {}    # task id -> weight version when the episode started (running episodes only)
        self._paused = threading.Event()
        self._stop = threading.Event()
        self._threads: list[threading.Thread] = []
        self._exc: Optional[BaseException] = None
        self._expected_keys: Optional[set] = None
        self._data_gen = None
        self._dump_fh = None
        self.queue_size = qsize
        self.rejected_count = 0

    # ------------------------------------------------------------------ lifecycle
    def initialize(self):
        self.runner.initialize()
        for fn, name in ((self._commit_loop, "rollout-commit"), (self._fetch_loop, "rollout-fetch")):
            t = threading.Thread(target=self._guard(fn), name=name, daemon=True)
            t.start()
            self._threads.append(t)
        return self

    def destroy(self):
        self._stop.set()
        for t in self._threads:
            t.join(timeout=5)
        self._threads.clear()
        self.runner.destroy()
        if self._dump_fh:
            self._dump_fh.close()

    def _guard(self, fn):
        def run():
            try:
                fn()
            except BaseException as e:  # fail fast: surfaced by the next public call
                logger.error("rollout thread failed: %r", e)
                self._exc = e
        return run

    def _check(self):
        if self._exc is not None:
            root = self._exc
            while root.__cause__ is not None:
                root = root.__cause__
            raise RuntimeError(f"rollout executor thread failed: {root!r}") from self._exc
        self.runner.check_health()

    # ------------------------------------------------------------------ producer / consumer
    def _commit_loop(self):
        while not self._stop.is_set():
            moved = False
            if not self._paused.is_set():
                while self.staleness.get_capacity() > 0:
                    with self._pending_lock:
                        if not self._pending:
                            break
                        tid, factory = self._pending.popleft()
                    try:
                        self.runner.submit(factory, task_id=tid)
                    except TaskQueueFullError:
                        with self._pending_lock:
                            self._pending.appendleft((tid, factory))
                        break
                    self.staleness.on_rollout_submitted()
                    moved = True
            if not moved:
                time.sleep(0.002)

    def _fetch_loop(self):
        while not self._stop.is_set():
            r = self.runner.poll(timeout=ROLLOUT_POLL_S)
            if r is None:
                continue
            self._start_version.pop(r.task_id, None)
            if r.error is not None:
                self.staleness.on_rollout_rejected()
                raise RuntimeError(f"workflow episode {r.task_id} failed") from r.error
            traj, accepted = r.data
            if accepted:
                self.staleness.on_rollout_accepted()
                self._trace("finish and accept rollout", r.task_id)
                with self._results_lock:
                    if r.task_id in self._tracked:      # handed out by ``wait_for_task`` only, never by ``wait``
                        self._task_results[r.task_id] = traj
                    else:
                        self._results.append(TaskResult(r.task_id, traj, r.create_time))
            else:
                self.staleness.on_rollout_rejected()
                self.rejected_count += 1
                self._trace("finish but reject rollout", r.task_id)
                with self._results_lock:
                    if r.task_id in self._tracked:
                        self._task_results[r.task_id] = None

    def _trace(self, what: str, task_id=None) -> None:
        """``rollout.enable_rollout_tracing``: one log line per life-cycle event with the admission counters
        (reference: ``areal/infra/workflow_executor.py:1239-1322``)."""
        if getattr(self.config, "enable_rollout_tracing", False):
            st = self.staleness.get_stats()
            logger.info("%s (task %s): enqueued %d, running %d, accepted %d, rejected %d, engine version %d", what, task_id,
                        st.enqueued, st.running, st.accepted, st.rejected, self.engine.get_version())

    # ------------------------------------------------------------------ workflow resolution
    def _resolve_workflow(self, workflow, workflow_kwargs) -> RolloutWorkflow:
        kw = workflow_kwargs or {}
        if isinstance(workflow, str):
            workflow = import_from_string(workflow)
        if inspect.isclass(workflow):
            workflow = workflow(**kw)
        if isinstance(workflow, RolloutWorkflow):
            return workflow
        if isinstance(workflow, AgentWorkflow) or hasattr(workflow, "run"):
            from .workflows.agent import AgentRolloutAdapter

            return AgentRolloutAdapter(workflow, self.config)
        raise TypeError(f"cannot use {workflow!r} as a rollout workflow")

    def _make_task(self, data, workflow: RolloutWorkflow, should_accept_fn, is_eval: bool, task_id: int):
        async def run():
            from . import workflow_context as wctx

            self._start_version[task_id] = self.engine.get_version()
            with wctx.scoped(is_eval=is_eval, task_id=task_id):
                traj = await workflow.arun_episode(self.engine, data)
            if traj is None:
                return None, False
            if self.config.check_trajectory_format:
                check_trajectory_format(traj, self._expected_keys)
                if self._expected_keys is None and isinstance(traj, dict):
                    self._expected_keys = set(traj.keys())
            ok = True if should_accept_fn is None else bool(should_accept_fn(traj))
            if ok and self.config.dump_to_file:
                self._dump(traj, task_id, is_eval)
            return traj, ok
        return run

    def _dump(self, traj, task_id, is_eval: bool = False):
        """One readable line per sample (see ``rollout/dump.py``); a failure here never fails the episode."""
        from . import dump as D

        try:
            root = D.dump_dir(self.config, is_eval) or os.path.join("/tmp/areal", "eval-rollout" if is_eval else "rollout")
            if getattr(self, "_dump_tokenizer", None) is None and getattr(self.config, "tokenizer_path", ""):
                from transformers import AutoTokenizer

                self._dump_tokenizer = AutoTokenizer.from_pretrained(self.config.tokenizer_path)
            D.dump_trajectory(traj, task_id, root, getattr(self, "_dump_tokenizer", None), self.engine.get_version())
        except Exception as e:  # noqa: BLE001
            logger.warning("trajectory of task %s not dumped: %s", task_id, e)

    # ------------------------------------------------------------------ public API
    def submit(self, data: dict[str, Any], workflow=None, workflow_kwargs=None, should_accept_fn=None,
               task_id: Optional[int] = None, is_eval: bool = False, track: bool = False) -> int:
        """Queues one episode. ``track=True`` keeps the episode's outcome (a trajectory, or ``None``
        when it was rejected) for ``wait_for_task`` instead of the shared result pool of ``wait``."""
        self._check()
        wf = self._resolve_workflow(workflow, workflow_kwargs)
        if isinstance(should_accept_fn, str):
            should_accept_fn = import_from_string(should_accept_fn)
        tid = task_id if task_id is not None else self.runner.new_task_id()
        if track:
            with self._results_lock:
                self._tracked.add(tid)
        with self._pending_lock:
            if len(self._pending) >= self.queue_size:
                raise TaskQueueFullError("pending rollout queue is full")
            self._pending.append((tid, self._make_task(data, wf, should_accept_fn, is_eval, tid)))
        self.staleness.on_rollout_enqueued()
        return tid

    def wait(self, count: int, timeout: Optional[float] = None, raise_timeout: bool = True) -> list:
        """Blocks until ``count`` accepted trajectories exist; returns them (oldest first,
        shuffled unless deterministic) and keeps the surplus for the next call."""
        deadline = time.monotonic() + (DEFAULT_WAIT_TIMEOUT_S if timeout is None else timeout)
        while True:
            self._check()
            with self._results_lock:
                if len(self._results) >= count:
                    key = (lambda r: r.task_id) if self.config.deterministic_sampling else (lambda r: r.create_time)
                    self._results.sort(key=key)
                    take, self._results = self._results[:count], self._results[count:]
                    break
            if deadline is not None and time.monotonic() > deadline:
                if raise_timeout:
                    raise TimeoutError(f"timed out waiting for {count} rollouts")
                return []
            time.sleep(0.005)
        if not self.config.deterministic_sampling:
            random.shuffle(take)
        self._trace(f"{count} rollout results are ready")
        return [r.data for r in take]

    def wait_for_task(self, task_id: int, timeout: Optional[float] = None, raise_timeout: bool = True):
        """Outcome of one episode: its trajectory, or ``None`` if it was rejected. An id that was not
        submitted with ``track=True`` is looked for in the shared pool (accepted episodes only)."""
        deadline = time.monotonic() + (DEFAULT_WAIT_TIMEOUT_S if timeout is None else timeout)
        while True:
            self._check()
            with self._results_lock:
                if task_id in self._task_results:
                    self._tracked.discard(task_id)
                    return self._task_results.pop(task_id)
                if task_id not in self._tracked:
                    hit = [r for r in self._results if r.task_id == task_id]
                    if hit:
                        self._results = [r for r in self._results if r.task_id != task_id]
                        return hit[0].data
            if deadline is not None and time.monotonic() > deadline:
                if raise_timeout:
                    raise TimeoutError(f"timed out waiting for task {task_id}")
                return None
            time.sleep(0.005)

    def rollout_batch(self, data: list[dict[str, Any]], workflow=None, workflow_kwargs=None, should_accept_fn=None
                      ) -> dict[str, Any]:
        """Synchronous helper: runs one episode per item and returns the accepted ones, concatenated.
        Rejected episodes and episodes that returned ``None`` count as finished (reference:
        areal/infra/workflow_executor.py:1358-1391 waits on completions and filters afterwards)."""
        tids = [self.submit(item, workflow, workflow_kwargs, should_accept_fn, track=True) for item in data]
        trajs = [self.wait_for_task(t) for t in tids]
        trajs = [t for t in trajs if t]
        if not trajs:
            raise RuntimeError("every episode of the batch was rejected or returned no trajectory")
        return D.concat_padded_tensors(trajs)

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None,
                      dynamic_bs: bool = False) -> dict[str, Any]:
        """Keeps the pipeline fed from ``dataloader`` and returns one training batch of
        ``dataloader.batch_size`` accepted trajectories (``dynamic_bs``: returns once accepted
        plus rejected reaches the batch size)."""
        if self._data_gen is None:
            self._data_gen = D.cycle_dataloader(dataloader)
        bs = getattr(dataloader, "batch_size", None) or self.consumer_bs
        bs = max(1, bs // self.dp_world_size) if self.dp_world_size > 1 else bs
        rej0 = self.rejected_count
        while True:
            self._check()
            with self._pending_lock:
                npending = len(self._pending)
            room = min(self.staleness.get_pending_limit() - npending,
                       self.queue_size - (self.runner.input_queue_size() + npending + bs))
            fed = 0
            while fed < room:
                items = next(self._data_gen)
                items = items if isinstance(items, list) else [items]
                for it in items:
                    self.submit(it, workflow, workflow_kwargs, should_accept_fn)
                    fed += 1
            with self._results_lock:
                have = len(self._results)
            if self._stragglers_due():
                time.sleep(0.002)           # strict bound: the oldest running episodes must make this batch
                continue
            if have >= bs or (dynamic_bs and have + (self.rejected_count - rej0) >= bs and have > 0):
                n = min(have, bs)
                return D.concat_padded_tensors(self.wait(n, timeout=1.0))
            time.sleep(0.01)

    def _stragglers_due(self) -> bool:
        """Strict staleness only: is an episode still running that started ``max_head_offpolicyness``
        or more versions ago? It has to be part of the batch about to be formed (the batch after it
        would train it one version too late), so the batch waits for it."""
        if not getattr(self.config, "strict_staleness", False):
            return False
        limit = self.engine.get_version() - self.config.max_head_offpolicyness
        return any(v <= limit for v in list(self._start_version.values()))

    def pause(self):
        """Stops admitting new episodes; running ones continue."""
        self._paused.set()

    def resume(self):
        self._paused.clear()

    def is_paused(self) -> bool:
        return self._paused.is_set()

    def get_capacity(self) -> int:
        return self.staleness.get_capacity()
