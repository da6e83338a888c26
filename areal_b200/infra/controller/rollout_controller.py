"""Controller-side proxy of a fleet of inference workers.

One worker process per inference replica. Admission control is global and lives here: a
controller-side :class:`WorkflowExecutor` owns the :class:`StalenessManager`; each admitted
episode becomes one ``submit`` + ``wait_for_task`` RPC pair against the least-loaded worker,
whose own executor runs the workflow next to the engine (its local admission is opened wide).
Trainers reach the controller through :class:`RolloutCallback` (pause / resume / version /
weight sync). Reference: ``areal/infra/controller/rollout_controller.py`` (worker creation
:162-233, ``_create_submit_callback`` :851-936, callback server :605-712).
"""
from __future__ import annotations

import asyncio
import concurrent.futures as cf
import copy
import dataclasses
import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Optional

from ...api.cli_args import InferenceEngineConfig, SchedulingSpec, SchedulingStrategy
from ...api.io_struct import WeightUpdateMeta
from ...api.scheduler_api import Job, Scheduler, Worker
from ...api.workflow_api import RolloutWorkflow
from ...rollout.executor import WorkflowExecutor
from ...utils import logging as alog
from ...utils.network import find_free_ports, gethostip
from ..rpc.serialization import deserialize_value, serialize_value

logger = alog.getLogger("rollout_controller")

_WIDE_OPEN = 1 << 20


def _path_of(x) -> Optional[str]:
    if x is None or isinstance(x, str):
        return x
    if isinstance(x, type):
        return f"{x.__module__}.{x.__qualname__}"
    if callable(x) and hasattr(x, "__module__") and hasattr(x, "__qualname__") and "<locals>" not in x.__qualname__:
        return f"{x.__module__}.{x.__qualname__}"
    raise TypeError("single-controller mode ships workflows and predicates by import path; got an instance of "
                    f"{type(x).__name__}. Pass 'pkg.module.Class' (plus workflow_kwargs) instead.")


class _RemoteEpisode(RolloutWorkflow):
    """The controller-side stand-in for a workflow: runs the real one on a worker."""

    def __init__(self, ctl: "RolloutController", workflow: Optional[str], workflow_kwargs: Optional[dict], should_accept: Optional[str]):
        self.ctl, self.workflow, self.kwargs, self.should_accept = ctl, workflow, workflow_kwargs, should_accept

    async def arun_episode(self, engine, data):
        ctl = self.ctl
        idx = ctl._pick_worker()
        w = ctl.workers[idx]
        loop = asyncio.get_running_loop()
        try:
            tid = await loop.run_in_executor(ctl._pool, lambda: ctl.scheduler.call_engine(
                w.id, "submit", data, engine_name=ctl.role, direct=True, workflow=self.workflow, workflow_kwargs=self.kwargs,
                should_accept_fn=self.should_accept))
            return await loop.run_in_executor(ctl._pool, lambda: ctl.scheduler.call_engine(
                w.id, "wait_for_task", tid, engine_name=ctl.role, direct=True, timeout=ctl.config.request_timeout))
        finally:
            ctl._release_worker(idx)


class RolloutController:
    def __init__(self, engine_cls: str, config: InferenceEngineConfig, scheduler: Scheduler, role: str = "rollout"):
        if not isinstance(engine_cls, str):
            engine_cls = f"{engine_cls.__module__}.{engine_cls.__qualname__}"
        self.engine_cls = engine_cls
        self.config = config
        self.scheduler = scheduler
        self.role = role
        self.workers: list[Worker] = []
        self._version = 0
        self._inflight: list[int] = []
        self._lock = threading.Lock()
        self._pool: Optional[cf.ThreadPoolExecutor] = None
        self._executor: Optional[WorkflowExecutor] = None
        self._cb_server = None
        self.callback_addr: Optional[str] = None
        self.proxy_addrs: list[str] = []
        self._gateway = None

    # ------------------------------------------------------------------ lifecycle
    def initialize(self, n_workers: int = 1, gpus_per_worker: int = 0, engine_args: tuple = (), engine_kwargs: Optional[dict] = None,
                   init_kwargs: Optional[dict] = None, train_data_parallel_size: int = 1, colocate_with: Optional[str] = None,
                   start_callback_server: bool = False):
        spec = SchedulingSpec(gpu=gpus_per_worker)
        strat = SchedulingStrategy(type="colocation", target=colocate_with) if colocate_with else SchedulingStrategy()
        self.scheduler.create_workers(Job(replicas=n_workers, tasks=[spec], scheduling_strategy=strat, role=self.role))
        self.workers = self.scheduler.get_workers(self.role)
        self._inflight = [0] * len(self.workers)
        self._pool = cf.ThreadPoolExecutor(max_workers=max(16, (self.config.max_concurrent_rollouts or 64) * 2),
                                           thread_name_prefix="rollout-rpc")
        # workers admit everything; the controller's staleness manager decides
        wcfg = copy.deepcopy(self.config)
        wcfg.max_head_offpolicyness = _WIDE_OPEN
        wcfg.max_concurrent_rollouts = max(self.config.max_concurrent_rollouts or 0, self.config.consumer_batch_size) * 4
        kw = dict(engine_kwargs or {})
        futs = [self._pool.submit(self.scheduler.create_engine, w.id, self.engine_cls, wcfg, *engine_args, name=self.role, **kw)
                for w in self.workers]
        [f.result() for f in futs]
        self._call_all("initialize", **(init_kwargs or {}))
        self._executor = WorkflowExecutor(self.config, self, dp_world_size=1).initialize()
        if start_callback_server:
            self._start_callback_server()
        return self

    # ------------------------------------------------------------------ agent mode
    def start_proxy(self, tokenizer: str, tokenizer_kwargs: Optional[dict] = None, gconfig: Optional[dict] = None,
                    admin_key: Optional[str] = None, chat_template_type: str = "hf") -> list[str]:
        """One OpenAI-compatible proxy beside every rollout worker, over that worker's engine (``tokenizer``: dotted
        path of a callable that returns the tokenizer). Returns their base urls (reference
        ``rollout_controller.py:406-471``)."""
        if self.proxy_addrs:
            return self.proxy_addrs
        if not self.workers:
            raise RuntimeError("initialize() first: the proxies sit beside the rollout workers")
        name = f"{self.role}-proxy"
        futs = [self._pool.submit(self.scheduler.create_engine, w.id, "areal_b200.openai.proxy.HostedProxy", name=name,
                                  engine_name=self.role, tokenizer=tokenizer, tokenizer_kwargs=tokenizer_kwargs, gconfig=gconfig,
                                  admin_key=admin_key, host=w.ip, chat_template_type=chat_template_type) for w in self.workers]
        [f.result() for f in futs]
        futs = [self._pool.submit(self.scheduler.call_engine, w.id, "initialize", engine_name=name, direct=True) for w in self.workers]
        self.proxy_addrs = [f.result() for f in futs]
        self._proxy_admin_key = admin_key
        return self.proxy_addrs

    def get_proxy_addr(self, rank: int) -> str:
        if not self.proxy_addrs:
            raise RuntimeError("start_proxy() first")
        return self.proxy_addrs[rank]

    def start_proxy_gateway(self, host: str = "127.0.0.1", port: Optional[int] = None) -> str:
        """One address for agents outside the job, in front of all proxies (sessions stick to the proxy that
        opened them). Reference ``rollout_controller.py:496-577``."""
        if self._gateway is None:
            from ...openai.proxy_gateway import ProxyGateway

            if not self.proxy_addrs:
                raise RuntimeError("start_proxy() first")
            self._gateway = ProxyGateway(self.proxy_addrs, getattr(self, "_proxy_admin_key", None), host=host, port=port).start()
        return self._gateway.addr

    @property
    def proxy_gateway_addr(self) -> str:
        if self._gateway is None:
            raise RuntimeError("proxy gateway not started")
        return self._gateway.addr

    def destroy(self):
        if self._gateway is not None:
            self._gateway.stop()
            self._gateway = None
        if self.proxy_addrs and self._pool is not None:
            for w in self.workers:
                try:
                    self.scheduler.call_engine(w.id, "destroy", engine_name=f"{self.role}-proxy", direct=True)
                except Exception as e:
                    logger.warning("stopping the proxy on %s failed: %r", w.id, e)
            self.proxy_addrs = []
        if self._executor is not None:
            self._executor.destroy()
            self._executor = None
        if self._cb_server is not None:
            self._cb_server.shutdown()
            self._cb_server = None
        if self._pool is not None:
            try:
                self._call_all("destroy")
            except Exception as e:
                logger.warning("destroy on rollout workers failed: %r", e)
            self.scheduler.delete_workers(self.role)
            self._pool.shutdown(wait=False)
            self._pool = None

    # ------------------------------------------------------------------ plumbing
    def _call_all(self, method: str, *args, **kwargs):
        futs = [self._pool.submit(self.scheduler.call_engine, w.id, method, *args, engine_name=self.role, **kwargs)
                for w in self.workers]
        return [f.result() for f in futs]

    def _pick_worker(self) -> int:
        with self._lock:
            i = min(range(len(self.workers)), key=lambda j: (self._inflight[j], j))
            self._inflight[i] += 1
            return i

    def _release_worker(self, i: int):
        with self._lock:
            self._inflight[i] -= 1

    # ------------------------------------------------------------------ InferenceEngine surface
    def get_version(self) -> int:
        return self._version

    def set_version(self, version: int) -> None:
        self._version = version
        self._call_all("set_version", version, direct=True)

    def submit(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None, task_id=None, is_eval=False) -> int:
        wf = _RemoteEpisode(self, _path_of(workflow), workflow_kwargs, _path_of(should_accept_fn))
        return self._executor.submit(data, wf, None, None, task_id, is_eval)

    def wait(self, count: int, timeout: Optional[float] = None, raise_timeout: bool = True):
        return self._executor.wait(count, timeout, raise_timeout)

    def wait_for_task(self, task_id: int, timeout: Optional[float] = None, raise_timeout: bool = True):
        return self._executor.wait_for_task(task_id, timeout, raise_timeout)

    def rollout_batch(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None):
        wf = _RemoteEpisode(self, _path_of(workflow), workflow_kwargs, _path_of(should_accept_fn))
        return self._executor.rollout_batch(data, wf, None, None)

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None, dynamic_bs: bool = False):
        wf = _RemoteEpisode(self, _path_of(workflow), workflow_kwargs, _path_of(should_accept_fn))
        return self._executor.prepare_batch(dataloader, wf, None, None, dynamic_bs)

    def pause(self):
        self._executor.pause()
        self._call_all("pause", direct=True)

    def resume(self):
        self._call_all("resume", direct=True)
        self._executor.resume()

    def pause_generation(self):
        self._call_all("pause_generation", direct=True)

    def continue_generation(self):
        self._call_all("continue_generation", direct=True)

    def update_weights_from_disk(self, meta: WeightUpdateMeta):
        self._call_all("update_weights_from_disk", meta)
        if meta.version is not None:
            self._version = meta.version

    def update_weights_from_handle(self, handle, meta: Optional[WeightUpdateMeta] = None):
        """``handle``: remote-tensor handle of the trainer's exported parameters; every worker
        pulls it from the trainer worker that holds it."""
        self._call_all("update_weights_from_tensors", handle, meta)
        if meta is not None and meta.version is not None:
            self._version = meta.version

    def export_stats(self) -> dict[str, float]:
        out: dict[str, float] = {}
        per = self._call_all("export_stats", direct=True)
        for d in per:
            for k, v in (d or {}).items():
                out[k] = out.get(k, 0.0) + float(v) / len(per)
        st = self._executor.staleness.get_stats()
        out.update({"rollout/accepted": float(st.accepted), "rollout/running": float(st.running),
                    "rollout/enqueued": float(st.enqueued), "rollout/rejected": float(st.rejected)})
        return out

    @property
    def staleness_manager(self):
        return self._executor.staleness

    # ------------------------------------------------------------------ callback server
    def _start_callback_server(self):
        """Lets engines on other processes (trainer workers) drive this controller:
        ``POST /callback/<method>`` with serialised args."""
        ctl = self
        allowed = {"pause", "resume", "set_version", "get_version", "pause_generation", "continue_generation",
                   "update_weights_from_disk", "update_weights_from_handle", "rollout_batch", "export_stats"}

        class H(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def do_POST(self):
                n = int(self.headers.get("Content-Length", "0"))
                req = deserialize_value(json.loads(self.rfile.read(n))) if n else {}
                name = self.path.rsplit("/", 1)[-1]
                try:
                    if name not in allowed:
                        raise PermissionError(f"callback '{name}' is not exposed")
                    res = getattr(ctl, name)(*req.get("args", []), **req.get("kwargs", {}))
                    body, code = json.dumps({"result": serialize_value(res)}).encode(), 200
                except BaseException as e:
                    body, code = json.dumps({"error": repr(e)}).encode(), 500
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

        port = find_free_ports(1)[0]
        self._cb_server = ThreadingHTTPServer(("0.0.0.0", port), H)
        self._cb_server.daemon_threads = True
        threading.Thread(target=self._cb_server.serve_forever, daemon=True, name="rollout-callback").start()
        self.callback_addr = f"127.0.0.1:{port}" if all(w.ip == "127.0.0.1" for w in self.workers) else f"{gethostip()}:{port}"
        return self.callback_addr
