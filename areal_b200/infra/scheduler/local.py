"""Local scheduler: RPC worker subprocesses on this host with GPU assignment, port
allocation, health polling, engine calls with retries, forked (colocated) roles and ordered
teardown. Reference: ``areal/infra/scheduler/local.py`` and the ``Scheduler`` contract
(``areal/api/scheduler_api.py:43-329``)."""
from __future__ import annotations

import asyncio
import json
import os
import signal
import subprocess
import sys
import time
import urllib.error
import urllib.request
from dataclasses import dataclass, field
from typing import Any, Optional

from ...api.scheduler_api import Job, Scheduler, Worker
from ...utils import logging as alog
from ...utils.network import find_free_ports
from ..rpc.serialization import deserialize_value, serialize_value
from .exceptions import (EngineCallError, EngineCreationError, GPUAllocationError, RPCConnectionError, WorkerCreationError,
                         WorkerFailedError, WorkerNotFoundError, WorkerTimeoutError)

logger = alog.getLogger("local_scheduler")


@dataclass
class _WorkerInfo:
    worker: Worker
    role: str
    process: Optional[subprocess.Popen]
    log_path: str
    env: dict = field(default_factory=dict)
    forked_from: Optional[str] = None


def http_json(url: str, payload: Optional[dict] = None, timeout: float = 3600.0, method: Optional[str] = None) -> dict:
    data = json.dumps(serialize_value(payload)).encode() if payload is not None else None
    req = urllib.request.Request(url, data=data, method=method or ("POST" if data is not None else "GET"),
                                 headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return json.loads(r.read() or b"{}")
    except urllib.error.HTTPError as e:
        body = e.read().decode(errors="replace")
        try:
            return {"__http_error__": e.code, **json.loads(body)}
        except json.JSONDecodeError:
            return {"__http_error__": e.code, "error": body}


class LocalScheduler(Scheduler):
    def __init__(self, gpu_devices: Optional[list[int]] = None, log_dir: str = "/tmp/areal/scheduler_logs",
                 startup_timeout: float = 120.0, experiment_name: str = "", trial_name: str = "", n_gpus: Optional[int] = None):
        if gpu_devices is None:
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                gpu_devices = [int(x) for x in vis.split(",") if x.strip() != ""]
            else:
                try:
                    import torch

                    gpu_devices = list(range(torch.cuda.device_count() if n_gpus is None else n_gpus))
                except Exception:
                    gpu_devices = []
        self.gpu_devices = gpu_devices
        self._gpu_cursor = 0
        self.log_dir = log_dir
        self.startup_timeout = startup_timeout
        self._workers: dict[str, list[_WorkerInfo]] = {}
        os.makedirs(log_dir, exist_ok=True)

    # ------------------------------------------------------------------ helpers
    def _alloc_gpus(self, n: int) -> list[int]:
        if n <= 0:
            return []
        if not self.gpu_devices:
            raise GPUAllocationError("no GPU is visible to the local scheduler")
        if n > len(self.gpu_devices):
            raise GPUAllocationError(f"requested {n} GPUs per worker but only {len(self.gpu_devices)} exist")
        out = [self.gpu_devices[(self._gpu_cursor + i) % len(self.gpu_devices)] for i in range(n)]
        self._gpu_cursor = (self._gpu_cursor + n) % len(self.gpu_devices)
        return out

    def _find(self, worker_id: str) -> _WorkerInfo:
        for infos in self._workers.values():
            for wi in infos:
                if wi.worker.id == worker_id:
                    return wi
        raise WorkerNotFoundError(worker_id)

    def _check_alive(self, wi: _WorkerInfo):
        p = wi.process
        if p is not None and p.poll() is not None:
            tail = ""
            try:
                with open(wi.log_path) as f:
                    tail = f.read()[-2000:]
            except OSError:
                pass
            raise WorkerFailedError(wi.worker.id, p.returncode, tail)

    # ------------------------------------------------------------------ Scheduler API
    def create_workers(self, job: Job, *args, **kwargs) -> list[str]:
        role = job.role
        if role in self._workers:
            raise WorkerCreationError(role, "role already exists")
        strat = job.scheduling_strategy
        if strat is not None and strat.type == "colocation" and strat.target:
            return self.fork_workers(role, strat.target)
        spec = job.tasks[0] if job.tasks else None
        infos = []
        for i in range(job.replicas):
            sp = job.tasks[i] if len(job.tasks) == job.replicas else spec
            gpus = self._alloc_gpus(sp.gpu if sp else 0)
            port = find_free_ports(1)[0]
            env = dict(os.environ)
            if gpus:
                env["CUDA_VISIBLE_DEVICES"] = ",".join(map(str, gpus))
            elif sp is not None and sp.gpu == 0:
                env["AREAL_FORCE_CPU"] = env.get("AREAL_FORCE_CPU", "1")
            env.update({k: str(v) for k, v in (sp.env_vars if sp else {}).items()})
            env["PYTHONPATH"] = os.pathsep.join([os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))),
                                                 env.get("PYTHONPATH", "")])
            cmd = (sp.cmd.split() if sp and sp.cmd else [sys.executable, "-m", "areal_b200.infra.rpc.rpc_server"])
            cmd += ["--port", str(port), "--role", role, "--index", str(i)]
            log_path = os.path.join(self.log_dir, f"{role}_{i}.log")
            logf = open(log_path, "w")
            try:
                proc = subprocess.Popen(cmd, env=env, stdout=logf, stderr=subprocess.STDOUT, start_new_session=True)
            except OSError as e:
                raise WorkerCreationError(role, "spawn failed", repr(e))
            w = Worker(id=f"{role}/{i}", ip="127.0.0.1", worker_ports=[str(port)], engine_ports=[], gpu_ids=gpus)
            infos.append(_WorkerInfo(w, role, proc, log_path, env={}))
        self._workers[role] = infos
        return [wi.worker.id for wi in infos]

    def fork_workers(self, role: str, target_role: str, command: Optional[str] = None) -> list[str]:
        """Colocation: the new role lives in the target role's processes (same GPUs)."""
        if target_role not in self._workers:
            raise WorkerNotFoundError(target_role)
        infos = []
        for i, t in enumerate(self._workers[target_role]):
            w = Worker(id=f"{role}/{i}", ip=t.worker.ip, worker_ports=list(t.worker.worker_ports), engine_ports=[],
                       gpu_ids=list(t.worker.gpu_ids))
            infos.append(_WorkerInfo(w, role, None, t.log_path, forked_from=t.worker.id))
        self._workers[role] = infos
        return [wi.worker.id for wi in infos]

    def get_workers(self, role: str, timeout: Optional[float] = None) -> list[Worker]:
        if role not in self._workers:
            raise WorkerNotFoundError(role)
        deadline = time.monotonic() + (timeout or self.startup_timeout)
        for wi in self._workers[role]:
            while True:
                if wi.process is not None:
                    self._check_alive(wi)
                try:
                    r = http_json(f"http://{wi.worker.address}/health", timeout=2.0)
                    if r.get("status") == "ok":
                        break
                except (urllib.error.URLError, ConnectionError, OSError):
                    pass
                if time.monotonic() > deadline:
                    raise WorkerTimeoutError(role, timeout or self.startup_timeout)
                time.sleep(0.1)
        return [wi.worker for wi in self._workers[role]]

    def delete_workers(self, role: Optional[str] = None):
        roles = [role] if role else list(self._workers)
        # forked roles first, then the processes that host them
        roles.sort(key=lambda r: 0 if all(w.process is None for w in self._workers.get(r, [])) else 1)
        for r in roles:
            for wi in self._workers.pop(r, []):
                if wi.process is None:
                    continue
                try:
                    http_json(f"http://{wi.worker.address}/kill", {}, timeout=2.0)
                except Exception:
                    pass
                try:
                    wi.process.wait(timeout=5)
                except subprocess.TimeoutExpired:
                    try:
                        os.killpg(os.getpgid(wi.process.pid), signal.SIGTERM)
                        wi.process.wait(timeout=5)
                    except Exception:
                        try:
                            os.killpg(os.getpgid(wi.process.pid), signal.SIGKILL)
                        except Exception:
                            pass

    def set_worker_env(self, worker_id: str, env: dict[str, str]) -> None:
        wi = self._find(worker_id)
        r = http_json(f"http://{wi.worker.address}/set_env", {"env": env}, timeout=30)
        if "__http_error__" in r:
            raise EngineCallError(worker_id, "set_env", r.get("error", ""))

    def create_engine(self, worker_id: str, engine: str, *args, name: Optional[str] = None, **kwargs) -> Any:
        wi = self._find(worker_id)
        if wi.process is not None:
            self._check_alive(wi)
        r = http_json(f"http://{wi.worker.address}/create_engine",
                      {"name": name or wi.role, "cls": engine, "args": list(args), "kwargs": kwargs}, timeout=600)
        if "__http_error__" in r:
            raise EngineCreationError(worker_id, r.get("error", "") + "\n" + r.get("traceback", ""), r["__http_error__"])
        return True

    def call_engine(self, worker_id: str, method: str, *args, engine_name: Optional[str] = None, retries: int = 1,
                    return_rtensor: bool = False, direct: bool = False, timeout: float = 7200.0, **kwargs) -> Any:
        wi = self._find(worker_id)
        last = ""
        for attempt in range(1, retries + 1):
            if wi.process is not None:
                self._check_alive(wi)
            try:
                r = http_json(f"http://{wi.worker.address}/call",
                              {"name": engine_name or wi.role, "method": method, "args": list(args), "kwargs": kwargs,
                               "return_rtensor": return_rtensor, "direct": direct}, timeout=timeout)
            except (urllib.error.URLError, ConnectionError, OSError) as e:
                last = repr(e)
                time.sleep(min(2.0, 0.2 * attempt))
                continue
            if "__http_error__" in r:
                # the engine raised: not retryable
                raise EngineCallError(worker_id, method, r.get("error", "") + "\n" + r.get("traceback", ""), attempt)
            return deserialize_value(r.get("result"))
        raise RPCConnectionError(f"worker '{worker_id}' unreachable for '{method}': {last}")

    async def async_call_engine(self, worker_id: str, method: str, *args, **kwargs) -> Any:
        loop = asyncio.get_running_loop()
        return await loop.run_in_executor(None, lambda: self.call_engine(worker_id, method, *args, **kwargs))
