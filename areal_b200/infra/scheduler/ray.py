"""Ray scheduler: every worker is a Ray actor that runs the RPC worker loop in its own
process with the requested GPUs; placement groups pack or spread roles, colocated roles reuse
the target's actors. ``ray`` is imported lazily (it is optional). Reference:
``areal/infra/scheduler/ray.py``."""
from __future__ import annotations

import time
from typing import Any, Optional

from ...api.scheduler_api import Job, Worker
from ...utils import logging as alog
from .exceptions import WorkerCreationError, WorkerFailedError, WorkerNotFoundError, WorkerTimeoutError
from .local import LocalScheduler, _WorkerInfo

logger = alog.getLogger("ray_scheduler")


def _import_ray():
    try:
        import ray  # type: ignore

        return ray
    except ImportError as e:  # pragma: no cover - depends on the environment
        raise RuntimeError("the Ray scheduler needs the 'ray' package") from e


def _actor_main(host_env: dict):
    """Body of the actor: starts the RPC server on a free port and reports its address."""
    import os
    import threading

    from ...utils.network import find_free_ports, gethostip
    from ..rpc import rpc_server

    os.environ.update({k: str(v) for k, v in host_env.items()})
    ip, port = gethostip(), find_free_ports(1)[0]
    threading.Thread(target=rpc_server.serve, args=(ip, port), daemon=True).start()
    return f"{ip}:{port}"


class RayScheduler(LocalScheduler):
    def __init__(self, startup_timeout: float = 300.0, log_dir: str = "/tmp/areal/ray_scheduler", ray_module=None,
                 placement_strategy: str = "PACK"):
        super().__init__(gpu_devices=[], log_dir=log_dir, startup_timeout=startup_timeout)
        self.ray = ray_module or _import_ray()
        self.placement_strategy = placement_strategy
        self._actors: dict[str, list[Any]] = {}
        self._pgs: dict[str, Any] = {}
        if not self.ray.is_initialized():
            self.ray.init(ignore_reinit_error=True)

    def create_workers(self, job: Job, *args, **kwargs) -> list[str]:
        ray, role = self.ray, job.role
        if role in self._workers:
            raise WorkerCreationError(role, "role already exists")
        if job.scheduling_strategy.type == "colocation" and job.scheduling_strategy.target:
            return self.fork_workers(role, job.scheduling_strategy.target)
        spec = job.tasks[0]
        bundles = [{"CPU": spec.cpu, **({"GPU": spec.gpu} if spec.gpu else {})} for _ in range(job.replicas)]
        try:
            pg = ray.util.placement_group(bundles, strategy=self.placement_strategy)
            ray.get(pg.ready(), timeout=self.startup_timeout)
        except Exception as e:
            raise WorkerCreationError(role, "placement group could not be scheduled", repr(e))
        self._pgs[role] = pg

        @ray.remote
        class _RPCActor:
            def start(self, env):
                return _actor_main(env)

            def ping(self):
                return True

        actors, infos = [], []
        for i in range(job.replicas):
            a = _RPCActor.options(num_cpus=spec.cpu, num_gpus=spec.gpu, placement_group=pg, placement_group_bundle_index=i,
                                  name=f"{role}-{i}-{int(time.time() * 1e3)}").remote()
            actors.append(a)
        try:
            addrs = ray.get([a.start.remote(dict(spec.env_vars)) for a in actors], timeout=self.startup_timeout)
        except Exception as e:
            raise WorkerFailedError(f"{role}/*", "actor start failed", repr(e))
        for i, addr in enumerate(addrs):
            ip, port = addr.rsplit(":", 1)
            infos.append(_WorkerInfo(Worker(id=f"{role}/{i}", ip=ip, worker_ports=[port]), role, None, ""))
        self._actors[role] = actors
        self._workers[role] = infos
        return [wi.worker.id for wi in infos]

    def delete_workers(self, role: Optional[str] = None):
        for r in ([role] if role else list(self._workers)):
            self._workers.pop(r, None)
            for a in self._actors.pop(r, []):
                try:
                    self.ray.kill(a)
                except Exception:
                    pass
            pg = self._pgs.pop(r, None)
            if pg is not None:
                try:
                    self.ray.util.remove_placement_group(pg)
                except Exception:
                    pass
