"""Slurm scheduler: each role is one ``sbatch`` job array-free batch script whose tasks start
RPC workers (``srun``); workers publish their address through ``name_resolve`` (NFS backend),
the scheduler polls ``squeue`` for state and cancels with ``scancel``. Engine calls go over
the same HTTP RPC as the local scheduler. Reference: ``areal/infra/scheduler/slurm.py``.
"""
from __future__ import annotations

import os
import re
import shlex
import subprocess
import time
from typing import Any, Optional

from ...api.scheduler_api import Job, Worker
from ...utils import logging as alog
from ...utils import name_resolve, names
from .exceptions import WorkerCreationError, WorkerFailedError, WorkerNotFoundError, WorkerTimeoutError
from .local import LocalScheduler, _WorkerInfo

logger = alog.getLogger("slurm_scheduler")

_FAILED_STATES = {"FAILED", "CANCELLED", "TIMEOUT", "NODE_FAIL", "OUT_OF_MEMORY", "PREEMPTED", "BOOT_FAIL"}


def render_sbatch_script(job_name: str, n_tasks: int, gpus_per_task: int, cpus_per_task: int, mem_gb: int, log_path: str,
                         command: str, partition: Optional[str] = None, nodelist: Optional[str] = None, exclude: Optional[str] = None,
                         time_limit: Optional[str] = None, container_image: str = "", container_mounts: str = "",
                         env: Optional[dict[str, str]] = None, extra_bash: Optional[list[str]] = None, tasks_per_node: Optional[int] = None,
                         reservation: Optional[str] = None, exclusive: bool = False, srun_additional_args: str = "",
                         container_type: str = "none") -> str:
    """Text of the batch script (pure function: unit-testable without Slurm). ``reservation`` / ``exclusive`` become
    ``#SBATCH`` options; ``srun_additional_args`` is appended to the ``srun`` line; ``container_type``: ``none`` /
    ``pyxis`` use srun's ``--container-image`` / ``--container-mounts``, ``apptainer`` (``singularity``) wraps the
    command in ``apptainer exec --nv --bind <mounts> <image>`` instead (reference:
    ``areal/infra/utils/slurm.py`` sbatch / srun templates, ``tests/test_slurm_reservation_and_env.py``)."""
    L = ["#!/bin/bash", f"#SBATCH --job-name={job_name}", f"#SBATCH --output={log_path}", "#SBATCH --open-mode=append",
         f"#SBATCH --ntasks={n_tasks}", f"#SBATCH --cpus-per-task={cpus_per_task}", f"#SBATCH --mem-per-cpu={max(1, mem_gb * 1024 // max(1, cpus_per_task))}M"]
    if gpus_per_task:
        L.append(f"#SBATCH --gres=gpu:{gpus_per_task * (tasks_per_node or 1)}")
    if tasks_per_node:
        L.append(f"#SBATCH --ntasks-per-node={tasks_per_node}")
    if partition:
        L.append(f"#SBATCH --partition={partition}")
    if nodelist:
        L.append(f"#SBATCH --nodelist={nodelist}")
    if exclude:
        L.append(f"#SBATCH --exclude={exclude}")
    if time_limit:
        L.append(f"#SBATCH --time={time_limit}")
    if reservation:
        L.append(f"#SBATCH --reservation={reservation}")
    if exclusive:
        L.append("#SBATCH --exclusive")
    L.append("")
    for k, v in (env or {}).items():
        L.append(f"export {k}={shlex.quote(str(v))}")
    L += list(extra_bash or [])
    srun = ["srun", "--kill-on-bad-exit=1", f"--ntasks={n_tasks}", f"--cpus-per-task={cpus_per_task}"]
    if gpus_per_task:
        srun.append(f"--gpus-per-task={gpus_per_task}")
    ctype = (container_type or "none").lower()
    if container_image and ctype in ("apptainer", "singularity"):
        bind = f"--bind {container_mounts} " if container_mounts else ""
        command = f"{ctype} exec --nv {bind}{shlex.quote(container_image)} bash -c {shlex.quote(command)}"
    elif container_image:
        srun += [f"--container-image={container_image}"] + ([f"--container-mounts={container_mounts}"] if container_mounts else [])
    if srun_additional_args:
        srun += shlex.split(srun_additional_args)
    L.append(" ".join(srun) + " bash -c " + shlex.quote(command))
    return "\n".join(L) + "\n"


class SlurmScheduler(LocalScheduler):
    """Shares the RPC client half with :class:`LocalScheduler`; only worker lifecycle differs."""

    def __init__(self, experiment_name: str, trial_name: str, fileroot: str, n_gpus_per_node: int = 8, container_image: str = "",
                 container_mounts: str = "", startup_timeout: float = 600.0, python: str = "python"):
        super().__init__(gpu_devices=[], log_dir=os.path.join(fileroot, "logs", experiment_name, trial_name, "slurm"),
                         startup_timeout=startup_timeout)
        self.experiment_name, self.trial_name, self.fileroot = experiment_name, trial_name, fileroot
        self.n_gpus_per_node = n_gpus_per_node
        self.container_image, self.container_mounts = container_image, container_mounts
        self.python = python
        self._job_ids: dict[str, str] = {}

    def _run(self, cmd: list[str]) -> str:
        return subprocess.check_output(cmd, text=True, stderr=subprocess.STDOUT)

    def create_workers(self, job: Job, *args, **kwargs) -> list[str]:
        role = job.role
        if role in self._workers:
            raise WorkerCreationError(role, "role already exists")
        if job.scheduling_strategy.type == "colocation" and job.scheduling_strategy.target:
            return self.fork_workers(role, job.scheduling_strategy.target)
        spec = job.tasks[0]
        key_root = names.worker_discovery(self.experiment_name, self.trial_name, role, 0).rsplit("/", 1)[0]
        worker_cmd = (f"{self.python} -m areal_b200.infra.rpc.rpc_server --host $(hostname -i | cut -d' ' -f1) --port 0 "
                      f"--role {role} --index $SLURM_PROCID --announce {key_root}")
        tpn = max(1, self.n_gpus_per_node // spec.gpu) if spec.gpu else None
        script = render_sbatch_script(
            f"{self.experiment_name}_{self.trial_name}:{role}", job.replicas, spec.gpu, spec.cpu, spec.mem,
            os.path.join(self.log_dir, f"{role}.log"), worker_cmd, spec.partition, spec.nodelist, spec.exclude, spec.time_limit,
            spec.image or self.container_image, spec.mount or self.container_mounts,
            {**spec.env_vars, "AREAL_NAME_RESOLVE_ROOT": os.path.join(self.fileroot, "name_resolve")}, spec.additional_bash_cmds,
            tasks_per_node=min(tpn, job.replicas) if tpn else None, reservation=spec.reservation, exclusive=spec.exclusive,
            srun_additional_args=spec.srun_additional_args, container_type=spec.container_type)
        path = os.path.join(self.log_dir, f"{role}.sbatch")
        with open(path, "w") as f:
            f.write(script)
        try:
            out = self._run(["sbatch", path])
        except (subprocess.CalledProcessError, FileNotFoundError) as e:
            raise WorkerCreationError(role, "sbatch failed", getattr(e, "output", repr(e)))
        m = re.search(r"Submitted batch job (\d+)", out)
        if not m:
            raise WorkerCreationError(role, "could not parse sbatch output", out)
        self._job_ids[role] = m.group(1)
        self._workers[role] = [_WorkerInfo(Worker(id=f"{role}/{i}", ip="", worker_ports=[]), role, None, path) for i in range(job.replicas)]
        return [w.worker.id for w in self._workers[role]]

    def job_state(self, role: str) -> str:
        jid = self._job_ids[role]
        out = self._run(["squeue", "-j", jid, "-h", "-o", "%T"]).strip()
        if not out:
            out = self._run(["sacct", "-j", jid, "-n", "-X", "-o", "State"]).strip()
        return out.split()[0] if out else "UNKNOWN"

    def get_workers(self, role: str, timeout: Optional[float] = None) -> list[Worker]:
        if role not in self._workers:
            raise WorkerNotFoundError(role)
        infos = self._workers[role]
        if infos and infos[0].forked_from:
            return [wi.worker for wi in infos]
        deadline = time.monotonic() + (timeout or self.startup_timeout)
        while True:
            st = self.job_state(role)
            if st in _FAILED_STATES:
                raise WorkerFailedError(f"{role}/*", st)
            missing = 0
            for i, wi in enumerate(infos):
                if wi.worker.worker_ports:
                    continue
                try:
                    addr = name_resolve.get(names.worker_discovery(self.experiment_name, self.trial_name, role, i))
                    ip, port = addr.rsplit(":", 1)
                    wi.worker.ip, wi.worker.worker_ports = ip, [port]
                except Exception:
                    missing += 1
            if missing == 0:
                break
            if time.monotonic() > deadline:
                raise WorkerTimeoutError(role, timeout or self.startup_timeout)
            time.sleep(1.0)
        return super().get_workers(role, timeout=max(1.0, deadline - time.monotonic()))

    def delete_workers(self, role: Optional[str] = None):
        for r in ([role] if role else list(self._workers)):
            self._workers.pop(r, None)
            jid = self._job_ids.pop(r, None)
            if jid:
                try:
                    self._run(["scancel", jid])
                except Exception as e:
                    logger.warning("scancel %s failed: %r", jid, e)
