"""Environment and command assembly shared by the launchers (reference:
``areal/infra/utils/launcher.py``)."""
from __future__ import annotations

import os
import sys
from typing import Optional

BASE_ENVIRONS = {
    "TOKENIZERS_PARALLELISM": "true",
    "PYTORCH_ALLOC_CONF": "expandable_segments:True",
    "CUDA_DEVICE_MAX_CONNECTIONS": "8",
    "NCCL_CUMEM_ENABLE": "1",
    "NCCL_NVLS_ENABLE": "1",
}


def get_env_vars(extra: Optional[dict] = None, env_string: str = "") -> dict[str, str]:
    """``BASE_ENVIRONS`` + ``K=V,K2=V2`` from the config + explicit overrides."""
    env = dict(BASE_ENVIRONS)
    for kv in filter(None, (s.strip() for s in env_string.split(","))):
        k, _, v = kv.partition("=")
        env[k] = v
    env.update({k: str(v) for k, v in (extra or {}).items()})
    return env


def torchrun_cmd(script: str, script_args: list[str], nproc: int, nnodes: int = 1, node_rank: int = 0,
                 master_addr: str = "127.0.0.1", master_port: int = 29500) -> list[str]:
    return [sys.executable, "-m", "torch.distributed.run", f"--nnodes={nnodes}", f"--nproc-per-node={nproc}",
            f"--node-rank={node_rank}", "--master-addr", master_addr, "--master-port", str(master_port), script, *script_args]


def server_cmd(model_path: str, port: int, experiment_name: str, trial_name: str, index: int, extra: Optional[dict] = None) -> list[str]:
    cmd = [sys.executable, "-m", "areal_b200.engine.server", "--port", str(port), "--experiment-name", experiment_name,
           "--trial-name", trial_name, "--server-index", str(index)]
    if model_path:
        cmd += ["--model-path", model_path]
    for k, v in (extra or {}).items():
        cmd += [f"--{k.replace('_', '-')}", str(v)]
    return cmd


def log_path(fileroot: str, experiment_name: str, trial_name: str, name: str) -> str:
    d = os.path.join(fileroot, "logs", experiment_name, trial_name)
    os.makedirs(d, exist_ok=True)
    return os.path.join(d, f"{name}.log")


# --------------------------------------------------------------------------- job records, waits, checks, hooks
import enum  # noqa: E402
import getpass  # noqa: E402
import subprocess  # noqa: E402
import time  # noqa: E402
from dataclasses import dataclass  # noqa: E402


class JobState(enum.Enum):
    NOT_FOUND = 0
    PENDING = 1
    RUNNING = 2
    COMPLETED = 3
    FAILED = 4
    CANCELLED = 5

    def active(self) -> bool:
        return self in (JobState.PENDING, JobState.RUNNING)


class JobException(Exception):
    def __init__(self, run_name: str, worker_type: str, host: str, reason: JobState):
        super().__init__(f"job {run_name}:{worker_type} on {host} ended as {reason.name}")
        self.run_name, self.worker_type, self.host, self.reason = run_name, worker_type, host, reason


@dataclass
class JobInfo:
    name: str
    state: JobState
    host: Optional[str] = None
    submit_time: Optional[str] = None
    start_time: Optional[str] = None
    slurm_id: Optional[int] = None


def wait_llm_server_addrs(experiment_name: str, trial_name: str, n_rollout_servers: int = 1, timeout: Optional[float] = 1200.0,
                          poll: float = 1.0) -> list[str]:
    """Blocks until ``n_rollout_servers`` generation servers have announced themselves under the trial's name-resolve
    key; returns their addresses."""
    from ...utils import name_resolve, names

    key = names.gen_servers(experiment_name, trial_name)
    t0 = time.perf_counter()
    while True:
        addrs = name_resolve.get_subtree(key)
        if len(addrs) >= n_rollout_servers:
            return list(addrs)
        if timeout is not None and time.perf_counter() - t0 > timeout:
            raise TimeoutError(f"waited {timeout:.0f}s for {n_rollout_servers} rollout servers, found {len(addrs)}")
        time.sleep(poll)


def validate_config_for_launcher(config, n_gpus_available: Optional[int] = None) -> None:
    """What a launcher checks before it starts anything: an RL layout needs ``actor`` and ``rollout`` sections, the
    layout's GPU count must fit the cluster, shared paths must be usable."""
    from ...api.alloc_mode import AllocationMode

    if not getattr(config, "allocation_mode", ""):
        return
    alloc = AllocationMode.from_str(config.allocation_mode)
    gen = getattr(alloc, "gen", None)
    train = getattr(alloc, "train", None)
    if gen is not None and train is not None and gen is not train:
        for section in ("actor", "rollout"):
            if not hasattr(config, section):
                raise RuntimeError(f"`{section}` is required when allocation_mode has an inference part ('{config.allocation_mode}'): "
                                   "use an RL config, or drop the inference part from the layout")
    cl = getattr(config, "cluster", None)
    if cl is not None:
        have = n_gpus_available if n_gpus_available is not None else int(cl.n_nodes) * int(cl.n_gpus_per_node)
        need = (gen.world_size if gen is not None and gen is not train else 0) + (train.world_size if train is not None else 0)
        if have > 0 and need > have:          # (0: a CPU-only launch, processes are not tied to devices)
            raise ValueError(f"allocation_mode '{config.allocation_mode}' needs {need} GPUs, the cluster section offers {have}")
        if gen is not None and gen.parallel.tp_size > int(cl.n_gpus_per_node):
            raise ValueError("a rollout replica's tensor-parallel group must fit one node")
        root = getattr(cl, "fileroot", None)
        if root:
            os.makedirs(root, exist_ok=True)
            if not os.access(root, os.W_OK):
                raise PermissionError(f"cluster.fileroot '{root}' is not writable")


def run_post_exit_hook(config, timeout: float = 600.0) -> Optional[int]:
    """Runs ``config.post_exit_hook`` after the job ended (success or not): a shell command (``LOG_DIR`` points at the
    trial's log directory) or the import path ``package.module:function`` of a callable taking the config. A failing or
    slow hook is logged and never raises: it must not stand in the way of recovery. Returns the command's exit code
    (0 for a callable that returned), ``None`` when there is no hook."""
    from ...utils import logging as alog

    log = alog.getLogger("launcher")
    hook = (getattr(config, "post_exit_hook", None) or "").strip()
    if not hook:
        return None
    try:
        if ":" in hook and " " not in hook and "/" not in hook.split(":")[0]:
            import importlib

            mod, _, fn = hook.partition(":")
            getattr(importlib.import_module(mod), fn)(config)
            return 0
        env = dict(os.environ)
        try:
            env["LOG_DIR"] = os.path.join(config.cluster.fileroot, "logs", getpass.getuser(), config.experiment_name, config.trial_name)
        except Exception:  # noqa: BLE001
            pass
        r = subprocess.run(hook, shell=True, timeout=timeout, capture_output=True, text=True, env=env)
        if r.stdout.strip():
            log.info("post-exit hook: %s", r.stdout.strip()[-2000:])
        if r.returncode != 0:
            log.warning("post-exit hook exited with code %d: %s", r.returncode, r.stderr.strip()[-2000:])
        return r.returncode
    except subprocess.TimeoutExpired:
        log.warning("post-exit hook timed out after %.0fs: %s", timeout, hook)
        return -1
    except Exception as e:  # noqa: BLE001
        log.warning("post-exit hook failed: %r", e)
        return -1
