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
