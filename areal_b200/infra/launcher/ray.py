"""SPMD launcher on a Ray cluster: every trainer rank and every rollout server becomes a Ray
task pinned to one GPU (placement group, STRICT_PACK per node), rank 0's address is the
``torch.distributed`` rendezvous. Reference: ``areal/infra/launcher/ray.py``.

    python -m areal_b200.infra.launcher.ray train_script.py --config cfg.yaml [overrides...]

Ray is imported lazily (it is not part of every image); :func:`plan_tasks` is a pure function."""
from __future__ import annotations

import os
import runpy
import sys
from typing import Optional

from ...api.alloc_mode import AllocationMode
from ...api.cli_args import BaseExperimentConfig, parse_cli_args, to_structured_cfg


def plan_tasks(cfg: BaseExperimentConfig) -> list[dict]:
    """``[{name, role, rank, world, gpus}]`` for the allocation of ``cfg``."""
    alloc = AllocationMode.from_str(cfg.allocation_mode) if cfg.allocation_mode else None
    tasks = []
    gen = alloc.gen if alloc is not None else None
    if gen is not None and alloc.train is not None and gen is not alloc.train:
        per = max(1, gen.parallel.tp_size * gen.parallel.pp_size)
        for i in range(gen.parallel.dp_size):
            tasks.append(dict(name=f"llm_server_{i}", role="server", rank=i, world=gen.parallel.dp_size, gpus=per))
    n_train = alloc.train.world_size if alloc is not None and alloc.train is not None else 1
    for r in range(n_train):
        tasks.append(dict(name=f"trainer_{r}", role="trainer", rank=r, world=n_train, gpus=1))
    return tasks


def _run_rank(script: str, argv: list[str], env: dict):
    os.environ.update(env)
    sys.argv = [script] + argv
    runpy.run_path(script, run_name="__main__")
    return 0


def launch(script: str, script_args: list[str], cfg: BaseExperimentConfig, ray_module=None, master_port: int = 29500) -> int:
    ray = ray_module
    if ray is None:
        import ray  # noqa: PLC0415
    if not ray.is_initialized():
        ray.init(address=os.environ.get("RAY_ADDRESS", "auto"))
    tasks = plan_tasks(cfg)
    remote_run = ray.remote(_run_rank)
    trainers = [t for t in tasks if t["role"] == "trainer"]
    master = os.environ.get("MASTER_ADDR", "127.0.0.1")
    futures = []
    for t in tasks:
        if t["role"] == "server":
            env = {"AREAL_SERVER_INDEX": str(t["rank"])}
            futures.append(remote_run.options(num_gpus=t["gpus"], name=t["name"]).remote(
                os.path.join(os.path.dirname(__file__), "..", "..", "engine", "server.py"),
                ["--model-path", getattr(getattr(cfg, "actor", None), "path", "") or "", "--experiment-name", cfg.experiment_name,
                 "--trial-name", cfg.trial_name, "--port", "0", "--announce"], env))
    runs = []
    for t in trainers:
        env = {"RANK": str(t["rank"]), "LOCAL_RANK": "0", "WORLD_SIZE": str(t["world"]), "MASTER_ADDR": master, "MASTER_PORT": str(master_port)}
        runs.append(remote_run.options(num_gpus=1, name=t["name"]).remote(script, script_args, env))
    codes = ray.get(runs)
    for f in futures:
        ray.cancel(f, force=True)
    from ..utils.launcher import run_post_exit_hook

    run_post_exit_hook(cfg)
    return 0 if all(c == 0 for c in codes) else 1


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        print(__doc__)
        return 2
    script, rest = argv[0], argv[1:]
    cfg_dict, _ = parse_cli_args(rest)
    cfg = to_structured_cfg(cfg_dict, BaseExperimentConfig, strict=False)
    return launch(script, rest, cfg)


if __name__ == "__main__":
    sys.exit(main())
