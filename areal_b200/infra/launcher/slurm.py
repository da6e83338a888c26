"""Multi-node SPMD launcher on Slurm: one ``sbatch`` job for the rollout servers of the
allocation and one for the trainer ranks (``srun`` + ``torch.distributed.run`` per node), with
the rendezvous address published through the shared name-resolve directory.

    python -m areal_b200.infra.launcher.slurm train_script.py --config cfg.yaml [overrides...]

Reference: ``areal/infra/launcher/slurm.py`` (job arrays for servers and trainers, restart on
failure). The sbatch text comes from :func:`areal_b200.infra.scheduler.slurm.render_sbatch_script`,
so the scheduler and this launcher describe jobs the same way. ``--dry-run`` prints the scripts
instead of submitting them."""
from __future__ import annotations

import os
import shlex
import subprocess
import sys
import time
from typing import Optional

from ...api.alloc_mode import AllocationMode
from ...api.cli_args import BaseExperimentConfig, parse_cli_args, to_structured_cfg
from ...utils import logging as alog
from ..scheduler.slurm import render_sbatch_script

logger = alog.getLogger("slurm_launcher")


def plan_jobs(script: str, script_args: list[str], cfg: BaseExperimentConfig, gpus_per_node: int = 8) -> list[dict]:
    """The jobs of one experiment: ``[{name, nodes, gpus_per_node, command}]``."""
    alloc = AllocationMode.from_str(cfg.allocation_mode) if cfg.allocation_mode else None
    n_train = alloc.train.world_size if alloc is not None and alloc.train is not None else gpus_per_node
    jobs = []
    py = shlex.quote(sys.executable)
    args = " ".join(shlex.quote(a) for a in script_args)
    gen = alloc.gen if alloc is not None else None
    if gen is not None and alloc.train is not None and gen is not alloc.train:
        per = max(1, gen.parallel.tp_size * gen.parallel.pp_size)
        n_gpus = per * gen.parallel.dp_size
        jobs.append(dict(name="llm_server", nodes=-(-n_gpus // gpus_per_node), gpus_per_node=min(gpus_per_node, n_gpus),
                         command=f"{py} -m areal_b200.engine.server --model-path {shlex.quote(getattr(getattr(cfg, 'actor', None), 'path', '') or '')} "
                                 f"--experiment-name {cfg.experiment_name} --trial-name {cfg.trial_name} --port 0 --announce"))
    nodes = -(-n_train // gpus_per_node)
    per_node = min(gpus_per_node, n_train)
    jobs.append(dict(name="trainer", nodes=nodes, gpus_per_node=per_node,
                     command=f"{py} -m torch.distributed.run --nnodes={nodes} --nproc-per-node={per_node} --node-rank=$SLURM_NODEID "
                             f"--master-addr=$(scontrol show hostnames $SLURM_JOB_NODELIST | head -n1) --master-port=29500 {shlex.quote(script)} {args}"))
    return jobs


def launch(script: str, script_args: list[str], cfg: BaseExperimentConfig, gpus_per_node: int = 8, dry_run: bool = False,
           sbatch: str = "sbatch", poll_s: float = 10.0) -> int:
    from ..utils.launcher import validate_config_for_launcher

    validate_config_for_launcher(cfg)
    log_dir = os.path.join(cfg.cluster.fileroot, "logs", cfg.experiment_name, cfg.trial_name)
    os.makedirs(log_dir, exist_ok=True)
    ids = []
    for j in plan_jobs(script, script_args, cfg, gpus_per_node):
        # one task per node; that task starts the node's ranks
        text = render_sbatch_script(f"{cfg.experiment_name}_{cfg.trial_name}:{j['name']}", n_tasks=j["nodes"], gpus_per_task=j["gpus_per_node"],
                                    cpus_per_task=getattr(cfg.launcher, "trainer_cpus_per_gpu", 4) * j["gpus_per_node"],
                                    mem_gb=max(1, getattr(cfg.launcher, "trainer_mem_per_gpu", 32768) * j["gpus_per_node"] // 1024),
                                    log_path=os.path.join(log_dir, f"{j['name']}.log"), command=j["command"], tasks_per_node=1)
        if dry_run:
            print(text)
            continue
        path = os.path.join(log_dir, f"{j['name']}.sbatch")
        with open(path, "w") as f:
            f.write(text)
        out = subprocess.run([sbatch, "--parsable", path], capture_output=True, text=True, check=True).stdout.strip()
        ids.append(out.split(";")[0])
        logger.info("submitted %s as job %s", j["name"], ids[-1])
    if dry_run or not ids:
        return 0
    trainer = ids[-1]
    while True:                                   # the experiment ends with the trainer job
        st = subprocess.run(["squeue", "-h", "-j", trainer, "-o", "%T"], capture_output=True, text=True).stdout.strip()
        if not st:
            break
        time.sleep(poll_s)
    for j in ids[:-1]:
        subprocess.run(["scancel", j])
    acct = subprocess.run(["sacct", "-n", "-j", trainer, "-o", "State", "-X"], capture_output=True, text=True).stdout
    from ..utils.launcher import run_post_exit_hook

    run_post_exit_hook(cfg)
    return 0 if "COMPLETED" in acct or not acct.strip() else 1


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    dry = "--dry-run" in argv
    argv = [a for a in argv if a != "--dry-run"]
    if not argv:
        print(__doc__)
        return 2
    script, rest = argv[0], argv[1:]
    cfg_dict, _ = parse_cli_args(rest)
    cfg = to_structured_cfg(cfg_dict, BaseExperimentConfig, strict=False)
    return launch(script, rest, cfg, gpus_per_node=getattr(cfg.cluster, "n_gpus_per_node", 8), dry_run=dry)


if __name__ == "__main__":
    sys.exit(main())
