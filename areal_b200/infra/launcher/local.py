"""Single-node SPMD launcher: starts the rollout servers of the allocation, then the trainer
ranks under ``torch.distributed.run``, and restarts the whole job (from the last recover
checkpoint) when a process dies, up to ``recover.retries`` times.

    python -m areal_b200.infra.launcher.local train_script.py --config cfg.yaml [overrides...]

GPU assignment: generation servers take the first ``gen.world_size`` devices (``tp*pp`` each),
trainers the next ``train.world_size``. Reference: ``areal/infra/launcher/local.py`` (restart
loop :432-452)."""
from __future__ import annotations

import os
import subprocess
import sys
import time
from typing import Optional

from ...api.alloc_mode import AllocationMode
from ...api.cli_args import BaseExperimentConfig, parse_cli_args, to_structured_cfg
from ...utils import logging as alog
from ...utils import name_resolve, names
from ...utils.network import find_free_ports
from ..utils.launcher import get_env_vars, log_path, server_cmd, torchrun_cmd
from ..utils.proc import terminate_popen

logger = alog.getLogger("local_launcher")


class JobFailed(RuntimeError):
    def __init__(self, name: str, code: int):
        super().__init__(f"process '{name}' exited with code {code}")
        self.name, self.code = name, code


class LocalLauncher:
    def __init__(self, experiment_name: str, trial_name: str, fileroot: str, n_gpus: Optional[int] = None):
        self.experiment_name, self.trial_name, self.fileroot = experiment_name, trial_name, fileroot
        if n_gpus is None:
            try:
                import torch

                n_gpus = torch.cuda.device_count()
            except Exception:
                n_gpus = 0
        self.n_gpus = n_gpus
        self._next_gpu = 0
        self.procs: dict[str, subprocess.Popen] = {}

    def _take_gpus(self, n: int) -> str:
        if n == 0:
            return ""
        if self._next_gpu + n > max(self.n_gpus, 0) and self.n_gpus > 0:
            raise RuntimeError(f"allocation needs more than the {self.n_gpus} visible GPUs")
        ids = list(range(self._next_gpu, self._next_gpu + n))
        self._next_gpu += n
        return ",".join(map(str, ids))

    def submit(self, name: str, cmd: list[str], gpus: int = 0, env: Optional[dict] = None) -> subprocess.Popen:
        e = dict(os.environ)
        e.update(env or {})
        if gpus and self.n_gpus:
            e["CUDA_VISIBLE_DEVICES"] = self._take_gpus(gpus)
        lp = log_path(self.fileroot, self.experiment_name, self.trial_name, name)
        logger.info("starting %s: %s (log: %s)", name, " ".join(cmd), lp)
        p = subprocess.Popen(cmd, env=e, stdout=open(lp, "a"), stderr=subprocess.STDOUT, start_new_session=True)
        self.procs[name] = p
        return p

    def wait(self, names_to_wait: Optional[list[str]] = None, poll: float = 0.5) -> None:
        """Returns when every waited process exited with 0; raises :class:`JobFailed` as soon
        as any process (waited or not) fails."""
        waited = set(names_to_wait or self.procs)
        while True:
            for n, p in self.procs.items():
                rc = p.poll()
                if rc is not None and rc != 0:
                    raise JobFailed(n, rc)
            if all(self.procs[n].poll() == 0 for n in waited):
                return
            time.sleep(poll)

    def stop_all(self):
        for p in self.procs.values():
            terminate_popen(p)
        self.procs.clear()
        self._next_gpu = 0


def launch(script: str, script_args: list[str], cfg: BaseExperimentConfig, n_gpus: Optional[int] = None, max_restarts: Optional[int] = None) -> int:
    from ..utils.launcher import run_post_exit_hook, validate_config_for_launcher

    validate_config_for_launcher(cfg, n_gpus_available=n_gpus)
    alloc = AllocationMode.from_str(cfg.allocation_mode) if cfg.allocation_mode else None
    la = LocalLauncher(cfg.experiment_name, cfg.trial_name, cfg.cluster.fileroot, n_gpus)
    os.environ.setdefault("AREAL_NAME_RESOLVE_ROOT", os.path.join(cfg.cluster.fileroot, "name_resolve", cfg.experiment_name, cfg.trial_name))
    name_resolve.reconfigure(type="nfs", record_root=os.environ["AREAL_NAME_RESOLVE_ROOT"])
    retries = cfg.recover.retries if max_restarts is None else max_restarts
    attempt = 0
    while True:
        name_resolve.clear_subtree(names.trial_root(cfg.experiment_name, cfg.trial_name))
        env = get_env_vars({"AREAL_NAME_RESOLVE_ROOT": os.environ["AREAL_NAME_RESOLVE_ROOT"],
                            "AREAL_RECOVER_RUN": "1" if attempt > 0 else "0"}, cfg.launcher.trainer_env_vars or "")
        senv = get_env_vars({"AREAL_NAME_RESOLVE_ROOT": os.environ["AREAL_NAME_RESOLVE_ROOT"]}, cfg.launcher.inference_server_env_vars or "")
        try:
            addrs = []
            gen = alloc.gen if alloc is not None else None
            if gen is not None and alloc.train is not None and gen is not alloc.train:
                per = max(1, gen.parallel.tp_size * gen.parallel.pp_size)
                for i in range(gen.parallel.dp_size):
                    port = find_free_ports(1)[0]
                    la.submit(f"llm_server_{i}", server_cmd(getattr(cfg, "actor").path if hasattr(cfg, "actor") else "", port,
                                                           cfg.experiment_name, cfg.trial_name, i,
                                                           {"max_running_requests": cfg.native_infer.max_running_requests,
                                                            "context_length": cfg.native_infer.context_length,
                                                            "mem_fraction_static": cfg.native_infer.mem_fraction_static}),
                              gpus=per, env=senv)
                    addrs.append(f"127.0.0.1:{port}")
                env["AREAL_LLM_SERVER_ADDRS"] = ",".join(addrs)
            n_train = alloc.train.world_size if alloc is not None and alloc.train is not None else max(1, la.n_gpus)
            la.submit("trainer", torchrun_cmd(script, script_args, n_train, master_port=find_free_ports(1)[0]), gpus=n_train, env=env)
            la.wait(["trainer"])
            la.stop_all()
            run_post_exit_hook(cfg)
            return 0
        except JobFailed as e:
            la.stop_all()
            attempt += 1
            if cfg.recover.mode in ("disabled", "off") or attempt > retries:
                logger.error("%s; giving up after %d attempt(s)", e, attempt)
                run_post_exit_hook(cfg)
                return e.code or 1
            logger.warning("%s; restarting the job (attempt %d of %d)", e, attempt, retries)
            time.sleep(1.0)
        except BaseException:
            la.stop_all()
            raise


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
