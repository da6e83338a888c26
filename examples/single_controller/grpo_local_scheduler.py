"""Single-controller deployment: this script is the only user process; it asks a scheduler for
worker processes, creates the engines inside them over RPC, and drives the same ``PPOTrainer``
loop through ``TrainController`` / ``RolloutController``.

    python examples/single_controller/grpo_local_scheduler.py --config examples/tiny/arithmetic_grpo.yaml \
        [n_train=2 n_rollout=1 gpus_per_worker=0]
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.infra.controller import RolloutController, TrainController
from areal_b200.infra.scheduler import LocalScheduler
from areal_b200.models.config import ModelConfig, preset
from areal_b200.trainer import PPOTrainer


def main(argv):
    extra = {k: int(v) for k, v in (a.split("=") for a in argv if a.split("=")[0] in ("n_train", "n_rollout", "gpus_per_worker"))}
    argv = [a for a in argv if a.split("=")[0] not in extra]
    config, _ = load_expr_config(argv, GRPOConfig)
    mc_d = dict(config.actor.model_config or {})
    mc = preset(mc_d.pop("preset"), **mc_d) if "preset" in mc_d else ModelConfig.from_pretrained(config.actor.path)
    gpw = extra.get("gpus_per_worker", 0)
    sched = LocalScheduler(gpu_devices=None if gpw else [])
    actor = TrainController("areal_b200.engine.train_engine.B200PPOActor", config.actor, sched, role="actor")
    rollout = RolloutController("areal_b200.engine.infer_engine.NativeInferenceEngine", config.rollout, sched, role="rollout")
    try:
        actor.initialize(model_config=mc, seed=config.seed, n_workers=extra.get("n_train", 2), gpus_per_worker=gpw,
                         group_size=config.gconfig.n_samples)
        rollout.initialize(n_workers=extra.get("n_rollout", 1), gpus_per_worker=gpw, engine_kwargs={"model_config": mc},
                           init_kwargs={"seed": config.seed})
        ds = get_custom_dataset(config.train_dataset.path, size=256)
        trainer = PPOTrainer(config, ds, model_config=mc, actor_engine=actor, rollout_engine=rollout)
        hist = trainer.train(workflow="areal_b200.rollout.workflows.rlvr.RLVRWorkflow",
                             workflow_kwargs={"reward_fn": "areal_b200.dataset.small_id_fraction_reward_fn", "gconfig": config.gconfig,
                                              "reward_in_process": True})
        print("steps:", len(hist), "last reward:", hist[-1]["ppo_actor/task_reward/avg"])
    finally:
        rollout.destroy()
        actor.destroy()
        sched.delete_workers()


if __name__ == "__main__":
    main(sys.argv[1:])
