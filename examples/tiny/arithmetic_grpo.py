"""Smallest end-to-end asynchronous GRPO run (no external files; CPU or one GPU)."""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset, small_id_fraction_reward_fn
from areal_b200.rollout.workflows.rlvr import RLVRWorkflow
from areal_b200.trainer import PPOTrainer


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    ds = get_custom_dataset(config.train_dataset.path, size=256)
    wf = RLVRWorkflow(small_id_fraction_reward_fn, config.gconfig, reward_in_process=True)
    with PPOTrainer(config, ds) as trainer:
        hist = trainer.train(workflow=wf)
    r = [h["ppo_actor/task_reward/avg"] for h in hist]
    print(f"reward: first 3 steps {sum(r[:3]) / 3:.3f} -> last 3 steps {sum(r[-3:]) / 3:.3f}")


if __name__ == "__main__":
    main(sys.argv[1:])
