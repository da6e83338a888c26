"""On-policy distillation next to the RL objective: a frozen teacher scores the student's own
samples and the actor loss adds ``distill_loss_weight * reverse-KL`` to ``rl_loss_weight *``
the GRPO term. The teacher is the ``teacher:`` section of the config (a train engine without
optimizer; ``teacher.path`` points at the larger checkpoint).

    python examples/distillation/gsm8k_distill.py --config examples/distillation/gsm8k_distill.yaml
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.reward import gsm8k_reward_fn
from areal_b200.rollout.workflows.rlvr import RLVRWorkflow
from areal_b200.trainer import PPOTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    if config.teacher is None:
        raise SystemExit("this example needs a `teacher:` section (see gsm8k_distill.yaml)")
    tok = load_hf_tokenizer(config.tokenizer_path)
    train = get_custom_dataset(config.train_dataset.path, type="rl", split="train", tokenizer=tok, max_length=config.train_dataset.max_length)
    with PPOTrainer(config, train, tokenizer=tok) as trainer:
        trainer.train(workflow=RLVRWorkflow(gsm8k_reward_fn, config.gconfig, tokenizer=tok))


if __name__ == "__main__":
    main(sys.argv[1:])
