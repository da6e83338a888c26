"""Countdown: reach a target with the given numbers (GRPO, rule-based reward; problems are
generated on the fly, so only a tokenizer / checkpoint is needed).

    python examples/countdown/train.py --config examples/math/gsm8k_grpo.yaml train_dataset.path=synthetic/countdown
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.reward import countdown_reward_fn
from areal_b200.rollout.workflows.rlvr import RLVRWorkflow
from areal_b200.trainer import PPOTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    tok = load_hf_tokenizer(config.tokenizer_path)
    train = get_custom_dataset("synthetic/countdown", tokenizer=None, size=16384, n_numbers=3)
    wf = RLVRWorkflow(countdown_reward_fn, config.gconfig, tokenizer=tok)
    with PPOTrainer(config, train, tokenizer=tok) as trainer:
        trainer.train(workflow=wf)


if __name__ == "__main__":
    main(sys.argv[1:])
