"""GRPO / PPO on GSM8K-style records: the canonical entry script.

    python examples/math/gsm8k_rl.py --config examples/math/gsm8k_grpo.yaml [key=value ...]

Mirrors the reference's ``examples/math/gsm8k_rl.py``: load the config, build datasets and the
trainer, hand it an RLVR workflow with the GSM8K reward, train."""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.reward import gsm8k_reward_fn
from areal_b200.rollout.workflows.rlvr import RLVRWorkflow
from areal_b200.trainer import PPOTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path)
    train = get_custom_dataset(config.train_dataset.path, type="rl", split="train", tokenizer=tokenizer,
                               max_length=config.train_dataset.max_length)
    valid = None
    if config.valid_dataset is not None:
        valid = get_custom_dataset(config.valid_dataset.path, type="rl", split="test", tokenizer=tokenizer)
    workflow = RLVRWorkflow(gsm8k_reward_fn, config.gconfig, tokenizer=tokenizer)
    # evaluation samples with its own generation settings when the config has an ``eval_gconfig`` section
    eval_g = config.eval_gconfig if config.eval_gconfig is not None else config.gconfig.new(temperature=0.6, n_samples=1)
    eval_workflow = RLVRWorkflow(gsm8k_reward_fn, eval_g, tokenizer=tokenizer)
    with PPOTrainer(config, train_dataset=train, valid_dataset=valid, tokenizer=tokenizer) as trainer:
        trainer.train(workflow=workflow, eval_workflow=eval_workflow)


if __name__ == "__main__":
    main(sys.argv[1:])
