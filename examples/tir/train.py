"""Tool-integrated reasoning on math problems: the policy may write ``python`` blocks, which run
in the local sandbox; their output is appended (masked from the loss) and the policy continues.

    python examples/tir/train.py --config examples/math/gsm8k_grpo.yaml
"""
import os
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.infra.sandbox.local import LocalSandbox, SandboxConfig
from areal_b200.reward import gsm8k_reward_fn
from areal_b200.rollout.workflows.rlvr import GroupedRolloutWorkflow
from areal_b200.rollout.workflows.tir import TIRWorkflow
from areal_b200.trainer import PPOTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    tok = load_hf_tokenizer(config.tokenizer_path)
    train = get_custom_dataset(config.train_dataset.path, type="rl", split="train", tokenizer=tok, max_length=config.train_dataset.max_length)
    one = TIRWorkflow(gsm8k_reward_fn, config.gconfig, tok, max_tool_calls=int(os.environ.get("MAX_TOOL_CALLS", 4)),
                      sandbox=LocalSandbox(SandboxConfig(timeout_s=5.0, memory_mb=512)))
    with PPOTrainer(config, train, tokenizer=tok) as trainer:
        trainer.train(workflow=GroupedRolloutWorkflow.from_gconfig(one, config.gconfig))


if __name__ == "__main__":
    main(sys.argv[1:])
