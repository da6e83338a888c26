"""Multi-turn self-correction: on a wrong answer the model is told so and tries again; the
final reward is discounted per retry. Uses the same YAML schema as ``examples/math`` plus
``+max_turns=3 +turn_discount=0.9`` style overrides read from the environment of this script."""
import os
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.reward import gsm8k_reward_fn
from areal_b200.rollout.workflows.multi_turn import MultiTurnWorkflow
from areal_b200.rollout.workflows.rlvr import GroupedRolloutWorkflow
from areal_b200.trainer import PPOTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    tok = load_hf_tokenizer(config.tokenizer_path)
    train = get_custom_dataset(config.train_dataset.path, type="rl", split="train", tokenizer=tok, max_length=config.train_dataset.max_length)
    one = MultiTurnWorkflow(gsm8k_reward_fn, config.gconfig, tok, max_turns=int(os.environ.get("MAX_TURNS", 3)),
                            turn_discount=float(os.environ.get("TURN_DISCOUNT", 0.9)))
    wf = GroupedRolloutWorkflow.from_gconfig(one, config.gconfig)
    with PPOTrainer(config, train, tokenizer=tok) as trainer:
        trainer.train(workflow=wf)


if __name__ == "__main__":
    main(sys.argv[1:])
