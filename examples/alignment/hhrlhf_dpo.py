"""Direct preference optimisation on chosen/rejected pairs (a frozen copy of the initial
policy is the reference)."""
import sys

from areal_b200.api.cli_args import DPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer import DPOTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, DPOConfig)
    tok = load_hf_tokenizer(config.tokenizer_path)
    train = get_custom_dataset(config.train_dataset.path, type="dpo", split="train", tokenizer=tok, max_length=config.train_dataset.max_length)
    with DPOTrainer(config, train, tokenizer=tok) as trainer:
        trainer.train()


if __name__ == "__main__":
    main(sys.argv[1:])
