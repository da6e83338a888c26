"""Bradley-Terry reward model on chosen/rejected pairs (HH-RLHF style records)."""
import sys

from areal_b200.api.cli_args import RWConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer import RWTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, RWConfig)
    tok = load_hf_tokenizer(config.tokenizer_path)
    train = get_custom_dataset(config.train_dataset.path, type="rw", split="train", tokenizer=tok, max_length=config.train_dataset.max_length)
    valid = get_custom_dataset(config.valid_dataset.path, type="rw", split="test", tokenizer=tok,
                               max_length=config.valid_dataset.max_length) if config.valid_dataset else None
    with RWTrainer(config, train, valid, tokenizer=tok) as trainer:
        trainer.train()


if __name__ == "__main__":
    main(sys.argv[1:])
