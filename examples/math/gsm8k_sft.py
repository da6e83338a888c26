"""Supervised fine-tuning on question/answer records.

    python -m torch.distributed.run --nproc-per-node 8 examples/math/gsm8k_sft.py --config examples/math/gsm8k_sft.yaml
"""
import sys

from areal_b200.api.cli_args import SFTConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer import SFTTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, SFTConfig)
    tok = load_hf_tokenizer(config.tokenizer_path)
    train = get_custom_dataset(config.train_dataset.path, type="sft", split="train", tokenizer=tok, max_length=config.train_dataset.max_length)
    valid = get_custom_dataset(config.valid_dataset.path, type="sft", split="test", tokenizer=tok,
                               max_length=config.valid_dataset.max_length) if config.valid_dataset else None
    with SFTTrainer(config, train, valid, tokenizer=tok) as trainer:
        trainer.train()


if __name__ == "__main__":
    main(sys.argv[1:])
