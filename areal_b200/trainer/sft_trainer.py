"""Supervised fine-tuning trainer (reference: ``areal/trainer/sft_trainer.py:58-465``).
Samples: ``input_ids`` + ``loss_mask`` (1 on answer tokens)."""
from __future__ import annotations

from ..engine.train_engine import B200LMEngine
from ._base import SupervisedTrainer


class SFTTrainer(SupervisedTrainer):
    engine_cls = B200LMEngine

    def train_step(self, batch):
        return self.engine.train_lm(batch)

    def eval_step(self, batch):
        return self.engine.evaluate_lm(batch)
