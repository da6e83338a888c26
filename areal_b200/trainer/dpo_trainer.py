"""DPO trainer (reference: ``areal/trainer/dpo_trainer.py:84-523``): reference log-probs from
a frozen copy of the initial policy (or ``config.ref``), then the preference loss on
alternating (chosen, rejected) sequences."""
from __future__ import annotations

import copy

import torch

from ..engine.train_engine import B200DPOEngine, B200TrainEngine
from ..utils import data as D
from ._base import SupervisedTrainer
from .rw_trainer import RWTrainer


def dpo_pair_collate(samples):
    seqs = []
    for s in samples:
        p = list(s.get("prompt_ids", []))
        for key in ("chosen_ids", "rejected_ids"):
            ids = torch.as_tensor(p + list(s[key]))
            mask = torch.tensor([0] * len(p) + [1] * (len(ids) - len(p)), dtype=torch.int32)
            seqs.append(dict(input_ids=ids, loss_mask=mask))
    return D.pad_sequences_to_tensors(seqs)


class DPOTrainer(RWTrainer):
    def __init__(self, config, train_dataset, valid_dataset=None, **kw):
        kw.setdefault("collate_fn", dpo_pair_collate)
        self._beta, self._loss_type = config.beta, config.loss_type
        SupervisedTrainer.__init__(self, config, train_dataset, valid_dataset, **kw)
        ref_cfg = copy.deepcopy(config.ref if config.ref is not None else config.actor)
        ref_cfg.optimizer = None
        self.ref = B200TrainEngine(ref_cfg)
        self.ref.create_process_group()
        self.ref.initialize(model_config=self.engine.model_config, seed=config.seed)
        with torch.no_grad():  # frozen copy of the policy at initialisation
            self.ref.store.flat_param.copy_(self.engine.store.flat_param)

    def _build_engine(self, ecfg, model_config):
        eng = B200DPOEngine(ecfg, beta=self._beta, loss_type=self._loss_type)
        eng.create_process_group()
        eng.initialize(ft_spec=self.ft_spec, model_config=model_config, seed=self.config.seed)
        return eng

    def _with_ref(self, batch):
        batch = dict(batch)
        batch["ref_logp"] = self.ref.forward_batch(batch, output="logprobs")
        return batch

    def train_step(self, batch):
        return self.engine.train_dpo(self._with_ref(batch))

    def eval_step(self, batch):
        return self.engine.evaluate_dpo(self._with_ref(batch))

    def close(self):
        self.ref.destroy()
        super().close()
