"""LoRA adapters: math, freezing, engine training, merge / adapter checkpoint."""
import os

import torch

from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig
from areal_b200.api.io_struct import SaveLoadMeta
from areal_b200.engine.train_engine import B200LMEngine
from areal_b200.models import hf_io
from areal_b200.models.config import preset
from areal_b200.models.decoder import build_model
from areal_b200.models.lora import apply_lora, load_adapter, lora_named_parameters, merge_lora_, resolve_targets, save_adapter, unmerge_lora_


def _ids(cfg, T=48, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg.vocab_size, (T,), generator=g), torch.tensor([0, 20, 48], dtype=torch.int32)


def test_lora_is_identity_at_init_and_merge_roundtrip(tmp_path):
    cfg = preset("tiny-qwen3")
    m = build_model(cfg, dtype=torch.float32, device="cpu", seed=1)
    ids, cu = _ids(cfg)
    base = m(ids, cu, max_seqlen=28).detach()
    apply_lora(m, rank=4, alpha=8, target_modules=["q_proj", "down_proj"])
    assert resolve_targets(["q_proj", "down_proj"]) == {"qkv_proj", "down_proj"}
    names = [n for n, _ in lora_named_parameters(m)]
    assert len(names) == 2 * 2 * cfg.num_layers and all(p.requires_grad for _, p in lora_named_parameters(m))
    assert all(not p.requires_grad for n, p in m.named_parameters() if "_lora_" not in n)
    assert torch.allclose(m(ids, cu, max_seqlen=28), base, atol=1e-6)               # B = 0
    with torch.no_grad():
        for n, p in lora_named_parameters(m):
            if n.endswith("_B"):
                p.normal_(0, 0.05)
    tuned = m(ids, cu, max_seqlen=28).detach()
    assert (tuned - base).abs().max() > 1e-3
    merge_lora_(m)
    assert torch.allclose(m(ids, cu, max_seqlen=28), tuned, atol=2e-5)               # folded in, adapters bypassed
    unmerge_lora_(m)
    assert torch.allclose(m(ids, cu, max_seqlen=28), tuned, atol=2e-5)
    save_adapter(m, str(tmp_path / "ad"))
    assert os.path.exists(tmp_path / "ad" / "adapter_config.json")
    m2 = build_model(cfg, dtype=torch.float32, device="cpu", seed=1)
    apply_lora(m2, rank=4, alpha=8, target_modules=["q_proj", "down_proj"], seed=9)
    load_adapter(m2, str(tmp_path / "ad"))
    assert torch.allclose(m2(ids, cu, max_seqlen=28), tuned, atol=2e-5)


def test_engine_trains_only_adapters_and_saves_merged(tmp_path):
    cfg = TrainEngineConfig(init_from_scratch=True, dtype="float32", use_lora=True, lora_rank=4, lora_alpha=8, target_modules=["all-linear"],
                            optimizer=OptimizerConfig(lr=5e-2, weight_decay=0.0), mb_spec=MicroBatchSpec(max_tokens_per_mb=256))
    eng = B200LMEngine(cfg)
    eng.create_process_group()
    mc = preset("tiny-qwen3")
    eng.initialize(model_config=mc, seed=2)
    base = {n: p.detach().clone() for n, p in eng.model.named_parameters() if "_lora_" not in n}
    assert eng.store.numel < 0.2 * sum(p.numel() for p in base.values())                 # optimizer state covers adapters only
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, mc.vocab_size, (4, 32), generator=g)
    batch = dict(input_ids=ids, attention_mask=torch.ones(4, 32, dtype=torch.bool), loss_mask=torch.ones(4, 32, dtype=torch.int32))
    losses = [eng.train_lm(batch)["nll"] if "nll" in (r := eng.train_lm(batch)) else r["loss"] for _ in range(6)]
    assert losses[-1] < losses[0]
    for n, p in eng.model.named_parameters():
        if "_lora_" not in n:
            assert torch.equal(p, base[n]), n                                               # base weights untouched
    eng.save(SaveLoadMeta(path=str(tmp_path / "ck"), weight_format="hf", with_optim=False))
    merged = build_model(mc, dtype=torch.float32, device="cpu", seed=0)
    hf_io.load_model_hf(merged, str(tmp_path / "ck"))
    x, cu = _ids(mc)
    eng.model.eval()
    assert torch.allclose(merged(x, cu, max_seqlen=28), eng.model(x, cu, max_seqlen=28), atol=3e-5)
    assert os.path.exists(tmp_path / "ck" / "adapter" / "adapter_model.safetensors")
    w = eng.export_weights()
    assert all("_lora_" not in n for n in w) and not torch.equal(w["layers.0.mlp.down_proj"], base["layers.0.mlp.down_proj"])
