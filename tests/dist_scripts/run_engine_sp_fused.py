"""Sequence-parallel train engine on 2 GPUs: the attention blocks with both Ulysses exchanges
inside the projection kernels against the same engine on NCCL all-to-alls (same seed, same
batch, bf16). Prints ENGINE_SP_FUSED_OK per rank."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig  # noqa: E402
from areal_b200.engine.train_engine import B200TrainEngine  # noqa: E402
from areal_b200.models.config import preset  # noqa: E402


def loss_fn(logp, ent, mb):
    m = mb["loss_mask"].bool()
    return -(logp * m).sum() / m.sum().clamp(min=1)


def weight_fn(mb):
    return mb["loss_mask"].count_nonzero()


def make_batch(vocab):
    g = torch.Generator().manual_seed(3)
    B, L = 12, 320
    lens = torch.randint(40, L + 1, (B,), generator=g)
    am = torch.arange(L)[None] < lens[:, None]
    ids = torch.randint(0, vocab, (B, L), generator=g) * am
    lm = am.clone()
    lm[:, :8] = False
    lm[torch.arange(B), lens - 1] = False
    return dict(input_ids=ids, attention_mask=am, loss_mask=lm.int())


def engine(fused: bool, mc):
    cfg = TrainEngineConfig(init_from_scratch=True, dtype="bfloat16", backend="d1c2", optimizer=OptimizerConfig(lr=1e-3, gradient_clipping=1.0),
                            mb_spec=MicroBatchSpec(max_tokens_per_mb=2048))
    cfg.fsdp.fuse_ulysses_projections = fused
    e = B200TrainEngine(cfg)
    e.create_process_group()
    e.initialize(model_config=mc, seed=7)
    return e


def main():
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl")
    mc = preset("tiny-qwen3")
    batch = make_batch(mc.vocab_size)
    a = engine(True, mc)
    assert a.sp_size == 2 and a._sp_fused is not None and a.model.layers[0].self_attn.sp_fused is a._sp_fused
    b = engine(False, mc)
    assert b._sp_fused is None
    for step in range(2):
        sa = a.train_batch(batch, loss_fn, weight_fn)
        sb = b.train_batch(batch, loss_fn, weight_fn)
        assert abs(sa["loss"] - sb["loss"]) < 2e-2 * max(1.0, abs(sb["loss"])), (step, sa, sb)
        assert abs(sa["grad_norm"] - sb["grad_norm"]) < 3e-2 * max(1.0, sb["grad_norm"]), (step, sa, sb)
    worst = 0.0
    pb = dict(b.model.named_parameters())
    for n, p in a.model.named_parameters():
        d = (p.detach().float() - pb[n].detach().float()).abs()
        worst = max(worst, d.max().item())
        assert d.mean().item() < 2e-4 and d.max().item() < 8e-3, f"{n}: mean {d.mean().item():.2e} max {d.max().item():.2e}"
    # forward-only path (log-probs of the behaviour policy) agrees too
    la = a.forward_batch(batch)
    lb = b.forward_batch(batch)
    assert (la.float() - lb.float()).abs().max().item() < 0.15, (la.float() - lb.float()).abs().max().item()
    if dist.get_rank() == 0:
        print(f"loss {sa['loss']:.4f} vs {sb['loss']:.4f}; grad norm {sa['grad_norm']:.4f} vs {sb['grad_norm']:.4f}; worst weight diff {worst:.2e}", flush=True)
    print("ENGINE_SP_FUSED_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
