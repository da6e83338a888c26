"""Train-engine parity with expert parallelism: d4e2 and d2e2 (gloo ranks) against a single-rank
engine on the same global batch of a tiny MoE model. Prints ENGINE_EP_OK per rank."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ["AREAL_FORCE_CPU"] = "1"

from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig  # noqa: E402
from areal_b200.api.io_struct import SaveLoadMeta  # noqa: E402
from areal_b200.engine.train_engine import B200TrainEngine  # noqa: E402
from areal_b200.models import hf_io  # noqa: E402
from areal_b200.models.config import preset  # noqa: E402
from areal_b200.models.decoder import build_model  # noqa: E402


def loss_fn(logp, ent, mb):
    m = mb["loss_mask"].bool()
    return -(logp * m).sum() / m.sum().clamp(min=1)


def weight_fn(mb):
    return mb["loss_mask"].count_nonzero()


def make_batch(vocab):
    g = torch.Generator().manual_seed(11)
    B, L = 8, 24
    lens = torch.tensor([24, 9, 17, 12, 20, 7, 15, 22])
    am = torch.arange(L)[None] < lens[:, None]
    ids = torch.randint(0, vocab, (B, L), generator=g) * am
    lm = am.clone()
    lm[:, :3] = False
    lm[torch.arange(B), lens - 1] = False
    return dict(input_ids=ids, attention_mask=am, loss_mask=lm.int())


def cfg_of(backend):
    return TrainEngineConfig(init_from_scratch=True, dtype="float32", backend=backend, optimizer=OptimizerConfig(lr=1e-2, gradient_clipping=0.5),
                             mb_spec=MicroBatchSpec(max_tokens_per_mb=64))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    mc = preset("tiny-qwen3-moe")
    eng = B200TrainEngine(cfg_of(f"native:d{world}e2"))
    eng.create_process_group()
    eng.initialize(model_config=mc, seed=5)
    assert eng.ep_size == 2 and eng.ep_rank == rank % 2 and eng.expert_store is not None
    assert eng.expert_store.world_size == world // 2
    batch = make_batch(mc.vocab_size)
    per = 8 // world
    mine = {k: v[rank * per:(rank + 1) * per] for k, v in batch.items()}
    stats = [eng.train_batch(mine, loss_fn, weight_fn) for _ in range(2)]
    ref = B200TrainEngine(cfg_of("d1"))
    ref.set_train_ranks([rank])
    ref.create_process_group()
    ref.initialize(model_config=mc, seed=5)
    rstats = [ref.train_batch(batch, loss_fn, weight_fn) for _ in range(2)]
    for a, b in zip(stats, rstats):
        assert abs(a["grad_norm"] - b["grad_norm"]) < 2e-3 * max(1.0, b["grad_norm"]), (a, b)
    full = {n: p.detach() for n, p in ref.model.named_parameters()}
    El = mc.num_experts // 2
    worst = 0.0
    for n, p in eng.model.named_parameters():
        want = full[n][eng.ep_rank * El:(eng.ep_rank + 1) * El] if n in eng._expert_param_names else full[n]
        diff = (p.detach() - want).abs()
        worst = max(worst, diff.max().item())
        assert diff.mean().item() < 2e-5 and diff.max().item() < 5e-3, f"weights diverged for {n}: max {diff.max().item()}"
    # HF export gathers the experts; reload slices them again
    path = os.environ["EP_SAVE_DIR"]
    eng.save(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
    dist.barrier()
    m = build_model(mc, dtype=torch.float32, device="cpu", seed=0)
    hf_io.load_model_hf(m, path)
    for n, p in m.named_parameters():
        assert (p.detach() - full[n]).abs().max().item() < 5e-3, n
    w = eng.export_weights()
    assert set(w) == set(full) and all(w[n].shape == full[n].shape for n in w)
    eng.load(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
    # recovery checkpoint round trip (weights + both optimizers)
    spath = os.path.join(path, "sharded")
    eng.save(SaveLoadMeta(path=spath, weight_format="sharded", with_optim=True))
    before = eng.expert_optimizer.exp_avg.clone()
    eng.expert_optimizer.exp_avg.zero_()
    eng.load(SaveLoadMeta(path=spath, weight_format="sharded", with_optim=True))
    assert torch.equal(before, eng.expert_optimizer.exp_avg)
    third = eng.train_batch(mine, loss_fn, weight_fn)
    rthird = ref.train_batch(batch, loss_fn, weight_fn)
    assert abs(third["grad_norm"] - rthird["grad_norm"]) < 3e-3 * max(1.0, rthird["grad_norm"]), (third, rthird)
    if rank == 0:
        print(f"grad norms {[round(s['grad_norm'], 4) for s in stats]} vs {[round(s['grad_norm'], 4) for s in rstats]}; worst weight diff {worst:.2e}", flush=True)
    print("ENGINE_EP_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
