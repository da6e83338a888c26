"""Sharded (recovery) checkpoints across data-parallel world sizes. ``PHASE=save``: N gloo ranks train two steps and
write a sharded checkpoint plus, from rank 0, the whole flat state as the reference. ``PHASE=load``: M ranks start from
another seed, load the checkpoint (their ranges are stitched from the saved shards that overlap them) and compare
parameters, fp32 master weights and both moments with the reference; then one more step runs. Prints RESHARD_OK."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ["AREAL_FORCE_CPU"] = "1"

import torch
import torch.distributed as dist

from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig
from areal_b200.api.io_struct import SaveLoadMeta
from areal_b200.engine.train_engine import B200TrainEngine
from areal_b200.models.config import preset


def loss_fn(logp, ent, mb):
    m = mb["loss_mask"].bool()
    return -(logp * m).sum() / m.sum().clamp(min=1)


def batch(rank):
    g = torch.Generator().manual_seed(5 + rank)
    ids = torch.randint(0, 1024, (4, 20), generator=g)
    am = torch.ones(4, 20, dtype=torch.bool)
    lm = am.clone().int()
    lm[:, :3] = 0
    return dict(input_ids=ids, attention_mask=am, loss_mask=lm)


def gather_full(eng, shard):
    parts = [torch.empty_like(shard) for _ in range(eng.dp_size)]
    if eng.dp_size > 1:
        dist.all_gather(parts, shard.contiguous(), group=eng._shard_group)
    else:
        parts = [shard]
    return torch.cat(parts)[: eng.store.numel].clone()


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    root = os.environ["CKPT_DIR"]
    phase = os.environ["PHASE"]
    cfg = TrainEngineConfig(init_from_scratch=True, dtype="float32", optimizer=OptimizerConfig(lr=1e-2), mb_spec=MicroBatchSpec(max_tokens_per_mb=128))
    eng = B200TrainEngine(cfg)
    eng.create_process_group()
    eng.initialize(model_config=preset("tiny-qwen3"), seed=1 if phase == "save" else 99)
    if phase == "save":
        for _ in range(2):
            eng.train_batch(batch(rank), loss_fn, lambda mb: mb["loss_mask"].count_nonzero())
        eng.set_version(7)
        eng.save(SaveLoadMeta(path=os.path.join(root, "ckpt"), weight_format="sharded", with_optim=True))
        full = {k: gather_full(eng, t) for k, t in (("param", eng.store.param_shard), ("master", eng.optimizer.master),
                                                    ("exp_avg", eng.optimizer.exp_avg), ("exp_avg_sq", eng.optimizer.exp_avg_sq))}
        if rank == 0:
            torch.save(dict(full, step_count=eng.optimizer.step_count), os.path.join(root, "ref.pt"))
    else:
        eng.load(SaveLoadMeta(path=os.path.join(root, "ckpt"), weight_format="sharded", with_optim=True))
        ref = torch.load(os.path.join(root, "ref.pt"))
        assert eng.get_version() == 7 and eng.optimizer.step_count == ref["step_count"]
        assert torch.equal(eng.store.flat_param[: eng.store.numel], ref["param"])
        for k, t in (("master", eng.optimizer.master), ("exp_avg", eng.optimizer.exp_avg), ("exp_avg_sq", eng.optimizer.exp_avg_sq)):
            assert torch.equal(gather_full(eng, t), ref[k]), k
        st = eng.train_batch(batch(rank), loss_fn, lambda mb: mb["loss_mask"].count_nonzero())
        assert st["update_successful"] == 1.0
    print("RESHARD_OK", phase, rank, flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
