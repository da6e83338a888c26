"""A vision-language model under Ulysses sequence parallelism over all ranks equals the single-rank engine: losses and
the parameter update of a few steps on a batch with pictures in two of four sequences. Prints VLM_SP_OK per rank."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ["AREAL_FORCE_CPU"] = "1"

import torch
import torch.distributed as dist

from areal_b200.api.alloc_mode import FSDPParallelStrategy
from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig
from areal_b200.engine.train_engine import B200TrainEngine
from areal_b200.models.config import preset
from tests.test_vlm import _vlm_batch


def loss_fn(logp, ent, mb):
    m = mb["loss_mask"].bool()
    return -(logp * m).sum() / m.sum().clamp(min=1)


def run(sp, rank, name):
    cfg = TrainEngineConfig(init_from_scratch=True, dtype="float32", optimizer=OptimizerConfig(type="sgd", lr=5e-2, weight_decay=0.0),
                            mb_spec=MicroBatchSpec(max_tokens_per_mb=256))
    eng = B200TrainEngine(cfg)
    if sp == 1:
        eng.set_train_ranks([rank], None)
    eng.create_process_group(FSDPParallelStrategy(data_parallel_size=1, context_parallel_size=sp) if sp > 1 else FSDPParallelStrategy())
    mc = preset(name)
    eng.initialize(model_config=mc, seed=3)
    batch = _vlm_batch(mc, eng.model.vcfg)
    p0 = eng.store.flat_param[: eng.store.numel].clone()
    stats = [eng.train_batch(dict(batch), loss_fn, lambda mb: mb["loss_mask"].count_nonzero()) for _ in range(2)]
    lp = eng.forward_batch(dict(batch))
    return [s["loss"] for s in stats], [s["grad_norm"] for s in stats], eng.store.flat_param[: eng.store.numel].clone() - p0, lp


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    for name in ("tiny-qwen2.5-vl", "tiny-qwen3-vl"):
        l2, g2, u2, lp2 = run(world, rank, name)
        l1, g1, u1, lp1 = run(1, rank, name)
        assert all(abs(a - b) < 1e-4 * max(1.0, abs(b)) for a, b in zip(l2, l1)), (name, l2, l1)
        assert all(abs(a - b) < 1e-3 * max(1.0, abs(b)) for a, b in zip(g2, g1)), (name, g2, g1)
        cos = float((u1 * u2).sum() / (u1.norm() * u2.norm()))
        assert cos > 0.9999 and float((u1 - u2).abs().max()) < 1e-4, (name, cos, float((u1 - u2).abs().max()))
        assert torch.allclose(lp1, lp2, atol=1e-4), (name, float((lp1 - lp2).abs().max()))
        if rank == 0:
            print(name, "losses", l2, "grad norms", g2, flush=True)
    print("VLM_SP_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
