"""A vision-language model with a tensor-parallel language model (image tower whole on every rank) equals the
single-rank engine: losses, gradient norms, weights after two steps (gathered), forward-only log-probs. Prints
VLM_TP_OK per rank."""
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


def run(tp, rank, name):
    cfg = TrainEngineConfig(init_from_scratch=True, dtype="float32", optimizer=OptimizerConfig(type="sgd", lr=5e-2, weight_decay=0.0, gradient_clipping=1.0),
                            mb_spec=MicroBatchSpec(max_tokens_per_mb=256))
    eng = B200TrainEngine(cfg)
    if tp == 1:
        eng.set_train_ranks([rank], None)
    eng.create_process_group(FSDPParallelStrategy(data_parallel_size=1, tensor_parallel_size=tp) if tp > 1 else FSDPParallelStrategy())
    mc = preset(name)
    eng.initialize(model_config=mc, seed=3)
    batch = _vlm_batch(mc, eng.model.vcfg)
    stats = [eng.train_batch(dict(batch), loss_fn, lambda mb: mb["loss_mask"].count_nonzero()) for _ in range(2)]
    lp = eng.forward_batch(dict(batch))
    return [s["loss"] for s in stats], [s["grad_norm"] for s in stats], eng.export_weights(), lp


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    for name in ("tiny-qwen2.5-vl", "tiny-qwen3-vl"):
        l2, g2, w2, lp2 = run(world, rank, name)
        l1, g1, w1, lp1 = run(1, rank, name)
        assert all(abs(a - b) < 1e-4 * max(1.0, abs(b)) for a, b in zip(l2, l1)), (name, l2, l1)
        assert all(abs(a - b) < 1e-3 * max(1.0, abs(b)) for a, b in zip(g2, g1)), (name, g2, g1)
        assert set(w1) == set(w2)
        worst = max(float((w1[n] - w2[n]).abs().max()) for n in w1)
        assert worst < 1e-4, (name, worst)
        assert torch.allclose(lp1, lp2, atol=1e-4), (name, float((lp1 - lp2).abs().max()))
        if rank == 0:
            print(name, "losses", l2, "grad norms", g2, "worst weight diff", worst, flush=True)
    print("VLM_TP_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
