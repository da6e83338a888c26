"""Train engine with expert parallelism on 2 GPUs (``native:d2e2``, bf16): the fused peer-memory
dispatch / combine path against the NCCL all-to-all path of the same engine, same seed, same
batch. Prints ENGINE_EP_GPU_OK per rank."""
import faulthandler
import os
import sys

faulthandler.dump_traceback_later(240, exit=True)
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig
from areal_b200.engine.train_engine import B200TrainEngine
from areal_b200.models.config import preset
from areal_b200.ops import lib as oplib


def loss_fn(logp, ent, mb):
    m = mb["loss_mask"].bool()
    return -(logp * m).sum() / m.sum().clamp(min=1)


def weight_fn(mb):
    return mb["loss_mask"].count_nonzero()


def make_batch(vocab, rank):
    g = torch.Generator().manual_seed(11 + rank)
    B, L = 8, 192
    lens = torch.tensor([192, 90, 170, 120, 60, 75, 150, 181])
    am = torch.arange(L)[None] < lens[:, None]
    ids = torch.randint(0, vocab, (B, L), generator=g) * am
    lm = am.clone()
    lm[:, :3] = False
    lm[torch.arange(B), lens - 1] = False
    return dict(input_ids=ids, attention_mask=am, loss_mask=lm.int())


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    mc = preset("tiny-qwen3-moe")
    batch = make_batch(mc.vocab_size, rank)
    out = {}
    for label, flag in (("fused", "1"), ("library", "0")):
        os.environ["AREAL_EP_FUSED"] = flag
        cfg = TrainEngineConfig(init_from_scratch=True, dtype="bfloat16", backend=f"native:d{world}e2",
                                optimizer=OptimizerConfig(lr=1e-3, gradient_clipping=1.0), mb_spec=MicroBatchSpec(max_tokens_per_mb=1024))
        eng = B200TrainEngine(cfg)
        eng.create_process_group()
        eng.initialize(model_config=mc, seed=5)
        assert eng.ep_size == 2
        comm = getattr(eng.model, "ep_fused_comm", None)
        assert (comm is not None) == (label == "fused"), (label, comm)
        stats = [eng.train_batch(batch, loss_fn, weight_fn) for _ in range(3)]
        if label == "fused":
            calls = sum(l.mlp.ep_dispatcher.fused_calls for l in eng.model.layers if hasattr(l.mlp, "ep_dispatcher") and l.mlp.ep_dispatcher is not None)
            assert calls > 0, "the fused dispatch never ran"
        assert oplib.kernel_error() == 0
        out[label] = [(s["grad_norm"], s.get("loss", 0.0)) for s in stats]
        assert all(torch.isfinite(torch.tensor(g)) for g, _ in out[label]), out[label]
    for (ga, _), (gb, _) in zip(out["fused"], out["library"]):
        assert abs(ga - gb) < 0.05 * max(1.0, gb), (out["fused"], out["library"])
    if rank == 0:
        print("grad norms fused / library:", out, flush=True)
    print("ENGINE_EP_GPU_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
