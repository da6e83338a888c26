"""Train engine with pipeline parallelism on 2 GPUs (``native:d1p2``, bf16): the split-backward
ZBH1 schedule (input gradients first, weight-gradient GEMMs deferred into the exchange) against
plain 1F1B, and the ZBV schedule (two chunks per rank in a V, loss on rank 0), same seed, same batch. Prints ENGINE_PP_GPU_OK per rank."""
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


def make_batch(vocab):
    g = torch.Generator().manual_seed(11)
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
    on_gpu = torch.cuda.is_available() and os.environ.get("AREAL_FORCE_CPU", "0") != "1"
    if on_gpu:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl" if on_gpu else "gloo")          # the gloo form is a dry run of the same script
    mc = preset("tiny-qwen3", num_layers=4)
    batch = make_batch(mc.vocab_size)
    out = {}
    for sched in ("1F1B", "ZBH1", "ZBV"):
        cfg = TrainEngineConfig(init_from_scratch=True, dtype="bfloat16" if on_gpu else "float32", backend=f"native:d1p{world}",
                                optimizer=OptimizerConfig(lr=1e-3, gradient_clipping=1.0), mb_spec=MicroBatchSpec(max_tokens_per_mb=256))
        cfg.archon.pp_schedule = sched
        eng = B200TrainEngine(cfg)
        eng.create_process_group()
        eng.initialize(model_config=mc, seed=5)
        assert eng.pp_size == world and eng._pp_runner.schedule == sched
        assert eng.is_pipeline_last_stage() == (eng.pp_rank == (0 if sched == "ZBV" else world - 1))
        stats = [eng.train_batch(batch, loss_fn, weight_fn) for _ in range(3)]
        assert not on_gpu or oplib.kernel_error() == 0
        out[sched] = [s["grad_norm"] for s in stats]
    for a, b in zip(out["1F1B"], out["ZBH1"]):
        assert abs(a - b) < 1e-3 * max(1.0, a), out
    for a, b in zip(out["1F1B"], out["ZBV"]):          # other chunk boundaries, same model: bf16 rounding apart
        assert abs(a - b) < 2e-2 * max(1.0, a), out
    if rank == 0:
        print("grad norms", out, flush=True)
    print("ENGINE_PP_GPU_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
