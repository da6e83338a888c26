"""Train engine with tensor parallelism and a sequence-parallel residual stream on 2 GPUs (``native:d1t2``, bf16):
the gather->GEMM / GEMM->reduce-scatter pairs as fused peer-memory kernels against the same engine on NCCL
collectives, and both against the all-reduce form of tensor parallelism; same seed, same batch. Prints
ENGINE_TP_SP_GPU_OK per rank."""
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
    for mode in ("allreduce", "sp_nccl", "sp_fused"):
        cfg = TrainEngineConfig(init_from_scratch=True, dtype="bfloat16" if on_gpu else "float32", backend=f"native:d1t{world}",
                                optimizer=OptimizerConfig(lr=1e-3, gradient_clipping=1.0), mb_spec=MicroBatchSpec(max_tokens_per_mb=512))
        cfg.fsdp.tp_sequence_parallel = mode != "allreduce"
        cfg.fsdp.fuse_tp_projections = mode == "sp_fused"
        eng = B200TrainEngine(cfg)
        eng.create_process_group()
        eng.initialize(model_config=mc, seed=5)
        assert eng.tp_size == world and getattr(eng.model, "tp_sequence_parallel", False) == (mode != "allreduce")
        assert (getattr(eng, "_tp_fused", None) is not None) == (mode == "sp_fused" and on_gpu)
        stats = [eng.train_batch(batch, loss_fn, weight_fn) for _ in range(3)]
        assert not on_gpu or oplib.kernel_error() == 0
        out[mode] = [(s["grad_norm"], s["loss"]) for s in stats]
        eng.destroy()
    tol = 3e-2 if on_gpu else 1e-4
    for mode in ("sp_nccl", "sp_fused"):
        for (g0, l0), (g1, l1) in zip(out["allreduce"], out[mode]):
            assert abs(g0 - g1) < tol * max(1.0, g0) and abs(l0 - l1) < tol * max(1.0, abs(l0)), out
    if rank == 0:
        print("(grad norm, loss) per step", out, flush=True)
    print("ENGINE_TP_SP_GPU_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
