"""Engine layouts that the CPU ranks verify in fp32, once more on 2 GPUs in bf16 over NCCL, each against a single-rank
engine (replicated parameters) on the same batch:

* ``sharded``   ``d2`` with ``fsdp.shard_parameters`` (ZeRO-3: asynchronous broadcasts / reductions on NCCL),
* ``hybrid-tp`` ``native:d1t2`` of a linear-attention (gated delta rule) model, heads of both mixers sliced,
* ``vlm-tp``    ``native:d1t2`` of a vision-language model, language model sliced, image tower whole;

and with 4 ranks (``LAYOUTS=ep-tp,ep-etp,pp-tp,pp-ep,sharded-tp``): whole experts over data x tensor ranks (``native:d2t2e2``), experts
sliced over the tensor-parallel group (``native:(attn:d2t2|ffn:e2t2)``), tensor parallelism inside pipeline stages
(``native:d1p2t2``), expert parallelism inside pipeline stages (``native:d2p2e2``), sharded parameters under tensor
parallelism (``d2t2`` with ``fsdp.shard_parameters``, a hybrid MoE model with a shared expert).

Prints ``LAYOUT_OK <name>`` per rank and layout, then ENGINE_LAYOUTS_GPU_OK."""
import faulthandler
import os
import sys

faulthandler.dump_traceback_later(280, exit=True)
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


def run(mc, batch, backend, on_gpu, rank, alone=False, shard=False, mine=None):
    cfg = TrainEngineConfig(init_from_scratch=True, dtype="bfloat16" if on_gpu else "float32", backend=backend,
                            optimizer=OptimizerConfig(lr=1e-3, gradient_clipping=1.0), mb_spec=MicroBatchSpec(max_tokens_per_mb=512))
    cfg.fsdp.shard_parameters = shard
    eng = B200TrainEngine(cfg)
    if alone:
        eng.set_train_ranks([rank])
    eng.create_process_group()
    eng.initialize(model_config=mc, seed=5)
    data = batch if mine is None else mine(eng)
    flat = lambda w: torch.cat([w[n].double().reshape(-1) for n in sorted(w)])      # noqa: E731
    before = flat(eng.export_weights())
    stats = [eng.train_batch(dict(data), loss_fn, weight_fn) for _ in range(3)]
    assert not on_gpu or oplib.kernel_error() == 0
    upd = flat(eng.export_weights()) - before
    eng.destroy()
    return [s["grad_norm"] for s in stats], upd


def compare(name, got, want, on_gpu, rank):
    (g1, v1), (g0, v0) = got, want
    tol = 3e-2 if on_gpu else 1e-3
    assert all(abs(a - b) < tol * max(1.0, b) for a, b in zip(g1, g0)), (name, g1, g0)
    # Adam's first steps turn a gradient near zero into a step of either sign, and bf16 runs differ in last bits: the
    # three-step updates are compared by direction and size
    cos = float((v1 * v0).sum() / (v1.norm() * v0.norm()).clamp(min=1e-30))
    ratio = float(v1.norm() / v0.norm().clamp(min=1e-30))
    assert float(v0.norm()) > 0 and cos > (0.95 if on_gpu else 0.9999) and abs(ratio - 1.0) < (0.1 if on_gpu else 1e-3), (name, cos, ratio)
    if rank == 0:
        print(f"{name}: grad norms {[round(x, 4) for x in g1]} vs {[round(x, 4) for x in g0]}; update cosine {cos:.5f}, size ratio {ratio:.4f}", flush=True)
    print(f"LAYOUT_OK {name}", flush=True)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    on_gpu = torch.cuda.is_available() and os.environ.get("AREAL_FORCE_CPU", "0") != "1"
    if on_gpu:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl" if on_gpu else "gloo")          # the gloo form is a dry run of the same script
    only = os.environ.get("LAYOUTS", "sharded,hybrid-tp,vlm-tp").split(",")
    if "sharded" in only:
        mc = preset("tiny-qwen3", num_layers=4)
        batch = make_batch(mc.vocab_size)
        half = lambda eng: {k: v[eng.dp_rank * 4:(eng.dp_rank + 1) * 4] for k, v in batch.items()}      # noqa: E731
        compare("sharded", run(mc, batch, f"d{world}", on_gpu, rank, shard=True, mine=half), run(mc, batch, "d1", on_gpu, rank, alone=True), on_gpu, rank)
    if "hybrid-tp" in only:
        mc = preset("tiny-qwen3.5")
        batch = make_batch(mc.vocab_size)
        compare("hybrid-tp", run(mc, batch, f"native:d1t{world}", on_gpu, rank), run(mc, batch, "d1", on_gpu, rank, alone=True), on_gpu, rank)
    if "vlm-tp" in only:
        from tests.test_vlm import _vlm_batch

        mc = preset("tiny-qwen3-vl")
        from areal_b200.models.vision import VisionConfig  # noqa: F401

        batch = _vlm_batch(mc, mc.vision_config())
        compare("vlm-tp", run(mc, batch, f"native:d1t{world}", on_gpu, rank), run(mc, batch, "d1", on_gpu, rank, alone=True), on_gpu, rank)
    four = {"ep-tp": ("tiny-qwen3-moe", "native:d2t2e2", False), "ep-etp": ("tiny-qwen3-moe", "native:(attn:d2t2|ffn:e2t2)", False),
            "pp-tp": ("tiny-qwen3", "native:d1p2t2", False), "pp-ep": ("tiny-qwen3-moe", "native:d2p2e2", False),
            "sharded-tp": ("tiny-qwen3.5-moe", "d2t2", True)}        # sharded parameters under tensor parallelism, shared expert sliced
    for name, (model, backend, shard) in four.items():
        if name in only:
            assert world == 4, "these layouts are written for 4 ranks"
            mc = preset(model)
            batch = make_batch(mc.vocab_size)
            share = lambda eng: {k: v[eng.dp_rank * (8 // eng.dp_size):(eng.dp_rank + 1) * (8 // eng.dp_size)] for k, v in batch.items()}   # noqa: E731
            compare(name, run(mc, batch, backend, on_gpu, rank, mine=share, shard=shard), run(mc, batch, "d1", on_gpu, rank, alone=True), on_gpu, rank)
    print("ENGINE_LAYOUTS_GPU_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
