"""Train-engine parity: dp2 x pp2 (4 gloo ranks) against a single-rank engine on the same global
batch, for an untied and a tied-embedding model. Prints ENGINE_PP_OK per rank."""
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


def cfg_of(backend, vpp=1, schedule="1F1B"):
    # several micro-batches per rank so that the 1F1B schedule has warm-up, steady and cool-down phases
    c = TrainEngineConfig(init_from_scratch=True, dtype="float32", backend=backend, optimizer=OptimizerConfig(lr=1e-2, gradient_clipping=0.5),
                          mb_spec=MicroBatchSpec(max_tokens_per_mb=32))
    c.megatron.virtual_pipeline_parallel_size = vpp
    c.archon.pp_schedule = schedule
    return c


def check(mc, tag, vpp=1, schedule="1F1B", loss_rank=1, backend="native:d2p2"):
    rank = dist.get_rank()
    eng = B200TrainEngine(cfg_of(backend, vpp, schedule))
    eng.create_process_group()
    eng.initialize(model_config=mc, seed=5)
    if backend == "native:d2p2e2":
        assert (eng.dp_size, eng.pp_size, eng.ep_size) == (2, 2, 2) and eng.pp_rank == rank // 2 and eng.ep_rank == rank % 2 and eng.expert_store is not None
        assert eng.model.layers[0].mlp.w_gate_up.shape[0] == mc.num_experts // 2
    elif backend == "native:d2p2":
        assert (eng.dp_size, eng.pp_size) == (2, 2) and eng.pp_rank == rank // 2 and eng.dp_rank == rank % 2
        assert eng.is_data_parallel_head() == (rank < 2) and eng.current_data_parallel_head() == rank % 2
    else:       # d{1,2}p2t2: index = (stage * dp + d) * tp + t
        dp_ = eng.dp_size
        assert (eng.pp_size, eng.tp_size) == (2, 2) and eng.pp_rank == rank // (2 * dp_) and eng.tp_rank == rank % 2 and eng.dp_rank == (rank // 2) % dp_
        assert eng.is_data_parallel_head() == (rank in (0, 2)[:dp_]) and eng.current_data_parallel_head() == 2 * eng.dp_rank
        assert eng.model.layers[0].self_attn.qkv_proj.shape[0] * 2 == (mc.num_heads + 2 * mc.num_kv_heads) * mc.head_dim
    assert eng.is_pipeline_last_stage() == (eng.pp_rank == loss_rank)
    batch = make_batch(mc.vocab_size)
    d, per = eng.dp_rank, 8 // eng.dp_size
    mine = {k: v[d * per:(d + 1) * per] for k, v in batch.items()}
    stats = [eng.train_batch(mine, loss_fn, weight_fn) for _ in range(2)]
    ref = B200TrainEngine(cfg_of("d1"))
    ref.set_train_ranks([rank])
    ref.create_process_group()
    ref.initialize(model_config=mc, seed=5)
    rstats = [ref.train_batch(batch, loss_fn, weight_fn) for _ in range(2)]
    for a, b in zip(stats, rstats):
        assert abs(a["grad_norm"] - b["grad_norm"]) < 2e-3 * max(1.0, b["grad_norm"]), (tag, a, b)
    full = {n: p.detach() for n, p in ref.model.named_parameters()}
    worst = 0.0
    from areal_b200.parallel import tp as TP

    experts = {eng.model.native_name(n) for n in getattr(eng, "_expert_param_names", [])}
    for n, p in eng.model.named_native_parameters(skip_tied_copy=False):
        want = TP.shard_tensor(mc, n, full[n], getattr(eng, "tp_size", 1), getattr(eng, "tp_rank", 0))
        if n in experts:
            El = mc.num_experts // eng.ep_size
            want = want[eng.ep_rank * El:(eng.ep_rank + 1) * El]
        diff = (p.detach() - want).abs()
        worst = max(worst, diff.max().item())
        assert diff.mean().item() < 2e-5 and diff.max().item() < 5e-3, f"{tag}: weights diverged for {n}: max {diff.max().item()}"
    # forward-only outputs reach every stage and match the unsplit engine
    lp = eng.forward_batch(mine)
    lref = ref.forward_batch(batch)[d * per:(d + 1) * per]
    assert lp.shape == mine["input_ids"].shape, (lp.shape, mine["input_ids"].shape)
    # a sequence's last position is scored against its packing neighbour's first token: compare inside the loss mask
    err = ((lp - lref[:, : lp.shape[1]]).abs() * mine["loss_mask"]).max().item()
    assert err < 5e-3, (tag, err)
    ev = eng.eval_batch(mine, loss_fn, weight_fn)
    assert torch.isfinite(ev)
    # HF export: stages write their own tensors, one index
    path = os.path.join(os.environ["PP_SAVE_DIR"], tag)
    eng.save(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
    dist.barrier()
    m = build_model(mc, dtype=torch.float32, device="cpu", seed=0)
    hf_io.load_model_hf(m, path)
    for n, p in m.named_parameters():
        assert (p.detach() - full[n]).abs().max().item() < 5e-3, n
    # the complete weight dictionary for the rollout side, on every stage
    w = eng.export_weights()
    assert set(w) == set(full), (sorted(set(full) - set(w))[:3], sorted(set(w) - set(full))[:3])
    # reload into the stages
    eng.load(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
    if rank == 0:
        print(f"{tag}: grad norms {[round(s['grad_norm'], 4) for s in stats]} vs {[round(s['grad_norm'], 4) for s in rstats]}; "
              f"loss {stats[-1]['loss']:.4f}; worst weight diff {worst:.2e}", flush=True)
    dist.barrier()


def main():
    dist.init_process_group("gloo")
    if os.environ.get("PP_LAYOUT"):           # one layout on its own world size (8 ranks: 2 replicas x 2 stages x 2 slices)
        check(preset("tiny-qwen3", tie_word_embeddings=True), "pp-tp-dp", backend=os.environ["PP_LAYOUT"])
        print("ENGINE_PP_OK", flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return
    check(preset("tiny-qwen3"), "untied")
    check(preset("tiny-qwen3", tie_word_embeddings=True), "tied")
    check(preset("tiny-qwen3", tie_word_embeddings=True), "zero-bubble-tied", schedule="ZBH1")   # split backward, weight gradients deferred
    check(preset("tiny-qwen3", num_layers=4), "interleaved", vpp=2)            # 2 ranks x 2 chunks, one layer each
    check(preset("tiny-qwen3", num_layers=4, tie_word_embeddings=True), "interleaved-tied", vpp=2)
    # two chunks per rank placed in a V (rank 0 holds the first and the last stage, so the loss lives there), greedy order
    check(preset("tiny-qwen3", num_layers=4), "zbv", schedule="ZBV", loss_rank=0)
    check(preset("tiny-qwen3", num_layers=4, tie_word_embeddings=True), "zbv-tied", schedule="ZBV", loss_rank=0)
    # linear-attention (gated delta rule) layers in the stages, dense and MoE
    check(preset("tiny-qwen3.5"), "hybrid")
    check(preset("tiny-qwen3.5-moe"), "hybrid-moe", schedule="ZBH1")     # split backward with per-expert weight views
    check(preset("tiny-qwen3-moe"), "moe-zbh1", schedule="ZBH1")
    # expert parallelism inside the stages: each stage's experts spread over its two data-parallel ranks
    check(preset("tiny-qwen3-moe"), "pp-ep", backend="native:d2p2e2")
    check(preset("tiny-qwen3-moe"), "pp-ep-zbh1", schedule="ZBH1", backend="native:d2p2e2")
    # tensor parallelism inside the stages: 2 stages x 2 slices
    check(preset("tiny-qwen3"), "pp-tp", backend="native:d1p2t2")
    check(preset("tiny-qwen3", tie_word_embeddings=True), "pp-tp-tied-zbh1", schedule="ZBH1", backend="native:d1p2t2")
    check(preset("tiny-qwen3", num_layers=4, tie_word_embeddings=True), "pp-tp-interleaved", vpp=2, backend="native:d1p2t2")
    print("ENGINE_PP_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
