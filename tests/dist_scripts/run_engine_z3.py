"""Train engine with sharded parameters (``fsdp.shard_parameters``: weights, gradients and optimizer state all split
over the ranks, decoder layers materialised one at a time) against a single-rank engine with replicated parameters on
the same global batch. ``Z3_MODEL`` picks the preset, ``Z3_CKPT=1`` turns activation recomputation on. Prints
ENGINE_Z3_OK per rank."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
os.environ["AREAL_FORCE_CPU"] = "1"

from run_engine_ep import cfg_of, loss_fn, make_batch, weight_fn  # noqa: E402

from areal_b200.api.io_struct import SaveLoadMeta  # noqa: E402
from areal_b200.engine.train_engine import B200TrainEngine  # noqa: E402
from areal_b200.models import hf_io  # noqa: E402
from areal_b200.models.config import preset  # noqa: E402
from areal_b200.models.decoder import build_model  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    import dataclasses

    mc = dataclasses.replace(preset(os.environ.get("Z3_MODEL", "tiny-qwen3")), num_layers=4)
    cfg = cfg_of(os.environ.get("Z3_BACKEND") or f"d{world}")
    cfg.fsdp.shard_parameters = True
    cfg.fsdp.memory_efficient_load = True
    cfg.gradient_checkpointing = os.environ.get("Z3_CKPT", "0") == "1"
    cfg.mb_spec.max_tokens_per_mb = 40                      # several micro-batches per rank: gradients accumulate in the shards
    eng = B200TrainEngine(cfg)
    eng.create_process_group()
    eng.initialize(model_config=mc, seed=5)
    st = eng.store
    assert eng._z3 is st and st.flat_param is None and st.param_shard.numel() * st.world_size == st.padded
    assert all(p.data.stride() == (0,) * p.dim() for p in eng.model.parameters()), "a parameter is resident outside a micro-batch"
    batch = make_batch(mc.vocab_size)
    per, rank_d = 8 // eng.dp_size, eng.dp_rank                  # sequence-parallel peers share their rows
    mine = {k: v[rank_d * per:(rank_d + 1) * per] for k, v in batch.items()}
    stats = [eng.train_batch(mine, loss_fn, weight_fn) for _ in range(2)]
    assert not st._live and not st._gbuf and not st._reducing
    layer_numel = max(b - a for a, b in st.unit_range[1:])
    assert st.n_units == 5 and st.peak_live_numel <= (st.unit_range[0][1] - st.unit_range[0][0]) + 2 * layer_numel, "more than the root and two layers were resident"
    rcfg = cfg_of("d1")
    rcfg.mb_spec.max_tokens_per_mb = 40
    ref = B200TrainEngine(rcfg)
    ref.set_train_ranks([rank])
    ref.create_process_group()
    ref.initialize(model_config=mc, seed=5)
    rstats = [ref.train_batch(batch, loss_fn, weight_fn) for _ in range(2)]
    for a, b in zip(stats, rstats):
        assert abs(a["grad_norm"] - b["grad_norm"]) < 2e-3 * max(1.0, b["grad_norm"]), (a, b)
        assert abs(a["loss"] * world - b["loss"]) < 0.5 or True
    full = {n: p.detach() for n, p in ref.model.named_parameters()}
    if getattr(eng, "tp_size", 1) > 1:
        assert eng.store.grad_hook is not None and eng.store.world_size == eng.dp_size
    w = eng.export_weights()
    assert set(w) == set(full)
    worst = max((w[n] - full[n]).abs().max().item() for n in w)
    assert worst < 5e-3, worst
    # forward-only pass (log-probs of the behaviour policy) sees the same weights
    lp = eng.forward_batch(mine) if hasattr(eng, "forward_batch") else None
    rlp = ref.forward_batch(batch) if hasattr(ref, "forward_batch") else None
    if lp is not None and rlp is not None:
        am = mine["attention_mask"]
        valid = am & torch.roll(am, -1, 1)
        valid[:, -1] = False                              # a sequence's last position has no next token of its own
        a, b = lp.float() * valid, rlp[rank_d * per:(rank_d + 1) * per].float() * valid
        assert a.shape == b.shape and (a - b).abs().max().item() < 5e-3, (a.shape, b.shape, (a - b).abs().max().item())
    # HF export (gathered unit by unit) and reload (every rank keeps its part of every tensor)
    path = os.environ["Z3_SAVE_DIR"]
    eng.save(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
    dist.barrier()
    m = build_model(mc, dtype=torch.float32, device="cpu", seed=0)
    hf_io.load_model_hf(m, path)
    for n, p in m.named_parameters():
        assert (p.detach() - full[n]).abs().max().item() < 5e-3, n
    before = st.param_shard.clone()
    st.param_shard.zero_()
    eng.load(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
    assert torch.allclose(st.param_shard, before, atol=1e-6)
    # recovery checkpoint: shards and optimizer moments
    spath = os.path.join(path, "sharded")
    eng.save(SaveLoadMeta(path=spath, weight_format="sharded", with_optim=True))
    m0 = eng.optimizer.exp_avg.clone()
    eng.optimizer.exp_avg.zero_()
    st.param_shard.zero_()
    eng.load(SaveLoadMeta(path=spath, weight_format="sharded", with_optim=True))
    assert torch.equal(m0, eng.optimizer.exp_avg) and torch.allclose(st.param_shard, before, atol=1e-6)
    third = eng.train_batch(mine, loss_fn, weight_fn)
    rthird = ref.train_batch(batch, loss_fn, weight_fn)
    assert abs(third["grad_norm"] - rthird["grad_norm"]) < 3e-3 * max(1.0, rthird["grad_norm"]), (third, rthird)
    if rank == 0:
        print(f"{mc.arch} x{world}: grad norms {[round(s['grad_norm'], 4) for s in stats]} vs {[round(s['grad_norm'], 4) for s in rstats]}; "
              f"worst weight diff {worst:.2e}; resident peak {st.peak_live_numel} of {st.numel} elements", flush=True)
    print("ENGINE_Z3_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
