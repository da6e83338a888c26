"""Parameter sharding (ZeRO-3): the store's arithmetic in one process, the engine on 2 and 4 gloo ranks."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_units_pieces_and_placeholders_single_process():
    import dataclasses

    from areal_b200.engine.sharded_params import ShardedParamStore, unit_of
    from areal_b200.models.config import preset
    from areal_b200.models.decoder import build_model

    assert unit_of("embed_tokens") == 0 and unit_of("norm") == 0 and unit_of("layers.0.mlp.down_proj") == 1 and unit_of("layers.11.input_layernorm") == 12
    mc = dataclasses.replace(preset("tiny-qwen3"), num_layers=3)
    m = build_model(mc, dtype=torch.float32, device="cpu", seed=1)
    want = {n: p.detach().clone() for n, p in m.named_parameters()}
    # four "ranks" built side by side over copies of the same model: together the shards hold every element once
    stores = []
    for r in range(4):
        mr = build_model(mc, dtype=torch.float32, device="cpu", seed=1)
        stores.append(ShardedParamStore(mr, 4, r, None, None, prefetch=False))
    st = stores[0]
    assert st.n_units == 4 and st.unit_range[0][0] == 0 and all(st.unit_range[u][1] == st.unit_range[u + 1][0] for u in range(3))
    assert st.unit_range[-1][1] <= st.padded and st.padded % 4 == 0
    flat = torch.cat([s.param_shard for s in stores])
    for n, t in want.items():
        off, numel = st.locate(n)
        assert torch.equal(flat[off:off + numel], t.reshape(-1)), n
    # every element of a unit has exactly one owner
    for u in range(st.n_units):
        a, b = st.unit_range[u]
        pcs = st._pieces(a, b)
        assert pcs[0][1] == a and pcs[-1][2] == b and all(x[2] == y[1] for x, y in zip(pcs, pcs[1:]))
        assert all(o * st.shard_numel <= lo < hi <= (o + 1) * st.shard_numel for o, lo, hi in pcs)
    # released parameters keep their shape, own no memory and read as NaN
    p = st.params[st.names.index("layers.1.mlp.down_proj")]
    assert p.shape == want["layers.1.mlp.down_proj"].shape and p.data.stride() == (0, 0) and torch.isnan(p.data).all()
    # piece-wise writes land where the whole tensor would
    name = "layers.2.mlp.gate_up_proj"
    full = torch.randn_like(want[name])
    half = full.shape[0] // 2
    for s in stores:
        s.write_piece(name, None, (0, half), full[:half])
        s.write_piece(name, None, (half, full.shape[0]), full[half:])
    off, numel = st.locate(name)
    assert torch.equal(torch.cat([s.param_shard for s in stores])[off:off + numel], full.reshape(-1))
    with pytest.raises(ValueError, match="shape mismatch"):
        st.write_piece(name, None, (0, half), full[: half - 1])


def test_one_rank_store_trains_like_the_replicated_store():
    """world size 1: the unit protocol alone (enter / leave around layers, gradients folded unit by unit)."""
    import dataclasses

    from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig
    from areal_b200.engine.train_engine import B200TrainEngine
    from areal_b200.models.config import preset

    os.environ["AREAL_FORCE_CPU"] = "1"
    mc = dataclasses.replace(preset("tiny-qwen3"), num_layers=3)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, mc.vocab_size, (4, 16), generator=g)
    batch = dict(input_ids=ids, attention_mask=torch.ones(4, 16, dtype=torch.bool), loss_mask=torch.ones(4, 16, dtype=torch.int32))

    def loss_fn(logp, ent, mb):
        m = mb["loss_mask"].bool()
        return -(logp * m).sum() / m.sum().clamp(min=1)

    out = []
    for shard, ckpt in ((False, False), (True, False), (True, True)):
        cfg = TrainEngineConfig(init_from_scratch=True, dtype="float32", backend="d1", optimizer=OptimizerConfig(lr=1e-2, gradient_clipping=1.0),
                                mb_spec=MicroBatchSpec(max_tokens_per_mb=32), gradient_checkpointing=ckpt)
        cfg.fsdp.shard_parameters = shard
        eng = B200TrainEngine(cfg)
        eng.create_process_group()
        eng.initialize(model_config=mc, seed=9)
        stats = [eng.train_batch(batch, loss_fn, lambda mb: mb["loss_mask"].count_nonzero()) for _ in range(2)]
        out.append((stats, eng.export_weights()))
    for stats, w in out[1:]:
        for a, b in zip(stats, out[0][0]):
            assert abs(a["grad_norm"] - b["grad_norm"]) < 1e-4 * max(1.0, b["grad_norm"]) and abs(a["loss"] - b["loss"]) < 1e-5
        assert set(w) == set(out[0][1]) and all(torch.allclose(w[n], out[0][1][n], atol=1e-5) for n in w)


@pytest.mark.parametrize("ranks,model,ckpt,backend,port", [(2, "tiny-qwen3", "0", "", 29961), (4, "tiny-qwen3", "1", "", 29963),
                                                         (2, "tiny-qwen3-moe", "1", "", 29965), (4, "tiny-qwen3", "1", "d2c2", 29967),
                                                         (4, "tiny-qwen3-moe", "1", "d2t2", 29969), (4, "tiny-qwen3.5", "0", "d2t2", 29971)])
def test_train_engine_with_sharded_parameters(tmp_path, ranks, model, ckpt, backend, port):
    """``fsdp.shard_parameters`` on gloo ranks against one rank with replicated parameters: gradient norm and weights
    after two steps over several micro-batches, at most the root and two layers resident at a time, forward-only pass,
    HF export / reload, recovery checkpoint; dense, MoE and linear-attention models, with and without recomputation, with
    Ulysses SP, and with tensor parallelism (every TP slice shards its weights over its data-parallel ranks; partial
    gradients of replicated parameters are summed over the TP group before a layer's gradients leave for their owners)."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1", Z3_SAVE_DIR=str(tmp_path), Z3_MODEL=model, Z3_CKPT=ckpt, Z3_BACKEND=backend)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "dist_scripts", "run_engine_z3.py")], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ENGINE_Z3_OK") == ranks


def test_colocated_grpo_loop_with_sharded_parameters(tmp_path):
    """The whole async GRPO loop on one CPU process with ``fsdp.shard_parameters``: the rollout engine keeps its own copy
    of the weights (the trainer's parameters exist only layer by layer), fed by the gathered tensors after every step."""
    os.environ["AREAL_FORCE_CPU"] = "1"
    from areal_b200.dataset import ArithmeticDataset
    from areal_b200.models.config import preset
    from areal_b200.rollout.workflows.rlvr import RLVRWorkflow
    from areal_b200.trainer import PPOTrainer
    from tests.test_e2e_cpu import _cfg, digit_reward

    cfg = _cfg(str(tmp_path), steps=5)
    cfg.actor.fsdp.shard_parameters = True
    mc = preset("tiny-qwen2", vocab_size=64, num_layers=2)
    with PPOTrainer(cfg, ArithmeticDataset(size=128), tokenizer=None, model_config=mc) as tr:
        assert tr.actor._z3 is not None and tr.rollout.model is not tr.actor.model
        hist = tr.train(workflow=RLVRWorkflow(digit_reward, cfg.gconfig, reward_in_process=True))
        assert tr.rollout.get_version() == 5
        # the engine's copy equals the trainer's gathered weights after the last update
        w = tr.actor.export_weights()
        for n, p in tr.rollout.model.named_parameters():
            assert torch.allclose(p.detach().float().cpu(), w[n].float(), atol=1e-6), n
    assert len(hist) == 5 and all(h["ppo_actor/update/update_successful"] == 1.0 for h in hist)


@pytest.mark.parametrize("name", ["tiny-qwen2.5-vl", "tiny-qwen3-vl"])
def test_vision_language_model_with_sharded_parameters(name):
    """The image tower belongs to the root unit (resident with the embedding for a micro-batch), the decoder layers come
    and go: two steps move the weights exactly as with replicated parameters."""
    os.environ["AREAL_FORCE_CPU"] = "1"
    from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig
    from areal_b200.engine.train_engine import B200TrainEngine
    from areal_b200.models.config import preset
    from tests.test_vlm import _vlm_batch

    def loss_fn(logp, ent, mb):
        m = mb["loss_mask"].bool()
        return -(logp * m).sum() / m.sum().clamp(min=1)

    res = []
    for shard in (False, True):
        cfg = TrainEngineConfig(init_from_scratch=True, dtype="float32", backend="d1", optimizer=OptimizerConfig(lr=1e-2, gradient_clipping=1.0),
                                mb_spec=MicroBatchSpec(max_tokens_per_mb=256))
        cfg.fsdp.shard_parameters = shard
        eng = B200TrainEngine(cfg)
        eng.create_process_group()
        mc = preset(name)
        eng.initialize(model_config=mc, seed=3)
        batch = _vlm_batch(mc, mc.vision_config())
        st = [eng.train_batch(dict(batch), loss_fn, lambda mb: mb["loss_mask"].count_nonzero()) for _ in range(2)]
        if shard:
            assert any(n.startswith("visual.") for n, u in zip(eng.store.names, eng.store.units_of) if u == 0)
        res.append(([s["grad_norm"] for s in st], eng.export_weights()))
    (g0, w0), (g1, w1) = res
    assert all(abs(a - b) < 1e-4 * max(1.0, a) for a, b in zip(g0, g1)) and all(torch.allclose(w0[n], w1[n], atol=1e-5) for n in w0)
