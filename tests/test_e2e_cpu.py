"""End-to-end slices on CPU: colocated async GRPO, trainer/rollout split over gloo, HF
checkpoint round trip, recover, weight-push plan."""
import math
import os
import subprocess
import sys

import pytest
import torch

from areal_b200.api.cli_args import (ClusterSpecConfig, DatasetConfig, GenerationHyperparameters, GRPOConfig,
                                     InferenceEngineConfig, MicroBatchSpec, NormConfig, OptimizerConfig, PPOActorConfig,
                                     RecoverConfig, SaverConfig, StatsLoggerConfig)
from areal_b200.api.io_struct import SaveLoadMeta
from areal_b200.dataset import ArithmeticDataset, CharTokenizer
from areal_b200.engine.flat_params import FlatParamStore
from areal_b200.engine.train_engine import B200PPOActor
from areal_b200.models import hf_io
from areal_b200.models.config import ModelConfig, preset
from areal_b200.models.decoder import build_model
from areal_b200.parallel.weight_push import build_push_plan, tp_layout_of
from areal_b200.rollout.workflows.rlvr import RLVRWorkflow
from areal_b200.trainer.rl_trainer import PPOTrainer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def digit_reward(prompt, completion, prompt_ids, completion_ids, **kw):
    """Shaped reward that a random-init model can climb: fraction of generated ids < 10."""
    return sum(1 for t in completion_ids if t < 10) / max(1, len(completion_ids))


def _cfg(root, steps=None, recover="disabled"):
    return GRPOConfig(
        experiment_name="e2e", trial_name="t0", total_train_epochs=1, total_train_steps=steps, seed=1,
        cluster=ClusterSpecConfig(fileroot=root), train_dataset=DatasetConfig(batch_size=8),
        gconfig=GenerationHyperparameters(n_samples=4, max_new_tokens=8, max_tokens=64),
        rollout=InferenceEngineConfig(max_concurrent_rollouts=16, consumer_batch_size=8, max_head_offpolicyness=1,
                                      check_trajectory_format=True),
        actor=PPOActorConfig(init_from_scratch=True, dtype="float32", optimizer=OptimizerConfig(lr=3e-3),
                             mb_spec=MicroBatchSpec(max_tokens_per_mb=512), use_decoupled_loss=True, recompute_logprob=True,
                             kl_ctl=0.0, ppo_n_minibatches=1,
                             reward_norm=NormConfig(mean_level="group", std_level="group", group_size=4)),
        saver=SaverConfig(fileroot=root, experiment_name="e2e", trial_name="t0"),
        recover=RecoverConfig(mode=recover, fileroot=root, experiment_name="e2e", trial_name="t0", freq_steps=1),
        stats_logger=StatsLoggerConfig(fileroot=root, experiment_name="e2e", trial_name="t0"))


def test_colocated_async_grpo_learns_shaped_reward(tmp_path):
    cfg = _cfg(str(tmp_path), steps=12)
    mc = preset("tiny-qwen2", vocab_size=64, num_layers=2)
    tok = CharTokenizer()
    with PPOTrainer(cfg, ArithmeticDataset(size=128), tokenizer=None, model_config=mc) as tr:
        wf = RLVRWorkflow(digit_reward, cfg.gconfig, reward_in_process=True)
        hist = tr.train(workflow=wf)
    assert len(hist) == 12
    r = [h["ppo_actor/task_reward/avg"] for h in hist]
    assert all(h["ppo_actor/update/update_successful"] == 1.0 for h in hist)
    assert max(h.get("ppo_actor/update/staleness/avg", 0) for h in hist) <= 1.0 + 1e-6      # max_head_offpolicyness respected
    assert sum(r[-3:]) / 3 > sum(r[:3]) / 3 + 0.05, r                                       # the policy improved
    assert os.path.exists(os.path.join(str(tmp_path), "logs"))


def test_hybrid_linear_attention_actor_trains_and_rolls_out(tmp_path):
    """The gated-delta-rule / gated-attention stack through the whole loop: rollout (recompute
    path of the engine), log-prob recompute, PPO update, weight hand-over."""
    cfg = _cfg(str(tmp_path), steps=3)
    mc = preset("tiny-qwen3.5", vocab_size=64, num_layers=2, layer_types=["linear_attention", "full_attention"])
    with PPOTrainer(cfg, ArithmeticDataset(size=64), tokenizer=None, model_config=mc) as tr:
        hist = tr.train(workflow=RLVRWorkflow(digit_reward, cfg.gconfig, reward_in_process=True))
        names = [n for n, _ in tr.actor.model.named_parameters()]
    assert len(hist) == 3 and all(h["ppo_actor/update/update_successful"] == 1.0 for h in hist)
    assert all(math.isfinite(h["ppo_actor/update/grad_norm"]) for h in hist)
    assert "layers.0.linear_attn.A_log" in names and "layers.1.self_attn.q_proj" in names


def test_recover_resumes_from_checkpoint(tmp_path):
    mc = preset("tiny-qwen2", vocab_size=64, num_layers=2)
    cfg = _cfg(str(tmp_path), steps=2, recover="auto")
    with PPOTrainer(cfg, ArithmeticDataset(size=64), model_config=mc) as tr:
        tr.train(workflow=RLVRWorkflow(digit_reward, cfg.gconfig, reward_in_process=True))
        w_end = tr.actor.store.flat_param.clone()
    cfg2 = _cfg(str(tmp_path), steps=3, recover="auto")
    with PPOTrainer(cfg2, ArithmeticDataset(size=64), model_config=mc) as tr2:
        assert tr2.start_step == 2 and tr2.actor.get_version() == 2 and tr2.rollout.get_version() == 2
        assert torch.equal(tr2.actor.store.flat_param, w_end)
        assert tr2.actor.optimizer.step_count == 2
        hist = tr2.train(workflow=RLVRWorkflow(digit_reward, cfg2.gconfig, reward_in_process=True))
        assert len(hist) == 1


@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-qwen3", "tiny-qwen3-moe", "tiny-qwen3.5"])
def test_hf_checkpoint_roundtrip_and_names(tmp_path, name):
    cfg = preset(name)
    m = build_model(cfg, dtype=torch.float32, seed=2)
    hf_io.save_model_hf(m, str(tmp_path), max_shard_bytes=2_000_000)
    files = os.listdir(tmp_path)
    assert "config.json" in files and any(f.endswith(".safetensors") for f in files)
    names = {k for k, _ in hf_io.iter_safetensors(str(tmp_path))}
    if cfg.is_hybrid:
        assert {"model.layers.0.linear_attn.in_proj_qkv.weight", "model.layers.0.linear_attn.in_proj_a.weight", "model.layers.0.linear_attn.A_log",
                "model.layers.3.self_attn.q_proj.weight", "model.layers.3.self_attn.v_proj.weight"} <= names
    else:
        assert "model.layers.0.self_attn.q_proj.weight" in names
    assert "model.embed_tokens.weight" in names
    if cfg.is_moe:
        assert "model.layers.0.mlp.experts.3.up_proj.weight" in names and "model.layers.0.mlp.gate.weight" in names
    m2 = build_model(ModelConfig.from_pretrained(str(tmp_path)), dtype=torch.float32, seed=99)
    hf_io.load_model_hf(m2, str(tmp_path))
    for (n, a), (_, b) in zip(m.named_parameters(), m2.named_parameters()):
        assert torch.equal(a, b), n


def test_engine_save_load_hf_and_sharded(tmp_path):
    cfg = PPOActorConfig(init_from_scratch=True, dtype="float32", optimizer=OptimizerConfig(lr=1e-3))
    e = B200PPOActor(cfg); e.create_process_group(); e.initialize(model_config=preset("tiny-qwen3"), seed=4)
    e.optimizer.exp_avg.fill_(0.25); e.optimizer.step_count = 5; e.set_version(9)
    e.save(SaveLoadMeta(path=str(tmp_path / "hf"), weight_format="hf", with_optim=True))
    e.save(SaveLoadMeta(path=str(tmp_path / "sh"), weight_format="sharded", with_optim=True))
    f = B200PPOActor(cfg); f.create_process_group(); f.initialize(model_config=preset("tiny-qwen3"), seed=5)
    assert not torch.equal(f.store.flat_param, e.store.flat_param)
    f.load(SaveLoadMeta(path=str(tmp_path / "sh"), weight_format="sharded", with_optim=True))
    assert torch.equal(f.store.flat_param, e.store.flat_param) and f.optimizer.step_count == 5 and f.get_version() == 9
    assert float(f.optimizer.exp_avg[0]) == 0.25
    g = B200PPOActor(cfg); g.create_process_group(); g.initialize(model_config=preset("tiny-qwen3"), seed=6)
    g.load(SaveLoadMeta(path=str(tmp_path / "hf"), weight_format="hf", with_optim=True))
    assert torch.equal(g.store.flat_param[: g.store.numel], e.store.flat_param[: e.store.numel])


@pytest.mark.parametrize("tp,world", [(1, 3), (2, 4), (4, 2)])
def test_weight_push_plan_covers_every_tp_slice(tp, world):
    cfg = preset("tiny-qwen2", num_heads=4, num_kv_heads=4)
    stores = [FlatParamStore(build_model(cfg, dtype=torch.float32, seed=0), world, r, with_grads=False) for r in range(world)]
    st = stores[0]
    shapes = [tuple(p.shape) for p in st.params]
    dst_offsets, sizes = [], []
    for j in range(tp):
        d, o = {}, 0
        for n, sh in zip(st.names, shapes):
            d[n] = o
            C = sh[1] if len(sh) > 1 else 1
            R = int(torch.tensor(sh).prod()) // C
            o += sum((b[1] - b[0]) * (b[3] - b[2]) for b in tp_layout_of(cfg, n, (R, C), tp)[j])
        dst_offsets.append(d); sizes.append(o)
    dst = [torch.full((s,), float("nan")) for s in sizes]
    for r in range(world):
        for op in build_push_plan(cfg, st.names, st.offsets, shapes, stores[r].shard_range, tp, dst_offsets):
            for rr in range(op.rows):
                a, b = op.dst_off + rr * op.ld_dst, op.src_off + rr * op.ld_src
                assert torch.isnan(dst[op.dst_tp][a:a + op.cols]).all(), "element written twice"
                dst[op.dst_tp][a:a + op.cols] = st.flat_param[b:b + op.cols]
    for j in range(tp):
        for n, sh, p in zip(st.names, shapes, st.params):
            C = sh[1] if len(sh) > 1 else 1
            t = p.data.reshape(-1, C)
            exp = torch.cat([t[b[0]:b[1], b[2]:b[3]].reshape(-1) for b in tp_layout_of(cfg, n, (t.shape[0], C), tp)[j]])
            got = dst[j][dst_offsets[j][n]: dst_offsets[j][n] + exp.numel()]
            assert torch.equal(got, exp), (tp, j, n)


SPLIT_SCRIPT = r'''
import faulthandler, os, sys
faulthandler.dump_traceback_later(150, exit=True)
sys.path.insert(0, %(root)r)
os.environ["AREAL_FORCE_CPU"] = "1"
import torch, torch.distributed as dist
from tests.test_e2e_cpu import _cfg, digit_reward
from areal_b200.dataset import ArithmeticDataset
from areal_b200.models.config import preset
from areal_b200.rollout.workflows.rlvr import RLVRWorkflow
from areal_b200.infra.spmd import init_split_world, make_split_trainer, run_rollout_rank
cfg = _cfg(%(tmp)r)
if os.environ.get("SPLIT_DELTA") == "1":
    cfg.actor.enable_delta_weight_update = True           # sparse (index, value) pushes after the first full one
    cfg.actor.optimizer.lr = 1e-10                         # fp32 weights here: a step far below half an ulp leaves most bit patterns alone
mc = preset(os.environ.get("SPLIT_MODEL", "tiny-qwen2"), vocab_size=64, num_layers=2, **({"layer_types": ["linear_attention", "full_attention"]} if "qwen3.5" in os.environ.get("SPLIT_MODEL", "") else {}))
split, groups, bus = init_split_world(int(os.environ["N_TRAIN"]), None, sp=int(os.environ.get("SPLIT_SP", "1")), rollout_tp=int(os.environ.get("SPLIT_RTP", "1")))
ds = ArithmeticDataset(size=128)
if split.is_trainer:
    tr = make_split_trainer(cfg, mc, split, groups, bus, ds)
    h = tr.train(max_steps=3)
    assert len(h) == 3 and all(x["ppo_actor/update/update_successful"] == 1.0 for x in h)
    assert max(x.get("ppo_actor/update/staleness/avg", 0) for x in h) <= 1.0 + 1e-6
    ref = tr.actor.store.flat_param.clone()
    if groups["shard"] is not None:
        dist.broadcast(ref, src=0, group=groups["shard"])
        assert torch.equal(ref, tr.actor.store.flat_param), "trainer replicas diverged"
    if split.rank == 0:
        if os.environ.get("SPLIT_DELTA") == "1":
            p_ = tr.actor._weight_pusher
            assert p_.delta and p_.deltas_since_anchor == 3 and p_.last_fraction < 1.0, (p_.deltas_since_anchor, p_.last_fraction)
            print("DELTA_FRACTION", round(p_.last_fraction, 4), flush=True)
        bus.put("final_sum", float(tr.actor.store.flat_param.double().sum()))
        bus.put("exit", 1)
    tr.close()
else:
    wf = RLVRWorkflow(digit_reward, cfg.gconfig, reward_in_process=True)
    w = run_rollout_rank(cfg, mc, split, groups, bus, ds, wf, torch.device("cpu"))
    assert w.engine.get_version() == 3, w.engine.get_version()
    assert getattr(w, "delta_pushes", 0) == (3 if os.environ.get("SPLIT_DELTA") == "1" else 0)     # the start-up push is full, the three step pushes are deltas
    if split.rollout_tp == 1:
        got = float(w.flat_param.double().sum())
        assert abs(got - bus.get("final_sum")) < 1e-6, "rollout replica does not hold the trainer's final weights"
    else:
        # every rank of a tensor-parallel replica holds exactly its slices of the trainer's final weights
        from areal_b200.parallel import tp as TP
        st = w.staging
        for name, off, shape in zip(st["names"], st["offsets"], st["shapes"]):
            full = st["flat"][off:off + int(torch.tensor(shape).prod())].view(shape)
            mine = dict(w.engine.model.named_parameters())[name].data
            assert torch.equal(mine, TP.shard_tensor(mc, name, full, split.rollout_tp, split.tp_rank_of(split.rank))), name
        assert abs(float(st["flat"].double().sum()) - bus.get("final_sum")) < 1e-6
dist.barrier(group=groups["world_cpu"])
print("SPLIT_OK", split.rank, flush=True)
'''


@pytest.mark.parametrize("n_train,world,port,model,sp,rtp", [
    (1, 2, 29811, "tiny-qwen2", 1, 1), (2, 4, 29821, "tiny-qwen2", 1, 1), (1, 2, 29831, "tiny-qwen3.5", 1, 1),
    (2, 4, 29841, "tiny-qwen2", 2, 2),        # one Ulysses pair of trainers, one tensor-parallel rollout replica
    (2, 4, 29851, "tiny-qwen2", 1, 2),        # two data-parallel trainers share one tensor-parallel replica
    (1, 3, 29861, "tiny-qwen2", 1, 1),        # one trainer merges the batches of two replicas
    (4, 8, 29871, "tiny-qwen2", 4, 2),        # the 8-GPU benchmark layout: one Ulysses group of four trainers, two TP = 2 replicas
    (2, 4, 29881, "tiny-qwen2-delta", 1, 1),  # delta weight transfer: a full push, then (index, value) pairs of changed elements
    (2, 4, 29891, "tiny-qwen2-delta", 1, 2)]) # ... into the staging buffer of a tensor-parallel replica
def test_trainer_rollout_split_over_gloo(tmp_path, n_train, world, port, model, sp, rtp):
    script = tmp_path / "split.py"
    script.write_text(SPLIT_SCRIPT % dict(root=ROOT, tmp=str(tmp_path)))
    delta = model.endswith("-delta")
    model = model[: -len("-delta")] if delta else model
    env = dict(os.environ, N_TRAIN=str(n_train), OMP_NUM_THREADS="1", SPLIT_MODEL=model, SPLIT_SP=str(sp), SPLIT_RTP=str(rtp), SPLIT_DELTA="1" if delta else "0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("SPLIT_OK") == world


def test_moe_router_variants():
    """Sigmoid gates, group-limited choice, scaling, and the auxiliary-loss-free balancing bias."""
    import torch

    from areal_b200.models.config import preset
    from areal_b200.models.decoder import MoEMLP

    torch.manual_seed(0)
    cfg = preset("tiny-qwen3-moe", router_score_func="sigmoid", num_expert_groups=4, num_limited_groups=2, router_scale=2.5,
                 router_bias_update_rate=0.01, norm_topk_prob=True)
    m = MoEMLP(cfg, torch.float32, "cpu")
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    m.train()
    x = torch.randn(64, cfg.hidden_size)
    w, e, _ = m.route(x)
    assert w.shape == (64, 2) and e.shape == (64, 2)
    # weights: normalised sigmoid gates of the chosen experts times the scale
    probs = torch.sigmoid(x @ m.router.t())
    chosen = probs.gather(1, e)
    assert torch.allclose(w, chosen / chosen.sum(-1, keepdim=True) * 2.5, atol=1e-6)
    # group-limited: 8 experts in 4 groups of 2, both experts of a token come from at most 2 groups
    assert ((e // 2)[:, 0:1] != (e // 2)).sum(-1).max() <= 1
    best_groups = probs.view(64, 4, 2).sum(-1).topk(2, dim=-1).indices   # with a bias: groups ranked by their two best experts
    assert all(int(g) in best_groups[i].tolist() for i in range(64) for g in (e[i] // 2))
    # balancing: the load was recorded; the update moves the bias against it and keeps it centred
    assert m.tokens_per_expert.sum() == 128
    load = m.tokens_per_expert.clone()
    m.update_expert_bias()
    assert m.tokens_per_expert.sum() == 0 and abs(float(m.expert_bias.sum())) < 1e-6
    over, under = load.argmax(), load.argmin()
    if load[over] > load.mean() > load[under]:
        assert m.expert_bias[over] < m.expert_bias[under]
    # the bias changes the choice only, not the weights
    m.expert_bias[:] = 0
    m.expert_bias[3] = 10.0
    w2, e2, _ = m.route(x)
    assert (e2 == 3).any(dim=-1).float().mean() > 0.4   # expert 3 is picked whenever its group is among the chosen ones
    p2 = probs.gather(1, e2)
    assert torch.allclose(w2, p2 / p2.sum(-1, keepdim=True) * 2.5, atol=1e-6)
    y = m(x)
    assert y.shape == x.shape and torch.isfinite(y).all()
    y.sum().backward()
    assert m.router.grad is not None and torch.isfinite(m.router.grad).all()


PARALLEL_TRAINER_SCRIPT = r'''
import faulthandler, os, sys
faulthandler.dump_traceback_later(200, exit=True)
sys.path.insert(0, %(root)r)
os.environ["AREAL_FORCE_CPU"] = "1"
import torch, torch.distributed as dist
from tests.test_e2e_cpu import _cfg, digit_reward
from areal_b200.dataset import ArithmeticDataset
from areal_b200.models.config import preset
from areal_b200.rollout.workflows.rlvr import RLVRWorkflow
from areal_b200.trainer.rl_trainer import PPOTrainer
dist.init_process_group("gloo")
cfg = _cfg(%(tmp)r, steps=4)
cfg.actor.backend = %(backend)r
mc = preset(%(model)r, vocab_size=64, num_layers=2)
with PPOTrainer(cfg, ArithmeticDataset(size=128), tokenizer=None, model_config=mc) as tr:
    hist = tr.train(workflow=RLVRWorkflow(digit_reward, cfg.gconfig, reward_in_process=True))
    # the rollout engine holds exactly the trainer's (gathered) weights
    want = tr.actor.export_weights()
    got = dict(tr.rollout.model.named_parameters())
    assert set(want) == set(got)
    for n, t in want.items():
        assert torch.equal(t, got[n].detach().cpu()), n
assert len(hist) == 4
print("PARALLEL_TRAINER_OK", dist.get_rank(), flush=True)
dist.barrier()
'''


@pytest.mark.parametrize("backend,model,port", [("native:d1p2", "tiny-qwen2", 29955), ("native:d2e2", "tiny-qwen3-moe", 29953),
                                                ("d1t2", "tiny-qwen2", 29957)])
def test_ppo_trainer_with_model_parallel_actor(tmp_path, backend, model, port):
    """Whole GRPO loop on 2 gloo ranks with a pipeline- / expert- / tensor-parallel actor: every rank's
    rollout engine keeps a full model that the trainer feeds with gathered weights."""
    script = tmp_path / "par.py"
    script.write_text(PARALLEL_TRAINER_SCRIPT % dict(root=ROOT, tmp=str(tmp_path), backend=backend, model=model))
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("PARALLEL_TRAINER_OK") == 2


def test_hybrid_rollout_on_carried_state_matches_recompute():
    """The rollout engine advances linear-attention models on per-sequence state (rule state,
    convolution tail, keys / values of the full layers); greedy generations must equal those of
    the path that re-runs the whole packed forward every step."""
    import asyncio

    from areal_b200.api.io_struct import ModelRequest
    from areal_b200.api.cli_args import NativeInferConfig
    from areal_b200.engine.infer_engine import NativeInferenceEngine

    mc = preset("tiny-qwen3.5", vocab_size=64)
    outs = {}
    for mode in ("state", "recompute"):
        eng = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=3, context_length=128), model_config=mc)
        if mode == "recompute":
            eng._step_recurrent = eng._step_cpu
        eng.initialize(device="cpu", start_executor=False, seed=5)
        g = GenerationHyperparameters(n_samples=1, max_new_tokens=12, max_tokens=100, greedy=True, ignore_eos=True)

        async def run():
            reqs = [ModelRequest(rid=f"r{i}", input_ids=[3 + i, 7, 11 + i, 2, 5][: 2 + i], gconfig=g) for i in range(4)]
            return await asyncio.gather(*[eng.agenerate(r) for r in reqs])
        res = asyncio.run(run())
        outs[mode] = [(r.output_tokens, r.output_logprobs) for r in res]
        eng.destroy()
    for (ta, la), (tb, lb) in zip(outs["state"], outs["recompute"]):
        assert ta == tb
        assert max(abs(x - y) for x, y in zip(la, lb)) < 1e-4


def test_colocated_loop_runs_a_hundred_steps_within_the_staleness_bound(tmp_path):
    """The asynchronous loop left alone for 120 steps (several epochs of the dataset, per-sample
    response budgets, strict staleness): every step succeeds, no trained token is older than the
    configured bound although episodes finish out of order, the executor holds no finished
    trajectory back and its bookkeeping does not grow."""
    from areal_b200.dataset import RandomTokenDataset, small_id_fraction_reward_fn

    cfg = _cfg(str(tmp_path), steps=120)
    cfg.train_dataset.batch_size = 2
    cfg.rollout.consumer_batch_size, cfg.rollout.max_concurrent_rollouts, cfg.rollout.max_head_offpolicyness = 2, 6, 2
    cfg.rollout.strict_staleness = True
    cfg.gconfig = GenerationHyperparameters(n_samples=4, max_new_tokens=12, max_tokens=64, ignore_eos=True)
    mc = preset("tiny-qwen2", vocab_size=64, num_layers=1)
    ds = RandomTokenDataset(size=16, prompt_len=8, vocab_size=64, seed=3, median_len=6, max_len=12, min_len=2, n_samples=4)
    with PPOTrainer(cfg, ds, tokenizer=None, model_config=mc) as tr:
        wf = RLVRWorkflow(small_id_fraction_reward_fn, cfg.gconfig, reward_in_process=True)
        hist = tr.train(workflow=wf)
        ex = tr.rollout.workflow_executor
        assert len(ex._task_results) == 0 and len(ex._tracked) == 0
        assert len(ex._results) <= cfg.rollout.max_concurrent_rollouts
    assert len(hist) == 120 and all(h["ppo_actor/update/update_successful"] == 1.0 for h in hist)
    assert max(h["ppo_actor/update/staleness/max"] for h in hist) <= 2 + 1e-6
    lens = {round(h["ppo_actor/seq_len/avg"], 2) for h in hist}
    assert len(lens) > 5                                           # the samples of a group really have different lengths


@pytest.mark.parametrize("n_load", [1, 3])
def test_sharded_checkpoint_reloads_under_another_world_size(tmp_path, n_load):
    """A recovery checkpoint written by two data-parallel ranks is read back by one and by three: parameters, fp32
    master weights, both Adam moments, step count and version arrive bit for bit, and training carries on."""
    script = os.path.join(ROOT, "tests", "dist_scripts", "run_reshard_ckpt.py")
    for phase, n, port in (("save", 2, 29961), ("load", n_load, 29963 + n_load)):
        env = dict(os.environ, OMP_NUM_THREADS="1", CKPT_DIR=str(tmp_path), PHASE=phase)
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
                            "--master-port", str(port), script], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        assert r.stdout.count("RESHARD_OK") == n
