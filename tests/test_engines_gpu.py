"""GPU parity of the train engine and the rollout engine against the CPU reference path."""
import asyncio

import pytest
import torch

from areal_b200.api.cli_args import (GenerationHyperparameters, InferenceEngineConfig, MicroBatchSpec, NativeInferConfig,
                                     OptimizerConfig, PPOActorConfig)
from areal_b200.api.io_struct import ModelRequest
from areal_b200.engine.infer_engine import NativeInferenceEngine
from areal_b200.engine.train_engine import B200PPOActor
from areal_b200.models.config import preset
from areal_b200.models.decoder import build_model
from areal_b200.ops import lib as oplib

pytestmark = pytest.mark.gpu


def _batch(B=6, L=300, V=1024, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, V, (B, L), generator=g)
    am = torch.ones(B, L, dtype=torch.bool)
    for i in range(B):
        am[i, L - 37 * i:] = False if i else True
    lm = torch.zeros(B, L, dtype=torch.int32)
    lm[:, 40:] = 1
    lm = lm * am
    return dict(input_ids=ids, attention_mask=am, loss_mask=lm, logprobs=torch.full((B, L), -6.9),
                versions=torch.zeros(B, L, dtype=torch.int32), rewards=torch.randn(B, generator=g))


@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-qwen3", "tiny-qwen3-moe", "tiny-qwen3.5"])
def test_forward_logprob_parity_with_cpu(name):
    cfg = preset(name)
    ref = build_model(cfg, dtype=torch.float32, device="cpu", seed=3)
    gpu = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=3)
    with torch.no_grad():
        for (n, p), (_, q) in zip(gpu.named_parameters(), ref.named_parameters()):
            q.copy_(p.float().cpu())  # identical (bf16-rounded) weights
    ids = torch.randint(0, cfg.vocab_size, (700,))
    cu = torch.tensor([0, 130, 450, 700], dtype=torch.int32)
    labels = torch.roll(ids, -1)
    with torch.no_grad():
        h_ref = ref(ids, cu)
        lp_ref, ent_ref = ref.logprobs_entropy(h_ref, labels)
        pad = torch.zeros(768 - 700, dtype=torch.long)
        ids_g = torch.cat([ids, pad]).cuda().int()
        cu_g = torch.tensor([0, 130, 450, 700, 768], dtype=torch.int32, device="cuda")
        h = gpu(ids_g, cu_g)
        lp, ent = gpu.logprobs_entropy(h, torch.roll(ids_g, -1))
    assert oplib.kernel_error() == 0
    d_lp = (lp[:699].float().cpu() - lp_ref[:699]).abs()
    d_ent = (ent[:699].float().cpu() - ent_ref[:699]).abs()
    if cfg.is_moe:
        # a near-tie in the router may pick a different expert in bf16: compare the bulk, not the worst token
        assert d_lp.median().item() < 0.02 and d_lp.mean().item() < 0.05
        assert d_ent.mean().item() < 0.05
    else:
        assert d_lp.max().item() < 0.08
        assert d_ent.max().item() < 0.08


def test_train_step_matches_cpu_engine():
    def make(dtype, force_cpu):
        cfg = PPOActorConfig(init_from_scratch=True, dtype=dtype, optimizer=OptimizerConfig(lr=1e-3, gradient_clipping=1.0),
                             mb_spec=MicroBatchSpec(max_tokens_per_mb=1024), use_decoupled_loss=True, recompute_logprob=True,
                             kl_ctl=0.0, ppo_n_minibatches=1, gradient_checkpointing=True)
        e = B200PPOActor(cfg)
        if force_cpu:
            import os
            os.environ["AREAL_FORCE_CPU"] = "1"
        try:
            e.create_process_group()
        finally:
            if force_cpu:
                os.environ.pop("AREAL_FORCE_CPU")
        e.initialize(model_config=preset("tiny-qwen3"), seed=5)
        return e

    g, c = make("bfloat16", False), make("float32", True)
    assert g.device.type == "cuda" and c.device.type == "cpu"
    with torch.no_grad():
        c.store.flat_param.copy_(g.store.flat_param.float().cpu())
        c.optimizer.resync_master()
        g.optimizer.resync_master()
    outs = []
    for e in (g, c):
        data = _batch()
        data["prox_logp"] = e.compute_logp(data)
        e.compute_advantages(data)
        st = e.ppo_update(data)[0]
        outs.append((data["prox_logp"], st))
    (pg, sg), (pc, sc) = outs
    assert oplib.kernel_error() == 0
    valid = torch.roll(_batch()["loss_mask"], -1, 1).bool()  # positions whose label is a real next token
    valid[:, -1] = False
    assert (pg - pc).abs()[valid].max().item() < 0.1
    assert abs(sg["grad_norm"] - sc["grad_norm"]) / max(sc["grad_norm"], 1e-6) < 0.1
    # parameters moved the same way
    dg = g.store.flat_param.float().cpu()
    dc = c.store.flat_param
    assert ((dg - dc).norm() / dc.norm()).item() < 2e-2


def test_rollout_engine_greedy_matches_cpu():
    cfg = preset("tiny-qwen3")
    gpu_model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=11)
    cpu_model = build_model(cfg, dtype=torch.float32, device="cpu", seed=11)
    with torch.no_grad():
        for (n, p), (_, q) in zip(gpu_model.named_parameters(), cpu_model.named_parameters()):
            q.copy_(p.float().cpu())
    ic = NativeInferConfig(max_running_requests=8, page_size=16, context_length=512)
    ic.num_pages = 256
    eg = NativeInferenceEngine(InferenceEngineConfig(), ic, model=gpu_model, eos_token_id=None).initialize(
        device="cuda", start_executor=False)
    ec = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=8), model=cpu_model,
                               eos_token_id=None).initialize(device="cpu", start_executor=False)
    g = GenerationHyperparameters(max_new_tokens=24, max_tokens=400, greedy=True)
    prompts = [list(range(5 + i, 40 + 3 * i)) for i in range(5)]

    async def run(e):
        return await asyncio.gather(*[e.agenerate(ModelRequest(input_ids=p, gconfig=g)) for p in prompts])

    rg, rc = asyncio.run(run(eg)), asyncio.run(run(ec))
    eg.destroy(); ec.destroy()
    assert oplib.kernel_error() == 0
    agree = 0
    total = 0
    for a, b in zip(rg, rc):
        assert len(a.output_tokens) == 24 and len(a.output_logprobs) == 24
        # random-init logits are nearly flat, so bf16 noise may flip an argmax; compare prefixes
        for x, y in zip(a.output_tokens, b.output_tokens):
            total += 1
            if x != y:
                break
            agree += 1
        assert abs(a.output_logprobs[0] - b.output_logprobs[0]) < 0.1
    assert agree >= 0.5 * total


def test_hybrid_model_rolls_out_on_carried_state_on_gpu():
    """Linear-attention stack on the GPU rollout engine: prompts absorbed by a packed forward, then one
    token per step on per-sequence state; the first log-prob matches the fp32 CPU engine and the
    generated log-probs match a packed forward of the finished sequences on the same GPU model."""
    cfg = preset("tiny-qwen3.5")
    gpu_model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=11)
    cpu_model = build_model(cfg, dtype=torch.float32, device="cpu", seed=11)
    with torch.no_grad():
        for (n, p), (_, q) in zip(gpu_model.named_parameters(), cpu_model.named_parameters()):
            q.copy_(p.float().cpu())
    mk = lambda m, dev: NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=3, context_length=256),  # noqa: E731
                                              model=m, eos_token_id=None).initialize(device=dev, start_executor=False)
    eg, ec = mk(gpu_model, "cuda"), mk(cpu_model, "cpu")
    g = GenerationHyperparameters(max_new_tokens=10, max_tokens=200, greedy=True)
    prompts = [list(range(5 + i, 20 + 9 * i)) for i in range(4)]

    async def run(e):
        return await asyncio.gather(*[e.agenerate(ModelRequest(input_ids=p, gconfig=g)) for p in prompts])

    rg, rc = asyncio.run(run(eg)), asyncio.run(run(ec))
    eg.destroy(); ec.destroy()
    for p, a, b in zip(prompts, rg, rc):
        assert len(a.output_tokens) == 10
        assert abs(a.output_logprobs[0] - b.output_logprobs[0]) < 0.1
        ids = torch.tensor(p + a.output_tokens, device="cuda")
        cu = torch.tensor([0, ids.numel()], dtype=torch.int32, device="cuda")
        with torch.no_grad():
            lp, _ = gpu_model.logprobs_entropy(gpu_model(ids, cu, max_seqlen=ids.numel()), torch.roll(ids, -1))
        got = torch.tensor(a.output_logprobs)
        want = lp[len(p) - 1: len(p) - 1 + 10].float().cpu()
        assert (got - want).abs().max().item() < 0.1, (got - want).abs().max().item()


def test_rollout_engine_sampling_logprobs_consistent_with_trainer():
    """Behaviour log-probs reported by the rollout engine match a trainer-side recompute."""
    cfg = preset("tiny-qwen3")
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=13)
    ic = NativeInferConfig(max_running_requests=16, page_size=16, context_length=512)
    ic.num_pages = 512
    e = NativeInferenceEngine(InferenceEngineConfig(), ic, model=model).initialize(device="cuda", start_executor=False)
    g = GenerationHyperparameters(max_new_tokens=40, max_tokens=400, temperature=1.0)

    async def run():
        return await asyncio.gather(*[e.agenerate(ModelRequest(input_ids=list(range(3 + i, 60 + i)), gconfig=g)) for i in range(12)])

    rs = asyncio.run(run())
    e.destroy()
    worst = 0.0
    for r in rs:
        seq = r.input_tokens + r.output_tokens
        T = len(seq)
        Tp = (T + 127) // 128 * 128
        ids = torch.tensor(seq + [0] * (Tp - T), dtype=torch.int32, device="cuda")
        cu = torch.tensor([0, T] + ([Tp] if Tp > T else []), dtype=torch.int32, device="cuda")
        with torch.no_grad():
            h = model(ids, cu)
            lp, _ = model.logprobs_entropy(h, torch.roll(ids, -1))
        got = torch.tensor(r.output_logprobs)
        ref = lp[len(r.input_tokens) - 1: T - 1].float().cpu()
        worst = max(worst, (got - ref).abs().max().item())
    assert oplib.kernel_error() == 0
    assert worst < 0.1, worst


DECODE_SWITCH_SCRIPT = r'''
import asyncio, json, sys
sys.path.insert(0, %(root)r)
import torch
from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeInferConfig
from areal_b200.api.io_struct import ModelRequest
from areal_b200.engine.infer_engine import NativeInferenceEngine
from areal_b200.models.config import preset
from areal_b200.ops import lib as oplib
mc = preset("qwen2.5-1.5b", num_layers=2, vocab_size=4096)
eng = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=8, context_length=256, mem_fraction_static=0.1), model_config=mc)
eng.initialize(seed=11, start_executor=False)
g = torch.Generator().manual_seed(0)
reqs = [ModelRequest(rid=f"r{i}", input_ids=torch.randint(0, 4096, (24 + 5 * i,), generator=g).tolist(),
                     gconfig=GenerationHyperparameters(max_new_tokens=12, max_tokens=200, greedy=True, ignore_eos=True)) for i in range(6)]
async def run():
    return await asyncio.gather(*[eng.agenerate(r) for r in reqs])
out = asyncio.run(run())
torch.cuda.synchronize()
print("RESULT " + json.dumps({"tokens": [o.output_tokens for o in out], "logp": [o.output_logprobs for o in out], "err": oplib.kernel_error()}))
eng.destroy()
'''


def test_decode_switches_agree_with_default(tmp_path):
    """The optional decode paths (split-K GEMMs, programmatic dependent launch) generate what the
    default path generates: same first-token log-probs, (almost) the same greedy tokens."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "gen.py"
    script.write_text(DECODE_SWITCH_SCRIPT % dict(root=root))

    def run(env_extra):
        env = dict(os.environ)
        env.update(env_extra)
        r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=300, env=env, cwd=root)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
        line = next(l for l in r.stdout.splitlines() if l.startswith("RESULT "))
        return json.loads(line[7:])

    base = run({"AB2_DECODE_SPLITK": "0", "AB2_PDL": "0"})
    assert base["err"] == 0
    for extra in ({"AB2_PDL": "1"}, {"AB2_DECODE_SPLITK": "1"}, {"AB2_DECODE_SPLITK": "1", "AB2_PDL": "1"}):
        got = run({"AB2_DECODE_SPLITK": "0", "AB2_PDL": "0", **extra})
        assert got["err"] == 0
        # random-init logits are nearly flat: a different summation order may flip an argmax, after which the
        # sequence diverges for good, so count agreement up to the first difference
        same = total = 0
        for ta, tb in zip(base["tokens"], got["tokens"]):
            total += len(ta)
            for a, b in zip(ta, tb):
                if a != b:
                    break
                same += 1
        assert same >= 0.5 * total, (extra, same, total)
        first = max(abs(a[0] - b[0]) for a, b in zip(base["logp"], got["logp"]))
        assert first < 0.05, (extra, first)
        if extra == {"AB2_PDL": "1"}:                      # same arithmetic, only the launch differs
            assert got["tokens"] == base["tokens"]


@pytest.mark.parametrize("prompt_len", [64, 75])       # whole pages only / a partial last page
def test_prefix_sharing_reuses_prompt_pages_and_matches_plain_engine(prompt_len):
    """Requests with the same prompt: one prefetch, shared full pages, first token sampled from the
    stored logits; greedy outputs equal those of an engine without sharing, and every page returns
    to the pool afterwards. A weight-version change invalidates the stored prompts."""
    cfg = preset("tiny-qwen3")
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=11)

    def engine(share):
        ic = NativeInferConfig(max_running_requests=8, page_size=16, context_length=512, enable_prefix_sharing=share)
        ic.num_pages = 256
        return NativeInferenceEngine(InferenceEngineConfig(), ic, model=model, eos_token_id=None).initialize(device="cuda", start_executor=False)

    g = GenerationHyperparameters(max_new_tokens=20, max_tokens=400, greedy=True, ignore_eos=True)
    shared = list(range(7, 7 + prompt_len))
    other = list(range(100, 100 + prompt_len - 3))
    prompts = [shared, shared, other, shared, shared]

    async def run(e):
        return await asyncio.gather(*[e.agenerate(ModelRequest(rid=f"r{i}", input_ids=p, gconfig=g)) for i, p in enumerate(prompts)])

    plain = engine(False)
    want = asyncio.run(run(plain))
    plain.destroy()
    eng = engine(True)
    got = asyncio.run(run(eng))
    assert oplib.kernel_error() == 0
    for a, b in zip(want, got):
        assert a.output_tokens == b.output_tokens
        assert max(abs(x - y) for x, y in zip(a.output_logprobs, b.output_logprobs)) < 1e-3
    assert eng.stats["prefix_hits"] == 3 and eng.stats["prefix_tokens_saved"] == 3 * prompt_len
    assert eng.stats["prefill_tokens"] == prompt_len + len(other)
    # only the cache's own references remain: the two prompts' full pages (+ a copy of each partial last page)
    held = sum(len(e["pages"]) + (e["tail_page"] is not None) for e in eng._prefix.values())
    assert len(eng.cache.free) == eng.cache.num_pages - held and held == 2 * (prompt_len // 16) + 2 * (prompt_len % 16 > 0)
    again = asyncio.run(run(eng))                                   # now all five prompts are cached
    assert [r.output_tokens for r in again] == [r.output_tokens for r in want] and eng.stats["prefix_hits"] == 8
    eng.set_version(3)                                              # new weights: stored prompts are stale
    asyncio.run(run(eng))
    assert eng.stats["prefix_hits"] == 8 + 3 and all(e["version"] == 3 for e in eng._prefix.values())
    eng.destroy()


@pytest.mark.parametrize("reserve_full", [True, False])
def test_prefix_eviction_under_page_pressure_keeps_rows_and_pages_consistent(reserve_full):
    """A page pool too small for the stored prompts plus the running sequences: stored prompts get
    evicted between the admission of a sequence that counted on them and its start. Such a sequence
    goes back to the waiting queue and must not also take a decode row (it used to: every such
    event leaked one row and left a page-less sequence in the decode batch). Many groups of
    identical prompts run through such a pool; outputs equal those of a roomy engine and every row
    and page is back afterwards."""
    cfg = preset("tiny-qwen3")
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=5)

    def engine(num_pages, share=True):
        ic = NativeInferConfig(max_running_requests=8, page_size=16, context_length=256, enable_prefix_sharing=share,
                               reserve_full_length=reserve_full)
        ic.num_pages = num_pages
        return NativeInferenceEngine(InferenceEngineConfig(), ic, model=model, eos_token_id=None).initialize(device="cuda", start_executor=False)

    g = GenerationHyperparameters(max_new_tokens=24, max_tokens=200, greedy=True, ignore_eos=True)
    prompts = [[(7 * k + i) % 1000 + 3 for i in range(40 + k)] for k in range(12)]      # 12 different prompts
    reqs = [(k, j) for k in range(12) for j in range(4)]                               # groups of 4

    async def run(e):
        return await asyncio.gather(*[e.agenerate(ModelRequest(rid=f"r{k}_{j}", input_ids=prompts[k], gconfig=g)) for k, j in reqs])

    roomy = engine(512, share=False)
    want = asyncio.run(run(roomy))
    roomy.destroy()
    # 8 running sequences need 8 * ceil((51 + 24) / 16) = 40 pages; 44 leaves next to nothing for stored prompts
    tight = engine(44)
    for _ in range(3):
        got = asyncio.run(run(tight))
        assert [r.output_tokens for r in got] == [r.output_tokens for r in want]
    assert oplib.kernel_error() == 0
    assert sorted(tight._rows_free) == list(range(tight.max_batch)) and all(s is None for s in tight._row_seq)
    held = sum(len(e["pages"]) + (e["tail_page"] is not None) for e in tight._prefix.values())
    assert len(tight.cache.free) == tight.cache.num_pages - held
    tight.destroy()


def test_on_demand_pages_preempt_and_resume_when_the_pool_runs_dry():
    """Pages are taken as sequences grow. A pool that cannot hold every running sequence at full
    length forces pre-emptions: the victim returns its partial output, its client resubmits it and
    the generation continues after a new prefetch. Every request still delivers exactly its budget
    of tokens with finite log-probs, and all rows and pages are back afterwards."""
    cfg = preset("tiny-qwen3")
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=9)
    ic = NativeInferConfig(max_running_requests=8, page_size=16, context_length=256, enable_prefix_sharing=False)
    ic.num_pages = 30                       # 8 sequences x ceil((20 + 100) / 16) = 64 pages would be needed at full length
    eng = NativeInferenceEngine(InferenceEngineConfig(), ic, model=model, eos_token_id=None).initialize(device="cuda", start_executor=False)
    g = GenerationHyperparameters(max_new_tokens=100, max_tokens=200, greedy=False, temperature=1.0, ignore_eos=True)

    async def run():
        return await asyncio.gather(*[eng.agenerate(ModelRequest(rid=f"p{i}", input_ids=[(11 * i + j) % 900 + 5 for j in range(20)], gconfig=g))
                                      for i in range(12)])

    outs = asyncio.run(run())
    assert oplib.kernel_error() == 0
    assert eng.stats["preempted"] > 0
    for o in outs:
        assert len(o.output_tokens) == 100 and len(o.output_logprobs) == 100 and o.stop_reason == "length"
        assert all(lp <= 0 and lp > -50 for lp in o.output_logprobs)
    assert sorted(eng._rows_free) == list(range(eng.max_batch)) and len(eng.cache.free) == eng.cache.num_pages
    eng.destroy()


def _tiny_actor(**opt_kw):
    cfg = PPOActorConfig(init_from_scratch=True, dtype="bfloat16", optimizer=OptimizerConfig(lr=1e-4, **opt_kw),
                         mb_spec=MicroBatchSpec(max_tokens_per_mb=1024), use_decoupled_loss=True, recompute_logprob=True,
                         kl_ctl=0.0, ppo_n_minibatches=1)
    eng = B200PPOActor(cfg)
    eng.create_process_group()
    eng.initialize(model_config=preset("tiny-qwen3"), seed=1)
    return eng


def test_optimizer_step_raises_when_a_device_wait_gave_up():
    """A bounded wait that ran out anywhere before the optimizer step (here: a tensor-parallel
    consumer whose peer never produced, limit 50 ms) must not be silent: the step reads the device
    error word with its own status read and raises; the next step is clean again."""
    from areal_b200.parallel.tp_decode import TPDecodeExchange

    eng = _tiny_actor()
    data = _batch()
    data["prox_logp"] = eng.compute_logp(data)
    eng.compute_advantages(data)
    eng.ppo_update(dict(data))                               # a normal step first (the update consumes keys of its batch)
    exs = TPDecodeExchange.emulated(2, "cuda", 256, 64, timeout_ms=50)
    x = torch.randn(16, 128, device="cuda").bfloat16()
    w = torch.randn(256, 128, device="cuda").bfloat16()
    p0 = exs[0].linear_bcast(x, w)                           # the second rank never produces
    exs[0].reduce_rmsnorm(p0, torch.ones(256, device="cuda").bfloat16(), 1e-6, torch.zeros(16, 256, device="cuda").bfloat16())
    with pytest.raises(oplib.KernelWaitTimeout):
        eng.ppo_update(dict(data))
    stats = eng.ppo_update(dict(data))                       # the word was cleared: training continues
    assert stats[0]["update_successful"] == 1.0
    eng.destroy()


def test_offloaded_and_bf16_state_optimizers_follow_the_default_on_gpu():
    """Host-resident optimizer state streamed through the GPU in (tiny, so several) chunks gives the
    same parameters as the resident fused AdamW; bf16 moments with compensated weights stay close."""
    data = _batch()
    outs = {}
    for name, kw in (("resident", {}), ("offload", dict(offload=True, offload_chunk_numel=1 << 16)), ("bf16", dict(type="adam_bf16"))):
        eng = _tiny_actor(**kw)
        d = dict(data)
        d["prox_logp"] = eng.compute_logp(d)
        eng.compute_advantages(d)
        init = eng.store.flat_param.float().clone()
        for _ in range(3):
            st = eng.ppo_update(dict(d))             # the update consumes some keys of the batch it is given
            assert st[0]["update_successful"] == 1.0
        outs[name] = (eng.store.flat_param.float() - init)[: eng.store.numel].double()
        if name == "offload":
            assert eng.optimizer.master.device.type == "cpu" and eng.optimizer.master.is_pinned()
        eng.destroy()
    # two runs of one path already differ in last bits (atomics in the backward kernels), and Adam's first steps
    # turn a gradient near zero into a step of either sign: the paths are compared by the direction and size of
    # the three-step update
    cos = lambda a, b: float((a * b).sum() / (a.norm() * b.norm()).clamp(min=1e-30))   # noqa: E731
    assert float(outs["resident"].norm()) > 0
    assert cos(outs["resident"], outs["offload"]) > 0.98 and cos(outs["resident"], outs["bf16"]) > 0.95
    assert abs(float(outs["offload"].norm() / outs["resident"].norm()) - 1.0) < 0.05
    assert oplib.kernel_error() == 0


def test_sharded_parameters_follow_the_replicated_store_on_gpu():
    """``fsdp.shard_parameters`` on the GPU kernels (one rank: the unit protocol alone): layers live in transient
    buffers between enter and leave, weight gradients accumulate into per-unit fp32 buffers opened in the backward;
    three PPO steps move the weights like the replicated store does."""
    data = _batch()
    outs = {}
    for name in ("replicated", "sharded"):
        cfg = PPOActorConfig(init_from_scratch=True, dtype="bfloat16", optimizer=OptimizerConfig(lr=1e-4),
                             mb_spec=MicroBatchSpec(max_tokens_per_mb=1024), use_decoupled_loss=True, recompute_logprob=True,
                             kl_ctl=0.0, ppo_n_minibatches=1)
        cfg.fsdp.shard_parameters = name == "sharded"
        eng = B200PPOActor(cfg)
        eng.create_process_group()
        eng.initialize(model_config=preset("tiny-qwen3"), seed=1)
        init = {n: t.double() for n, t in eng.export_weights().items()}
        d = dict(data)
        d["prox_logp"] = eng.compute_logp(d)
        eng.compute_advantages(d)
        norms = []
        for _ in range(3):
            st = eng.ppo_update(dict(d))
            assert st[0]["update_successful"] == 1.0
            norms.append(st[0]["grad_norm"])
        after = eng.export_weights()
        outs[name] = (torch.cat([(after[n].double() - init[n]).reshape(-1) for n in sorted(init)]), norms)
        if name == "sharded":
            st_ = eng.store
            assert st_.flat_param is None and not st_._live and not st_._gbuf and all(p.data.stride() == (0,) * p.dim() for p in eng.model.parameters())
        eng.destroy()
    (ur, nr), (us, ns) = outs["replicated"], outs["sharded"]
    cos = float((ur * us).sum() / (ur.norm() * us.norm()).clamp(min=1e-30))
    assert float(ur.norm()) > 0 and cos > 0.98 and abs(float(us.norm() / ur.norm()) - 1.0) < 0.05, (cos, float(us.norm()), float(ur.norm()))
    assert all(abs(a - b) <= 0.05 * abs(b) + 0.05 for a, b in zip(ns, nr)), (ns, nr)
    assert oplib.kernel_error() == 0


def test_colocated_loop_runs_sixty_steps_on_gpu(tmp_path):
    """Trainer and rollout engine sharing one GPU (shared weights, CUDA graphs, prefix sharing, pages
    on demand in a small pool) for 60 steps: the configuration whose long runs used to die."""
    from areal_b200.api.cli_args import (ClusterSpecConfig, DatasetConfig, GRPOConfig, NormConfig, SaverConfig, StatsLoggerConfig)
    from areal_b200.dataset import RandomTokenDataset, bernoulli_reward_fn
    from areal_b200.rollout.workflows.rlvr import RLVRWorkflow
    from areal_b200.trainer.rl_trainer import PPOTrainer

    root = str(tmp_path)
    ic = NativeInferConfig(max_running_requests=32, page_size=16, context_length=256, retain_kv_on_weight_update=True,
                           enable_prefix_sharing=True)
    ic.num_pages = 160
    cfg = GRPOConfig(
        experiment_name="gpu-loop", trial_name="t0", total_train_epochs=100, seed=1, cluster=ClusterSpecConfig(fileroot=root),
        train_dataset=DatasetConfig(batch_size=2, shuffle=True, drop_last=True),
        gconfig=GenerationHyperparameters(n_samples=8, max_new_tokens=96, max_tokens=200, temperature=1.0, ignore_eos=True),
        rollout=InferenceEngineConfig(max_concurrent_rollouts=6, consumer_batch_size=2, max_head_offpolicyness=2),
        native_infer=ic,
        actor=PPOActorConfig(init_from_scratch=True, dtype="bfloat16", gradient_checkpointing=True,
                             optimizer=OptimizerConfig(lr=1e-5), mb_spec=MicroBatchSpec(max_tokens_per_mb=2048),
                             use_decoupled_loss=True, recompute_logprob=True, kl_ctl=0.0, ppo_n_minibatches=1,
                             reward_norm=NormConfig(mean_level="group", std_level="group", group_size=8)),
        saver=SaverConfig(fileroot=root, experiment_name="gpu-loop", trial_name="t0"),
        stats_logger=StatsLoggerConfig(fileroot=root, experiment_name="gpu-loop", trial_name="t0", jsonl=False))
    mc = preset("tiny-qwen3")
    ds = RandomTokenDataset(size=64, prompt_len=40, vocab_size=mc.vocab_size, seed=2, median_len=40, max_len=96, min_len=4, n_samples=8)
    with PPOTrainer(cfg, ds, model_config=mc) as tr:
        hist = tr.train(workflow=RLVRWorkflow(bernoulli_reward_fn, cfg.gconfig, reward_in_process=True), max_steps=60)
        eng = tr.rollout
        assert eng._exc is None
    assert len(hist) == 60 and all(h["ppo_actor/update/update_successful"] == 1.0 for h in hist)
    assert oplib.kernel_error() == 0


def test_pausable_memory_keeps_addresses_and_contents():
    """A pausable buffer gives its physical memory back (free memory grows by about its size), keeps its
    address, and holds the same bytes after resume; a CUDA graph captured on it replays correctly
    afterwards; a buffer that does not keep its contents comes back usable."""
    from areal_b200.ops import vmm

    if not vmm.available():
        pytest.skip("driver without the virtual-memory API")
    n = 64 << 20
    buf = vmm.PausableBuffer(n, "cuda", keep_contents=True)
    t = buf.tensor(torch.float32)
    t.copy_(torch.arange(t.numel(), device="cuda", dtype=torch.float32))
    out = torch.zeros(1, device="cuda")
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        out.copy_(t[:1024].sum().reshape(1))
        s.synchronize()
        with torch.cuda.graph(g, stream=s):
            out.copy_(t[:1024].sum().reshape(1))
    g.replay()
    torch.cuda.synchronize()
    want = float(out)
    ptr = t.data_ptr()
    free0, _ = torch.cuda.mem_get_info()
    buf.pause()
    assert buf.paused
    free1, _ = torch.cuda.mem_get_info()
    assert free1 - free0 >= n * 0.9
    buf.resume()
    torch.cuda.synchronize()
    assert not buf.paused and t.data_ptr() == ptr
    assert float(t[12345]) == 12345.0 and float(t[-1]) == float(t.numel() - 1)
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert float(out) == want
    scratch = vmm.PausableBuffer(8 << 20, "cuda", keep_contents=False)
    scratch.pause()
    scratch.resume()
    scratch.tensor(torch.int32).fill_(7)
    assert int(scratch.tensor(torch.int32)[100]) == 7
    pool = vmm.MemoryPool()
    a = pool.empty((1024, 1024), torch.bfloat16, tag="weights")
    b = pool.empty((1 << 20,), torch.uint8, tag="kv_cache", keep_contents=False)
    a.fill_(1.5)
    assert pool.pause(["kv_cache"]) == b.numel() and pool.resume(["kv_cache"]) == b.numel()
    assert pool.pause() == a.numel() * 2 + b.numel()
    pool.resume()
    torch.cuda.synchronize()
    assert float(a[5, 5]) == 1.5


def test_engine_offload_returns_the_kv_pool_and_keeps_its_graphs():
    """Rollout engine with a pausable KV pool: offload() hands the pool's memory back to the device,
    onload() takes it again; the decode graphs captured before keep working (same greedy outputs)."""
    from areal_b200.ops import vmm

    if not vmm.available():
        pytest.skip("driver without the virtual-memory API")
    cfg = preset("tiny-qwen3")
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=21)
    ic = NativeInferConfig(max_running_requests=8, page_size=16, context_length=256, pausable_kv_cache=True)
    ic.num_pages = 4096                                     # 4096 x 16 tokens x 2 layers x 2 (K, V) x 2 kv heads x 64 x 2 B = 64 MiB
    eng = NativeInferenceEngine(InferenceEngineConfig(), ic, model=model, eos_token_id=None).initialize(device="cuda", start_executor=False)
    g = GenerationHyperparameters(max_new_tokens=16, max_tokens=200, greedy=True, ignore_eos=True)

    async def run():
        return await asyncio.gather(*[eng.agenerate(ModelRequest(rid=f"o{i}", input_ids=list(range(5 + i, 45 + i)), gconfig=g)) for i in range(4)])

    first = asyncio.run(run())
    n_graphs = len(eng._graphs)
    assert n_graphs > 0
    free0, _ = torch.cuda.mem_get_info()
    eng.offload()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 - free0 > 48 << 20
    eng.onload()
    again = asyncio.run(run())
    assert [r.output_tokens for r in again] == [r.output_tokens for r in first]
    assert len(eng._graphs) == n_graphs                    # nothing was re-captured
    assert oplib.kernel_error() == 0
    eng.destroy()
