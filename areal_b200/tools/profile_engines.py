"""Profiles one training step or a burst of rollout decoding on the current GPU and prints
where the device time goes (kernel table from the PyTorch profiler, optionally a Chrome trace).

    python -m areal_b200.tools.profile_engines train   --model qwen3-8b --layers 6 --tokens-per-mb 8192 [--ckpt] [--trace out.json]
    python -m areal_b200.tools.profile_engines rollout --model qwen3-8b --layers 36 --batch 128 --ctx 256 --new 64

``--layers`` truncates the architecture so a profile fits in a minute; per-layer costs are the
same as in the full model. Reference: ``areal/tools/profile_engines.py``, ``profile_fsdp.py``,
``profile_archon.py``."""
from __future__ import annotations

import argparse
import asyncio
import json
import sys
import time

import torch


def _train_engine(a):
    from ..api.cli_args import MicroBatchSpec, OptimizerConfig, PPOActorConfig
    from ..engine.train_engine import B200PPOActor
    from ..models.config import preset

    cfg = PPOActorConfig(init_from_scratch=True, dtype="bfloat16", gradient_checkpointing=bool(a.ckpt), optimizer=OptimizerConfig(lr=1e-6),
                         mb_spec=MicroBatchSpec(max_tokens_per_mb=a.tokens_per_mb), use_decoupled_loss=True, recompute_logprob=True,
                         kl_ctl=0.0, ppo_n_minibatches=1, logprobs_chunk_size=2048, prox_logp_method="reuse_train_logp")
    e = B200PPOActor(cfg)
    e.create_process_group()
    kw = {"num_layers": a.layers} if a.layers else {}
    e.initialize(model_config=preset(a.model, **kw), seed=1)
    return e


def _train_batch(a, vocab: int, gen):
    B, L = a.seqs, a.seq_len
    ids = torch.randint(0, vocab, (B, L), generator=gen)
    lm = torch.zeros(B, L, dtype=torch.int32)
    lm[:, L // 2:] = 1
    return dict(input_ids=ids, attention_mask=torch.ones(B, L, dtype=torch.bool), loss_mask=lm, logprobs=torch.full((B, L), -11.9),
                versions=torch.zeros(B, L, dtype=torch.int32), rewards=torch.randn(B, generator=gen))


def profile_train(a) -> dict:
    from torch.profiler import ProfilerActivity, profile

    e = _train_engine(a)
    gen = torch.Generator().manual_seed(0)

    def step():
        d = _train_batch(a, e.model_config.vocab_size, gen)
        e.compute_advantages(d)
        return e.ppo_update(d)
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    step()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        step()
        torch.cuda.synchronize()
    print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=a.rows, max_name_column_width=70))
    if a.trace:
        prof.export_chrome_trace(a.trace)
    n_tok = a.seqs * a.seq_len
    flops = 6.0 * e.model_config.num_params() * n_tok * (4.0 / 3.0 if a.ckpt else 1.0)
    res = {"what": "train_step", "model": a.model, "layers": e.model_config.num_layers, "tokens": n_tok, "tokens_per_mb": a.tokens_per_mb,
           "gradient_checkpointing": bool(a.ckpt), "wall_s": round(wall, 4), "model_tflops_per_s": round(flops / wall / 1e12, 1)}
    print(json.dumps(res), flush=True)
    return res


def profile_rollout(a) -> dict:
    from torch.profiler import ProfilerActivity, profile

    from ..api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeInferConfig
    from ..api.io_struct import ModelRequest
    from ..engine.infer_engine import NativeInferenceEngine
    from ..models.config import preset

    kw = {"num_layers": a.layers} if a.layers else {}
    mc = preset(a.model, **kw)
    eng = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=a.batch, context_length=a.ctx + a.new + 64,
                                                                           mem_fraction_static=0.5), model_config=mc)
    eng.initialize(start_executor=False)
    g = GenerationHyperparameters(max_new_tokens=a.new, max_tokens=a.ctx + a.new + 8, ignore_eos=True)
    gen = torch.Generator().manual_seed(0)

    async def run():
        reqs = [ModelRequest(input_ids=torch.randint(0, mc.vocab_size, (a.ctx,), generator=gen).tolist(), gconfig=g) for _ in range(a.batch)]
        return await asyncio.gather(*[eng.agenerate(r) for r in reqs])
    asyncio.run(run())
    torch.cuda.synchronize()
    s0 = eng.stats["decode_steps"]
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        t0 = time.perf_counter()
        out = asyncio.run(run())
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
    print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=a.rows, max_name_column_width=70))
    if a.trace:
        prof.export_chrome_trace(a.trace)
    steps = eng.stats["decode_steps"] - s0
    res = {"what": "rollout_burst", "model": a.model, "layers": mc.num_layers, "batch": a.batch, "ctx": a.ctx, "new": a.new,
           "wall_s_under_profiler": round(wall, 3), "decode_steps": int(steps), "tokens": sum(r.output_len for r in out)}
    print(json.dumps(res), flush=True)
    eng.destroy()
    return res


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["train", "rollout"])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--tokens-per-mb", type=int, default=8192)
    ap.add_argument("--seqs", type=int, default=64)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--ckpt", action="store_true")
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=256)
    ap.add_argument("--new", type=int, default=64)
    ap.add_argument("--rows", type=int, default=40)
    ap.add_argument("--trace", default="")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("profile_engines needs a GPU", file=sys.stderr)
        return 2
    (profile_train if a.what == "train" else profile_rollout)(a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
