"""Drives the asynchronous-GRPO throughput benchmark through the public trainer API.

N = 1: trainer and rollout engine colocated on one GPU (shared bf16 weights, concurrent
generation and training). N >= 2: trainer ranks ``[0, N/2)`` and rollout ranks ``[N/2, N)`` of
one ``torch.distributed`` world; gradients are reduced and parameters refreshed by the fused
peer-memory kernels, weights are pushed shard-direct over NVLink after every step.

Measured quantities (rank 0 reports):
* ``value``: trained tokens per second over K steps, device-timed with CUDA events on the
  trainer ranks (barrier + synchronize on both sides, max over ranks);
* ``e2e``: the same metric over K further steps, wall-clock around ``PPOTrainer.train`` (the
  user-facing call), which every step copies the step's inputs host->device from pinned memory
  and reads the step's statistics back device->host; byte counts are accumulated from the
  tensors actually copied.
"""
from __future__ import annotations

import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from ..api.cli_args import (ClusterSpecConfig, DatasetConfig, GenerationHyperparameters, GRPOConfig, InferenceEngineConfig,
                            MicroBatchSpec, NativeInferConfig, NormConfig, OptimizerConfig, PPOActorConfig,
                            RejectionSamplingConfig, SaverConfig, StatsLoggerConfig)
from ..dataset import RandomTokenDataset, bernoulli_reward_fn
from ..models.config import preset
from ..ops import lib as oplib
from ..utils import logging as alog

logger = alog.getLogger("bench")


class _ByteCounter:
    h2d = 0
    d2h = 0


def _instrument_transfers(engine):
    """Counts host->device bytes of micro-batch inputs and device->host bytes of step results."""
    orig = engine._mb_to_device

    def counted(mb):
        for v in mb.values():
            if torch.is_tensor(v) and v.device.type == "cpu":
                _ByteCounter.h2d += v.numel() * v.element_size()
        return orig(mb)
    engine._mb_to_device = counted
    orig_step = engine.optimizer_step

    def counted_step():
        out = orig_step()
        _ByteCounter.d2h += 16  # the 4-float optimizer state read back per step
        return out
    engine.optimizer_step = counted_step


def _make_config(args, n_pairs: int, max_running: int, fileroot: str) -> GRPOConfig:
    bs = args.prompts_per_gpu_pair
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # Activation memory policy: one trainer GPU that also holds the whole optimizer state
    # (colocated, or 1 trainer + 1 rollout) has ~30 GB left, so it recomputes activations
    # (colocated) or uses small micro-batches; from 2 trainer ranks on the optimizer state is
    # sharded and full activations of 8k-token micro-batches fit.
    ckpt = getattr(args, "grad_ckpt", -1)
    if ckpt < 0:
        ckpt = 1 if world == 1 else 0
    mb_tokens = args.max_tokens_per_mb
    if mb_tokens <= 0:
        mb_tokens = 16384 if ckpt else (4096 if n_pairs == 1 else 8192)
    args._resolved = {"gradient_checkpointing": bool(ckpt), "max_tokens_per_mb": mb_tokens}
    return GRPOConfig(
        experiment_name="bench-async-grpo", trial_name="t0", total_train_epochs=1000, seed=1,
        cluster=ClusterSpecConfig(fileroot=fileroot),
        train_dataset=DatasetConfig(batch_size=bs, shuffle=True, drop_last=True),
        gconfig=GenerationHyperparameters(n_samples=args.group_size, max_new_tokens=args.max_len,
                                          max_tokens=args.prompt_len + args.max_len + 8, temperature=1.0, ignore_eos=True),
        rollout=InferenceEngineConfig(max_concurrent_rollouts=bs * (args.staleness + 1), consumer_batch_size=bs,
                                      max_head_offpolicyness=args.staleness),
        native_infer=NativeInferConfig(max_running_requests=max_running, page_size=64,
                                       context_length=args.prompt_len + args.max_len + 64, mem_fraction_static=0.35 if n_pairs == 1 and int(os.environ.get('WORLD_SIZE', '1')) == 1 else 0.6,
                                       max_prefill_tokens=16384,
                                       retain_kv_on_weight_update=bool(getattr(args, "retain_kv", 1)),
                                       enable_prefix_sharing=bool(getattr(args, "prefix_sharing", 1))),
        actor=PPOActorConfig(init_from_scratch=True, dtype="bfloat16", gradient_checkpointing=bool(ckpt),
                             optimizer=OptimizerConfig(lr=1e-6, weight_decay=0.01, gradient_clipping=1.0),
                             mb_spec=MicroBatchSpec(max_tokens_per_mb=mb_tokens),
                             use_decoupled_loss=True, recompute_logprob=True, kl_ctl=0.0, ppo_n_minibatches=1,
                             prox_logp_method=args.prox_logp_method,
                             eps_clip=0.2, rejection_sampling=RejectionSamplingConfig(upper=5.0),
                             reward_norm=NormConfig(mean_level="group", std_level="group", group_size=args.group_size),
                             weight_update_mode="p2p", logprobs_chunk_size=2048),
        saver=SaverConfig(fileroot=fileroot, experiment_name="bench", trial_name="t0"),
        stats_logger=StatsLoggerConfig(fileroot=fileroot, experiment_name="bench", trial_name="t0", jsonl=False),
    )


def _dataset(args, model_cfg, seed: int):
    return RandomTokenDataset(size=4096, prompt_len=args.prompt_len, vocab_size=model_cfg.vocab_size, seed=seed,
                              median_len=args.median_len, max_len=args.max_len, min_len=16)


def _tokens_of(history) -> float:
    return float(sum(h.get("ppo_actor/n_tokens", 0.0) for h in history))


def run_async_grpo_bench(args, clock_sampler_cls) -> Optional[dict]:
    from ..rollout.workflows.rlvr import RLVRWorkflow
    from ..trainer.rl_trainer import PPOTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py ...")
    torch.cuda.set_device(local_rank)
    model_cfg = preset(args.model)
    fileroot = f"/tmp/areal_bench_{os.getpid()}"
    W, K = args.warmup, args.steps

    if world == 1:
        cfg = _make_config(args, 1, max_running=256, fileroot=fileroot)
        ds = _dataset(args, model_cfg, seed=1)
        trainer = PPOTrainer(cfg, ds, model_config=model_cfg)
        _instrument_transfers(trainer.actor)
        wf = RLVRWorkflow(bernoulli_reward_fn, cfg.gconfig, reward_in_process=True)
        return _timed_loop(args, trainer, wf, clock_sampler_cls, world, rank, model_cfg, parallelism="colocated-1gpu")

    # ---------------------------------------------------------------- split world
    from .spmd import init_split_world, make_split_trainer, run_rollout_rank

    dev = torch.device("cuda", local_rank)
    n_train = world // 2
    split, groups, bus = init_split_world(n_train, dev)
    cfg = _make_config(args, n_train, max_running=256, fileroot=fileroot)
    if split.is_trainer:
        ds = _dataset(args, model_cfg, seed=1)  # only sizes the trainer's bookkeeping
        trainer = make_split_trainer(cfg, model_cfg, split, groups, bus, ds, seed=1)
        _instrument_transfers(trainer.actor)
        res = _timed_loop(args, trainer, None, clock_sampler_cls, world, rank, model_cfg,
                          parallelism=f"train:dp{n_train}+rollout:dp{world - n_train}", groups=groups)
        if rank == 0:
            bus.put("exit", 1)
        dist.barrier(group=groups["world_cpu"])
        return res if rank == 0 else None
    ds = _dataset(args, model_cfg, seed=1000 + rank)
    wf = RLVRWorkflow(bernoulli_reward_fn, cfg.gconfig, reward_in_process=True)
    run_rollout_rank(cfg, model_cfg, split, groups, bus, ds, wf, dev, seed=1)
    dist.barrier(group=groups["world_cpu"])
    return None


def _timed_loop(args, trainer, wf, clock_sampler_cls, world, rank, model_cfg, parallelism: str, groups=None):
    W, K = args.warmup, args.steps
    n_train = max(1, world // 2) if world > 1 else 1
    cpu_group = groups["cpu"] if groups else None

    def sync():
        torch.cuda.synchronize()
        if cpu_group is not None:
            dist.barrier(group=cpu_group)
        torch.cuda.synchronize()

    trainer.train(workflow=wf, max_steps=W)
    trainer.start_step += W
    # ---- region A: device-timed
    sampler = clock_sampler_cls(torch.cuda.current_device())
    sync()
    launches0 = oplib.launch_count()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    hist_a = trainer.train(workflow=wf, max_steps=K)
    e1.record()
    sync()
    clocks = sampler.stop()
    launches = oplib.launch_count() - launches0
    trainer.start_step += K
    ms_a = e0.elapsed_time(e1)
    tok_a = _tokens_of(hist_a)
    # ---- region B: end-to-end through the public API, wall clock
    _ByteCounter.h2d = _ByteCounter.d2h = 0
    sync()
    t0 = time.perf_counter()
    hist_b = trainer.train(workflow=wf, max_steps=K)
    sync()
    wall_b = time.perf_counter() - t0
    tok_b = _tokens_of(hist_b)
    stats = torch.tensor([ms_a, tok_a, wall_b, tok_b, float(_ByteCounter.h2d), float(_ByteCounter.d2h), float(launches)],
                         dtype=torch.float64)
    if cpu_group is not None:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=cpu_group)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM, group=cpu_group)
        ms_a, wall_b = float(mx[0]), float(mx[2])
        # ``ppo_actor/n_tokens`` is exported after a reduction over the trainer ranks, so every
        # rank already holds the GLOBAL token count of a step: take it once, do not sum it again
        tok_a, tok_b = float(mx[1]), float(mx[3])
        h2d, d2h, launches = float(sm[4]), float(sm[5]), int(sm[6])
    else:
        h2d, d2h = float(stats[4]), float(stats[5])
    push_ms = getattr(getattr(trainer.actor, "_weight_pusher", None), "last_ms", None)
    phases = {}
    for h in hist_a:
        for k_, v_ in h.items():
            if k_.startswith("timeperf/"):
                phases[k_[9:]] = phases.get(k_[9:], 0.0) + float(v_) / max(1, len(hist_a))
    trainer.close()
    if rank != 0:
        return None
    value = tok_a / (ms_a / 1e3)
    e2e = tok_b / wall_b
    seq_len = args.prompt_len + args.median_len
    return {
        "metric": "async GRPO trained tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms_a / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform-random prompts, forced log-normal response lengths, Bernoulli rewards, random-init weights)",
        "impl": "native",
        "config": {"model": args.model, "global_batch": args.prompts_per_gpu_pair * args.group_size * n_train,
                   "seq_len": seq_len, "prompt_len": args.prompt_len, "response_median": args.median_len,
                   "response_cap": args.max_len, "group_size": args.group_size, "parallelism": parallelism,
                   "max_staleness": args.staleness, "prox_logp_method": args.prox_logp_method, **getattr(args, "_resolved", {}),
                   "inflight_weight_update": "running requests keep their KV cache" if getattr(args, "retain_kv", 1) else "running requests are re-prefilled",
                   "prefix_sharing": bool(getattr(args, "prefix_sharing", 1)),
                   "decode_switches": {k_: os.environ.get(k_, "0") for k_ in ("AB2_PDL", "AB2_DECODE_SPLITK")},
                   "l2_policy": "inputs larger than L2 (16 GB of weights stream every step)",
                   "params_b": model_cfg.num_params() / 1e9, "weight_sync_ms": push_ms,
                   "phase_seconds_per_step": {k_: round(v_, 4) for k_, v_ in sorted(phases.items())}},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d / K, "d2h_bytes_per_step": d2h / K},
        "gpu_launches": int(launches),
    }
