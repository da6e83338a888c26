"""Drives the asynchronous-GRPO throughput benchmark through the public trainer API.

N = 1: trainer and rollout engine colocated on one GPU (shared bf16 weights, concurrent
generation and training). N >= 2: trainer ranks ``[0, T)`` and rollout ranks ``[T, N)`` of one
``torch.distributed`` world (``T = N / 2`` unless ``--train-gpus``): the trainers shard the
optimizer state over all of them (ZeRO) and split every packed micro-batch over groups of
``--sp`` ranks (Ulysses, projections fused with the exchanges); the rollout ranks form
tensor-parallel replicas of ``--rollout-tp`` GPUs (partial sums exchanged from the GEMM epilogue,
decode steps graph captured); weights are pushed shard-direct over NVLink after every step and
re-sharded into the tensor-parallel layout in flight.

Measured quantities (rank 0 reports):
* ``value``: trained tokens per second over K steps, device-timed with CUDA events on the
  trainer ranks (barrier + synchronize on both sides, max over ranks);
* ``e2e``: the same metric over K further steps, wall-clock around ``PPOTrainer.train`` (the
  user-facing call), which every step copies the step's inputs host->device from pinned memory
  and reads the step's results back device->host; byte counts are accumulated from the
  tensors actually copied;
* ``config.nccl_path_tokens_per_s`` (N >= 2): a few more steps of the SAME job with this
  repository's library-collective path switched on (NCCL reduce-scatter + all-gather around the
  optimizer, NCCL all-to-all around attention, NCCL broadcast weight update): the baseline that
  the fused kernels are there to beat. It is not the reference implementation.
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
    """Counts host->device bytes of micro-batch inputs; device->host bytes are counted by the
    engine itself wherever it reads results back (``engine.d2h_bytes``)."""
    orig = engine._mb_to_device

    def counted(mb):
        for v in mb.values():
            if torch.is_tensor(v) and v.device.type == "cpu":
                _ByteCounter.h2d += v.numel() * v.element_size()
        return orig(mb)
    engine._mb_to_device = counted


def resolve_layout(args, world: int) -> dict:
    """GPU roles of an N-GPU job: one rule for every N."""
    if world == 1:
        return dict(n_train=1, n_rollout=1, sp=1, dp=1, rollout_tp=1, replicas=1, colocated=True)
    n_train = args.train_gpus or world // 2
    n_roll = world - n_train
    if n_train < 1 or n_roll < 1:
        raise SystemExit("--train-gpus must leave at least one trainer and one rollout GPU")
    sp = args.sp or min(4, n_train)
    while n_train % sp:
        sp -= 1
    tp = args.rollout_tp or (2 if n_roll >= 2 and n_roll % 2 == 0 else 1)
    if n_roll % tp:
        raise SystemExit(f"--rollout-tp {tp} does not divide the {n_roll} rollout GPUs")
    return dict(n_train=n_train, n_rollout=n_roll, sp=sp, dp=n_train // sp, rollout_tp=tp, replicas=n_roll // tp, colocated=False)


def _make_config(args, lay: dict, fileroot: str) -> GRPOConfig:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    global_prompts = max(1, int(round(args.prompts_per_gpu * world)))
    # batches travel leader -> head: a head merges the batches of its `feeders` leaders
    feeders = max(1, lay["replicas"] // lay["dp"])
    bs = max(1, -(-global_prompts // (lay["dp"] * feeders)))
    global_prompts = bs * lay["dp"] * feeders
    mb_tokens = args.max_tokens_per_mb
    if mb_tokens <= 0:
        mb_tokens = 8192
    elif lay["colocated"]:
        # one GPU holds the whole optimizer state, the gradients AND the KV cache: quarter-size micro-batches,
        # so that most of what is left can hold KV pages
        mb_tokens = min(mb_tokens, 8192)
    ctx = args.prompt_len + args.max_len + 64
    args._resolved = {"gradient_checkpointing": bool(args.grad_ckpt) if not (args.grad_ckpt < 0 and lay["colocated"]) else "memory_budget: all layers recomputed (colocated: the KV cache takes the rest)",
                      "max_tokens_per_mb": mb_tokens,
                      "prompts_per_step": global_prompts, "prompts_per_batch": bs}
    if lay["colocated"]:
        # what trainer and engine need beside the resident state and the KV pool. Measured peak with 8k-token
        # micro-batches and every layer recomputed: 19.5 GB (layer-input checkpoints, one layer's activations and
        # gradients, LM-head chunks, prefill activations of up to 16k tokens); the decode graphs of the larger
        # buckets and allocator fragmentation come on top
        reserve = float(os.environ.get("AREAL_BENCH_RESERVE_GB", "0") or 0) or (10.0 + mb_tokens * 2.0e-3)
        infer = dict(reserve_free_gb=reserve, max_running_requests=256)
    else:
        infer = dict(mem_fraction_static=0.8, max_running_requests=512)   # the rest: CUDA graphs' pools, the broadcast path's staging buffer
    return GRPOConfig(
        experiment_name="bench-async-grpo", trial_name="t0", total_train_epochs=1000, seed=1,
        cluster=ClusterSpecConfig(fileroot=fileroot),
        train_dataset=DatasetConfig(batch_size=bs, shuffle=True, drop_last=True),
        gconfig=GenerationHyperparameters(n_samples=args.group_size, max_new_tokens=args.max_len,
                                          max_tokens=args.prompt_len + args.max_len + 8, temperature=1.0, ignore_eos=True),
        rollout=InferenceEngineConfig(max_concurrent_rollouts=bs * (args.staleness + 1), consumer_batch_size=bs,
                                      max_head_offpolicyness=args.staleness),
        native_infer=NativeInferConfig(page_size=64, context_length=ctx, max_prefill_tokens=16384,
                                       retain_kv_on_weight_update=bool(args.retain_kv),
                                       enable_prefix_sharing=bool(args.prefix_sharing), **infer),
        actor=PPOActorConfig(init_from_scratch=True, dtype="bfloat16", gradient_checkpointing=bool(args.grad_ckpt),
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


def _cap_micro_batch(args, actor) -> None:
    """Caps the packed micro-batch size by what the trainer GPU has left once parameters, gradients
    and optimizer state are resident: about 0.8 MB per micro-batch token (layer-input checkpoints,
    one layer's activations and their gradients, LM-head chunks) plus 6 GB of slack."""
    free, _ = torch.cuda.mem_get_info()
    sp = max(1, getattr(actor, "sp_size", 1))
    cap = int((free / 2 ** 30 - 6.0) / 0.8e-3) * sp // 1024 * 1024
    if actor.cpu_group is not None:          # every trainer rank must split the batch the same way
        t = torch.tensor([cap], dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=actor.cpu_group)
        cap = int(t[0])
    mb = actor.config.mb_spec.max_tokens_per_mb
    if cap < mb:
        cap = max(4096, cap)
        logger.info("micro-batches capped at %d tokens (%.1f GB free on the trainer GPU)", cap, free / 2 ** 30)
        actor.config.mb_spec.max_tokens_per_mb = cap
        args._resolved["max_tokens_per_mb"] = cap
        args._resolved["max_tokens_per_mb_capped_by_memory"] = True


def kept_layers_for(free_gb: float, tokens: int, n_layers: int, hidden: int) -> int:
    """Layers whose activations fit: 0.30 MB per token and kept layer at hidden 4096 (bf16 activations of attention and
    MLP plus what autograd saves), 8 KB per token and layer for the recomputed layers' inputs, one layer's working set,
    5 GB for the LM-head chunks and 12 GB of slack."""
    per_layer_gb = tokens * 0.30e-3 * (hidden / 4096.0)
    avail = free_gb - 12.0 - 5.0 - per_layer_gb - n_layers * tokens * 8e-6
    return max(0, min(n_layers, int(avail / per_layer_gb)))


def plan_activation_policy(free_gb: float, tokens: int, n_layers: int, hidden: int, floor_tokens: int) -> tuple[int, int]:
    """(tokens per rank and micro-batch, kept layers). Recomputing a layer costs a third of its forward + backward time;
    a smaller micro-batch costs next to nothing as long as its GEMMs still have thousands of rows (gradients accumulate
    locally, no collective per micro-batch). So the micro-batch shrinks by halves, not below ``floor_tokens`` (4096 per
    rank, and the longest sequence), until every layer's activations fit; what then still does not fit is recomputed."""
    t = tokens
    while kept_layers_for(free_gb, t, n_layers, hidden) < n_layers and t // 2 >= floor_tokens:
        t //= 2
    return t, kept_layers_for(free_gb, t, n_layers, hidden)


def _pick_recompute(args, actor, model_cfg) -> None:
    """The activation policy, one rule at every N (``--grad-ckpt -1``): keep the activations of as
    many layers as the memory left after parameters, gradients and optimizer state holds, recompute
    the rest in backward (``memory_budget`` checkpointing; the kept layers are the last ones, whose
    activations live shortest). Estimate per token of a rank's micro-batch slice: 0.30 MB per kept
    layer (bf16 activations of attention and MLP plus what autograd saves), 8 KB per recomputed
    layer (its input), one layer's working set, 5 GB for the LM-head chunks and 12 GB of slack."""
    if args.grad_ckpt >= 0:
        return
    free, _ = torch.cuda.mem_get_info()
    sp = max(1, getattr(actor, "sp_size", 1))
    n = model_cfg.num_layers

    def kept_layers(t: int) -> int:
        return kept_layers_for(free / 2 ** 30, t, n, model_cfg.hidden_size)

    t = actor.config.mb_spec.max_tokens_per_mb // sp
    longest = -(-(args.prompt_len + args.max_len) // 1024) * 1024
    t, keep = plan_activation_policy(free / 2 ** 30, t, n, model_cfg.hidden_size, max(4096, -(-longest // sp)))
    if actor.cpu_group is not None:               # every trainer rank must split the batch the same way
        tt = torch.tensor([t], dtype=torch.int64)
        dist.all_reduce(tt, op=dist.ReduceOp.MIN, group=actor.cpu_group)
        t = int(tt[0])
        tt = torch.tensor([kept_layers(t)], dtype=torch.int64)
        dist.all_reduce(tt, op=dist.ReduceOp.MIN, group=actor.cpu_group)
        keep = int(tt[0])
    if t * sp != actor.config.mb_spec.max_tokens_per_mb:
        actor.config.mb_spec.max_tokens_per_mb = t * sp
        args._resolved["max_tokens_per_mb"] = t * sp
        args._resolved["max_tokens_per_mb_shrunk_to_keep_activations"] = True
    frac = 1.0 - keep / n
    actor.model.set_activation_checkpointing("memory_budget", frac)
    args._resolved["gradient_checkpointing"] = f"memory_budget: {n - keep} of {n} layers recomputed"
    args._resolved["free_gb_before_activations"] = round(free / 2 ** 30, 1)
    logger.info("activation policy: %d of %d layers recomputed (%.1f GB free, %d tokens per rank and micro-batch)", n - keep, n,
                free / 2 ** 30, t)


def _dataset(args, model_cfg, seed: int):
    return RandomTokenDataset(size=4096, prompt_len=args.prompt_len, vocab_size=model_cfg.vocab_size, seed=seed,
                              median_len=args.median_len, max_len=args.max_len, min_len=16, n_samples=args.group_size)


def _sum_of(history, key: str) -> float:
    return float(sum(h.get(key, 0.0) for h in history))


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
    lay = resolve_layout(args, world)
    cfg = _make_config(args, lay, fileroot)

    if world == 1:
        ds = _dataset(args, model_cfg, seed=1)
        trainer = PPOTrainer(cfg, ds, model_config=model_cfg)
        _instrument_transfers(trainer.actor)
        wf = RLVRWorkflow(bernoulli_reward_fn, cfg.gconfig, reward_in_process=True)
        return _timed_loop(args, trainer, wf, clock_sampler_cls, world, rank, model_cfg, lay, parallelism="colocated-1gpu")

    # ---------------------------------------------------------------- split world
    from .spmd import init_split_world, make_split_trainer, run_rollout_rank

    dev = torch.device("cuda", local_rank)
    split, groups, bus = init_split_world(lay["n_train"], dev, sp=lay["sp"], rollout_tp=lay["rollout_tp"])
    par = (f"train:d{lay['dp']}s{lay['sp']} (ZeRO over {lay['n_train']})+rollout:{lay['replicas']}xtp{lay['rollout_tp']}")
    if split.is_trainer:
        ds = _dataset(args, model_cfg, seed=1)  # only sizes the trainer's bookkeeping
        trainer = make_split_trainer(cfg, model_cfg, split, groups, bus, ds, seed=1)
        _instrument_transfers(trainer.actor)
        _cap_micro_batch(args, trainer.actor)
        _pick_recompute(args, trainer.actor, model_cfg)
        res = _timed_loop(args, trainer, None, clock_sampler_cls, world, rank, model_cfg, lay, parallelism=par, groups=groups)
        if rank == 0:
            bus.put("exit", 1)
        dist.barrier(group=groups["world_cpu"])
        if rank == 0 and res is not None:
            rs = [bus.poll(f"rollout_stats/{r}") for r in split.leaders]
            rs = [x for x in rs if x]
            if rs:
                busy = [x.get("infer/busy_seconds", 0.0) / max(1e-9, x.get("infer/alive_seconds", 1.0)) for x in rs]
                res["config"]["rollout_busy_fraction"] = round(sum(busy) / len(busy), 3)
                res["config"]["rollout_decode_steps"] = int(sum(x.get("infer/decode_steps", 0) for x in rs))
                res["config"]["rollout_generated_tokens"] = int(sum(x.get("infer/generated_tokens", 0) for x in rs))
        return res if rank == 0 else None
    ds = _dataset(args, model_cfg, seed=1000 + rank)
    wf = RLVRWorkflow(bernoulli_reward_fn, cfg.gconfig, reward_in_process=True)
    worker = run_rollout_rank(cfg, model_cfg, split, groups, bus, ds, wf, dev, seed=1)
    if split.is_leader(rank):
        bus.put(f"rollout_stats/{rank}", worker.engine.export_stats())
    dist.barrier(group=groups["world_cpu"])
    return None


def _timed_loop(args, trainer, wf, clock_sampler_cls, world, rank, model_cfg, lay, parallelism: str, groups=None):
    W, K = args.warmup, args.steps
    cpu_group = groups["cpu"] if groups else None
    actor = trainer.actor

    def sync():
        torch.cuda.synchronize()
        if cpu_group is not None:
            dist.barrier(group=cpu_group)
        torch.cuda.synchronize()

    mem_base = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
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
    tok_a = _sum_of(hist_a, "ppo_actor/n_tokens")
    resp_a = _sum_of(hist_a, "ppo_actor/n_valid_tokens")
    # ---- region B: end-to-end through the public API, wall clock
    _ByteCounter.h2d = 0
    actor.d2h_bytes = 0
    sync()
    t0 = time.perf_counter()
    hist_b = trainer.train(workflow=wf, max_steps=K)
    sync()
    wall_b = time.perf_counter() - t0
    trainer.start_step += K
    tok_b = _sum_of(hist_b, "ppo_actor/n_tokens")
    h2d_b, d2h_b = float(_ByteCounter.h2d), float(actor.d2h_bytes)
    push_ms = getattr(getattr(actor, "_weight_pusher", None), "last_ms", None)
    push_dev_ms = getattr(getattr(actor, "_weight_pusher", None), "last_dev_ms", None)
    push_gbs = getattr(getattr(actor, "_weight_pusher", None), "last_gbps", None)
    # ---- region C: the same job on the library-collective path (NCCL), a few steps
    Kc = args.nccl_steps if args.nccl_steps >= 0 else (max(2, K // 5) if world >= 2 else 0)
    ms_c = tok_c = 0.0
    if Kc > 0 and world >= 2:
        actor.use_library_collectives(True)
        trainer.train(workflow=wf, max_steps=1)          # NCCL communicators connect outside the timed steps
        trainer.start_step += 1
        sync()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        hist_c = trainer.train(workflow=wf, max_steps=Kc)
        c1.record()
        sync()
        trainer.start_step += Kc
        ms_c, tok_c = c0.elapsed_time(c1), _sum_of(hist_c, "ppo_actor/n_tokens")
        push_ms_c = getattr(getattr(actor, "_weight_pusher", None), "last_ms", None)
    stats = torch.tensor([ms_a, tok_a, wall_b, tok_b, h2d_b, d2h_b, float(launches), resp_a, ms_c, tok_c], dtype=torch.float64)
    if cpu_group is not None:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=cpu_group)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM, group=cpu_group)
        ms_a, wall_b, ms_c = float(mx[0]), float(mx[2]), float(mx[8])
        # ``ppo_actor/n_tokens`` is exported after a reduction over the trainer ranks that saw different
        # tokens, so every rank already holds the GLOBAL count of a step: take it once, do not sum it again
        tok_a, tok_b, resp_a, tok_c = float(mx[1]), float(mx[3]), float(mx[7]), float(mx[9])
        h2d_b, d2h_b, launches = float(sm[4]), float(sm[5]), int(sm[6])
    phases = {}
    for h in hist_a:
        for k_, v_ in h.items():
            if k_.startswith("timeperf/"):
                phases[k_[9:]] = phases.get(k_[9:], 0.0) + float(v_) / max(1, len(hist_a))
    stale = [h.get("ppo_actor/update/staleness/avg") for h in hist_a if h.get("ppo_actor/update/staleness/avg") is not None]
    stale_max = [h.get("ppo_actor/update/staleness/max") for h in hist_a if h.get("ppo_actor/update/staleness/max") is not None]
    trainer.close()
    if rank != 0:
        return None
    value = tok_a / (ms_a / 1e3)
    e2e = tok_b / wall_b
    step_s = max(1e-9, phases.get("step", ms_a / 1e3 / K))
    cfgd = {"model": args.model, "preset": args.preset, "length_scale": args.length_scale,
            "global_batch": args._resolved["prompts_per_step"] * args.group_size,
            "prompts_per_step": args._resolved["prompts_per_step"], "group_size": args.group_size,
            "seq_len": args.prompt_len + args.median_len, "prompt_len": args.prompt_len, "response_median": args.median_len,
            "response_cap": args.max_len, "response_lengths": "log-normal per sample (sigma 0.6), forced",
            "parallelism": parallelism, "trainer_gpus": lay["n_train"], "rollout_gpus": lay["n_rollout"] if world > 1 else 1,
            "ulysses_sp": lay["sp"], "rollout_tp": lay["rollout_tp"], "rollout_replicas": lay["replicas"],
            "max_staleness": args.staleness, "prox_logp_method": args.prox_logp_method, **args._resolved,
            "loss": "decoupled PPO (GRPO advantages), fp32 master weights + AdamW moments",
            "inflight_weight_update": "running requests keep their KV cache" if args.retain_kv else "running requests are re-prefilled",
            "prefix_sharing": bool(args.prefix_sharing),
            "decode_switches": {k_: os.environ.get(k_, "0") for k_ in ("AB2_PDL", "AB2_DECODE_SPLITK")},
            "nccl_nvls": os.environ.get("NCCL_NVLS_ENABLE", "default"),
            "l2_policy": "inputs larger than L2 (16 GB of weights stream every step)",
            "params_b": model_cfg.num_params() / 1e9, "weight_sync_ms": push_ms, "weight_sync_device_ms": push_dev_ms,
            "weight_sync_gbs_per_trainer_gpu": round(push_gbs, 1) if push_gbs else None,
            "tokens_counted": "prompt + response tokens of the trained sequences",
            "response_tokens_per_s": resp_a / (ms_a / 1e3),
            "peak_memory_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
            "peak_memory_over_resident_gb": round((torch.cuda.max_memory_allocated() - mem_base) / 2 ** 30, 1),
            "trainer_busy_fraction": round(1.0 - phases.get("rollout", 0.0) / step_s, 3),
            "staleness_avg": round(sum(stale) / len(stale), 3) if stale else None,
            "staleness_max": max(stale_max) if stale_max else None,
            "phase_seconds_per_step": {k_: round(v_, 4) for k_, v_ in sorted(phases.items())}}
    if ms_c > 0:
        cfgd["nccl_path_tokens_per_s"] = tok_c / (ms_c / 1e3)
        cfgd["nccl_path_steps"] = Kc
        cfgd["nccl_path_weight_sync_ms"] = push_ms_c
        cfgd["fused_over_nccl_path"] = round(value / max(1e-9, cfgd["nccl_path_tokens_per_s"]), 3)
        cfgd["nccl_path_note"] = ("this repository's own library-collective path (NCCL reduce-scatter / all-gather / all-to-all / "
                                  "broadcast), same job and step loop; not the reference implementation")
    return {
        "metric": "async GRPO trained tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms_a / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform-random prompts, forced log-normal response lengths, Bernoulli rewards, random-init weights)",
        "impl": "native", "config": cfgd, "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d_b / K, "d2h_bytes_per_step": d2h_b / K},
        "gpu_launches": int(launches),
    }
