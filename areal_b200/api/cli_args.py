"""Experiment configuration: a typed dataclass tree loaded from YAML with ``key=value``
command-line overrides and ``${a.b}`` interpolation.

The field names and defaults follow the reference's ``areal/api/cli_args.py`` (NormConfig
:43, MicroBatchSpec :100, GenerationHyperparameters :164, OptimizerConfig :377,
TrainEngineConfig :1248, RejectionSamplingConfig :1505, PPOActorConfig :1672,
PPOCriticConfig :1990, InferenceEngineConfig :2478, SaverConfig :2735, RecoverConfig :2760,
BaseExperimentConfig :3179, PPOConfig :3397, GRPOConfig :3468; loader :3474-3568) so the
reference's YAML files load unchanged. The loader is self-contained (PyYAML only): the
reference's Hydra/OmegaConf machinery is replaced by ``_merge_into_dataclass`` below, which
type-checks while it merges.
"""
from __future__ import annotations

import argparse
import copy
import dataclasses
import os
import re
import types
import typing
from dataclasses import MISSING, asdict, dataclass, field, fields, is_dataclass
from pathlib import Path
from typing import Any, Optional, Union, get_args, get_origin, get_type_hints

import yaml


# --------------------------------------------------------------------------- leaf configs
@dataclass
class NormConfig:
    """Mean / std normalisation of rewards or advantages."""

    mean_level: Optional[str] = "batch"  # batch | group | none
    mean_leave1out: bool = False
    std_level: Optional[str] = "batch"
    std_unbiased: bool = True
    eps: float = 1e-5
    group_size: int = 1

    def __post_init__(self):
        for lvl in (self.mean_level, self.std_level):
            if lvl not in ("batch", "group", "none", None):
                raise ValueError(f"normalisation level must be batch|group|none, got {lvl}")


@dataclass
class MicroBatchSpec:
    n_mbs: Optional[int] = 1
    granularity: int = 1
    max_tokens_per_mb: Optional[int] = None
    n_mbs_divisor: int = 1
    packing_algorithm: str = "ffd"  # ffd | kk

    @classmethod
    def new(cls, mb_spec: "MicroBatchSpec", **kwargs) -> "MicroBatchSpec":
        d = dict(n_mbs=mb_spec.n_mbs, granularity=mb_spec.granularity, max_tokens_per_mb=mb_spec.max_tokens_per_mb,
                 n_mbs_divisor=mb_spec.n_mbs_divisor, packing_algorithm=mb_spec.packing_algorithm)
        d.update(kwargs)
        return cls(**d)


@dataclass
class GenerationHyperparameters:
    n_samples: int = 1
    max_new_tokens: int = 16384
    min_new_tokens: int = 0
    max_tokens: int = 32768
    greedy: bool = False
    top_p: float = 1.0
    top_k: int = int(1e8)
    temperature: float = 1.0
    stop_token_ids: list[int] = field(default_factory=list)
    ignore_eos: bool = False
    skip_special_tokens: bool = True
    stop: Optional[list[str]] = None
    frequency_penalty: float = 0.0
    seed: Optional[int] = None
    lora_name: str = ""
    use_beam_search: bool = False
    reward_normalization: bool = False
    drop_incomplete_group: bool = False

    def new(self, **kwargs) -> "GenerationHyperparameters":
        d = {f.name: copy.copy(getattr(self, f.name)) for f in fields(self)}
        d.update(kwargs)
        return GenerationHyperparameters(**d)


@dataclass
class OptimizerConfig:
    type: str = "adam"  # adam | adam_bf16 | sgd
    lr: float = 1e-3
    weight_decay: float = 0.01
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    min_lr_ratio: float = 0.0
    lr_scheduler_type: str = "constant"  # constant | linear | cosine
    warmup_steps_proportion: float = 0.001
    warmup_steps: Optional[int] = None
    offload: bool = False             # fp32 master weights + moments in pinned host memory, streamed through the GPU in chunks
    offload_chunk_numel: int = 1 << 26  # elements per streamed chunk (three fp32 buffers of this size, double buffered)
    initial_loss_scale: float = 2 ** 32
    min_loss_scale: float = 1.0
    loss_scale_window: float = 5
    hysteresis: int = 2
    gradient_clipping: float = 1.0

    def __post_init__(self):
        if self.type not in ("adam", "adam_bf16", "sgd", "adamw"):
            raise ValueError(f"unknown optimizer type {self.type}")
        if self.lr_scheduler_type not in ("constant", "linear", "cosine"):
            raise ValueError(f"unknown lr scheduler {self.lr_scheduler_type}")


@dataclass
class FSDPWrapPolicy:
    transformer_layer_cls_to_wrap: Optional[list[str]] = None


@dataclass
class FSDPEngineConfig:
    wrap_policy: Optional[FSDPWrapPolicy] = None
    offload_params: bool = False
    memory_efficient_load: bool = False
    reshard_after_forward: bool = True
    shard_parameters: bool = False           # ZeRO-3: weights and gradients sharded too, decoder layers gathered one at a time (for models that do not fit replicated)
    fuse_reduce_scatter_adamw: bool = True   # fused RS + cast/scale + sharded AdamW kernel
    fuse_ulysses_projections: bool = True    # sequence-parallel all-to-alls folded into the QKV / output projection kernels
    tp_sequence_parallel: bool = False       # tensor parallel with the residual stream split by rows (gather -> GEMM, GEMM -> reduce-scatter)
    fuse_tp_projections: bool = True         # ... those pairs as one peer-memory kernel each on CUDA
    context_parallel: str = "ulysses"  # ulysses (heads exchanged by all-to-all) | zigzag (sequence chunks, K/V gathered; any head count)
    reduce_in_switch: bool = False           # gradient reduce-scatter by multimem.ld_reduce (NVLS) when a multicast mapping exists
    bucket_mb: int = 256
    per_layer_optim_step: bool = False        # accepted for compatibility (the flat sharded optimizer steps once)
    optim_step_prefetch_layers: int = 1
    shard_vision_across_sp: bool = True       # Ulysses + image tower: each rank encodes its share of the pictures (False: every rank encodes all of them)


@dataclass
class FP8Config:
    """Block-scaled fp8 (1x128 activation blocks, 128x128 weight blocks)."""

    enabled: bool = False
    include_experts: bool = True
    include_dense: bool = False


@dataclass
class ArchonEngineConfig:
    attn_type: str = "varlen"
    enable_compile: bool = False
    ac_mode: str = "selective"  # none | full | selective | memory_budget
    pp_schedule: str = "1F1B"
    fp8: FP8Config = field(default_factory=FP8Config)
    fuse_ep_dispatch: bool = True     # expert-parallel dispatch / combine as peer-memory kernels instead of NCCL all-to-alls
    offload_params: bool = False
    extra: dict = field(default_factory=dict)   # backend-specific keys of the reference, accepted and kept
    __allow_extra__ = True


@dataclass
class MegatronEngineConfig:
    wrap_with_ddp: bool = True
    use_distributed_optimizer: bool = True
    virtual_pipeline_parallel_size: int = 1
    recompute_granularity: Optional[str] = "full"
    moe_token_dispatcher_type: str = "alltoall"
    moe_enable_deepep: bool = False
    fp8: FP8Config = field(default_factory=FP8Config)
    extra: dict = field(default_factory=dict)   # backend-specific keys of the reference, accepted and kept
    __allow_extra__ = True


@dataclass
class SchedulingSpec:
    cpu: int = 4
    gpu: int = 0
    mem: int = 32
    port_count: int = 2
    image: str = ""
    task_type: str = "worker"
    env_vars: dict[str, str] = field(default_factory=dict)
    cmd: Optional[str] = None
    nodelist: Optional[str] = None
    exclude: Optional[str] = None
    partition: Optional[str] = None
    time_limit: Optional[str] = None
    additional_bash_cmds: Optional[list[str]] = None
    srun_additional_args: str = ""
    container_type: str = "none"
    mount: str = ""
    reservation: Optional[str] = None
    exclusive: bool = False
    ray_placement_strategy: str = "PACK"


@dataclass
class SchedulingStrategy:
    type: str = "separation"  # separation | colocation
    target: Optional[str] = None
    fork: bool = True


@dataclass
class TrainEngineConfig:
    experiment_name: str = ""
    trial_name: str = ""
    path: str = ""
    attn_impl: str = "flash_attention_2"
    init_from_scratch: bool = False
    is_critic: bool = False
    temperature: float = 1.0
    logprobs_chunk_size: int = 1024
    mb_spec: MicroBatchSpec = field(default_factory=MicroBatchSpec)
    pad_to_maximum: bool = False
    disable_dropout: bool = False
    gradient_checkpointing: bool = False
    activation_checkpointing: Optional[str] = None   # none | full | selective | memory_budget (overrides the flag above)
    activation_memory_budget: float = 0.5            # fraction of layers recomputed in memory_budget mode
    use_kernels: bool = True                          # accepted for compatibility: the sm_100a kernels are always used
    weight_update_delta_method: str = "none"          # none | exact | adamw_inversion (see wsync/delta.py)
    weight_update_anchor_interval: int = 0            # full (non-delta) push every k updates; 0 = never forced
    admin_api_key: str = "areal-admin-key"
    log_level: str = "info"
    request_timeout: float = 3600.0
    setup_timeout: float = 300.0
    workers_ready_timeout: float = 600.0
    dtype: str = "bfloat16"
    grad_reduce_dtype: str = "float32"
    optimizer_dtype: str = "float32"
    optimizer: Optional[OptimizerConfig] = None
    weight_update_mode: str = "xccl"  # disk | xccl | p2p | awex
    enable_delta_weight_update: bool = False
    fsdp: FSDPEngineConfig = field(default_factory=FSDPEngineConfig)
    archon: ArchonEngineConfig = field(default_factory=ArchonEngineConfig)
    megatron: MegatronEngineConfig = field(default_factory=MegatronEngineConfig)
    offload: bool = False
    use_lora: bool = False
    lora_rank: int = 32
    lora_alpha: int = 16
    target_modules: list[str] = field(default_factory=list)
    peft_type: str = "lora"
    enable_tree_training: bool = False
    scheduling_spec: list[SchedulingSpec] = field(default_factory=lambda: [SchedulingSpec(gpu=1)])
    scheduling_strategy: SchedulingStrategy = field(default_factory=SchedulingStrategy)
    backend: str = ""
    _version: str = "v1"
    model_config: Optional[dict] = None  # inline architecture (random-init experiments)


@dataclass
class RejectionSamplingConfig:
    level: str = "token"  # token | sequence
    action: str = "mask"  # mask | clamp
    metric: str = "ratio"  # ratio | kl_k1 | kl_k2 | kl_k3 | binary_kl
    agg: str = "mean"  # sum | mean | max (sequence level)
    upper: Optional[float] = 5.0
    lower: Optional[float] = None

    def __post_init__(self):
        if self.level not in ("token", "sequence"):
            raise ValueError("rejection_sampling.level must be token|sequence")
        if self.action not in ("mask", "clamp"):
            raise ValueError("rejection_sampling.action must be mask|clamp")
        if self.metric not in ("ratio", "kl_k1", "kl_k2", "kl_k3", "binary_kl"):
            raise ValueError(f"unknown rejection metric {self.metric}")
        if self.agg not in ("sum", "mean", "max"):
            raise ValueError("rejection_sampling.agg must be sum|mean|max")
        if self.upper is None and self.lower is None:
            raise ValueError("rejection sampling needs at least one bound")
        if self.action == "clamp":
            if self.metric != "ratio":
                raise ValueError("action='clamp' only supports metric='ratio' (a divergence cannot be truncated into a weight)")
            if self.lower is None:
                self.lower = 0.0
        if self.metric == "ratio":
            if self.upper is not None and self.upper <= 1.0:
                raise ValueError("ratio metric: upper must be > 1.0 (an on-policy token has ratio 1)")
            if self.lower is not None and (self.lower < 0.0 or (self.lower == 0.0 and self.action == "mask")):
                raise ValueError("ratio metric: lower must be positive")
        elif self.metric in ("kl_k2", "kl_k3", "binary_kl") and self.upper is not None and self.upper <= 0.0:
            raise ValueError(f"{self.metric}: upper must be positive (the estimator is non-negative)")
        if self.lower is not None and self.upper is not None and self.lower > self.upper:
            raise ValueError("rejection sampling: lower must not exceed upper")
        if self.level == "token" and self.agg != "mean":
            import warnings

            warnings.warn(f"rejection_sampling.agg='{self.agg}' is ignored at token level", UserWarning, stacklevel=2)


@dataclass
class PPOActorConfig(TrainEngineConfig):
    ppo_n_minibatches: int = 4
    eps_clip: float = 0.2
    eps_clip_higher: Optional[float] = None
    c_clip: Optional[float] = None
    m2_threshold: Optional[float] = None
    reward_norm: Optional[NormConfig] = None
    reward_scaling: float = 1.0
    reward_bias: float = 0.0
    reward_clip: float = 20.0
    overlong_reward_penalty: bool = False
    overlong_tokens: Optional[int] = None
    overlong_penalty_factor: Optional[float] = None
    mask_no_eos_with_zero: bool = False
    discount: float = 1.0
    gae_lambda: float = 1.0
    gae_lambda_kwargs: dict = field(default_factory=dict)   # parameters of a lambda schedule (see algo/advantages.py)
    gae_timestep_unit: str = "token"  # token | turn
    adv_norm: Optional[NormConfig] = None
    kl_ctl: float = 0.1
    kl_estimator: str = "k1"
    use_sapo_loss: bool = False
    sapo_tau_pos: float = 1.0
    sapo_tau_neg: float = 1.05
    use_cispo_loss: bool = False
    recompute_logprob: bool = False
    use_decoupled_loss: bool = False
    rejection_sampling: Optional[RejectionSamplingConfig] = None
    behave_imp_weight_cap: Optional[float] = None  # legacy alias -> rejection_sampling.upper
    importance_sampling_level: str = "token"  # token | sequence (GSPO)
    prox_logp_method: str = "recompute"  # recompute | loglinear | linear | reuse_train_logp | metrics (recompute + approximation errors logged)
    log_agent_stats: bool = False
    log_agent_stats_keys: list[str] = field(default_factory=list)
    max_new_tokens: int = 1024

    def __post_init__(self):
        if self.c_clip is not None and self.c_clip <= 1.0:
            raise ValueError("c_clip must be > 1")
        if self.behave_imp_weight_cap is not None and self.rejection_sampling is None:
            self.rejection_sampling = RejectionSamplingConfig(upper=self.behave_imp_weight_cap)
        if self.use_sapo_loss and self.use_decoupled_loss:
            raise ValueError("SAPO loss requires use_decoupled_loss=false")
        if self.use_sapo_loss and self.use_cispo_loss:
            raise ValueError("choose at most one of SAPO / CISPO")
        if self.prox_logp_method not in ("recompute", "loglinear", "linear", "reuse_train_logp", "metrics"):
            raise ValueError(f"unknown prox_logp_method {self.prox_logp_method}")
        if self.prox_logp_method == "reuse_train_logp" and self.ppo_n_minibatches != 1:
            raise ValueError("prox_logp_method='reuse_train_logp' requires ppo_n_minibatches=1: only then are the update "
                             "forward's log-probs those of the policy before the update")
        if self.kl_estimator not in ("k1", "k2", "k3"):
            raise ValueError("kl_estimator must be k1|k2|k3")


@dataclass
class PPOCriticConfig(TrainEngineConfig):
    ppo_n_minibatches: int = 4
    eps_clip: float = 0.5
    mask_no_eos_with_zero: bool = False
    value_loss_type: str = "mse"  # mse | huber

    def __post_init__(self):
        self.is_critic = True


@dataclass
class TeacherConfig(TrainEngineConfig):
    rl_loss_weight: float = 1.0
    distill_loss_weight: float = 0.005
    engine_type: str = "train"                # train: forward with a train engine; rollout: score through an inference engine
    rollout: Optional[dict] = None
    train: Optional[dict] = None


@dataclass
class vLLMConfig:
    model: str = ""
    seed: int = 1
    skip_tokenizer_init: bool = False
    enforce_eager: bool = False
    dtype: str = "bfloat16"
    max_num_seqs: int = 256
    block_size: int = 16
    swap_space: int = 4
    cpu_offload_gb: float = 0
    max_model_len: Optional[int] = 32768
    enable_chunked_prefill: bool = False
    enable_prefix_caching: bool = False
    gpu_memory_utilization: float = 0.9
    worker_extension_cls: str = ""
    enable_sleep_mode: bool = False
    uvicorn_log_level: str = "warning"
    enable_lora: bool = False
    max_lora_rank: int = 16
    extra: dict = field(default_factory=dict)   # server flags of the reference's backend, accepted and kept
    __allow_extra__ = True

    @staticmethod
    def build_args(cfg: "vLLMConfig", tp_size: int = 1, pp_size: int = 1, host: Optional[str] = None, port: Optional[int] = None,
                   dist_init_addr: Optional[str] = None, n_nodes: int = 1, node_rank: int = 0) -> dict:
        """Flags of a vLLM OpenAI-compatible server for this configuration (reference: ``areal/api/cli_args.py:2081-2117``)."""
        a = {k: v for k, v in dataclasses.asdict(cfg).items() if k != "extra"}
        a.update(cfg.extra or {})
        a.update(tokenizer=cfg.model, load_format="auto", trust_remote_code=True, tensor_parallel_size=tp_size, pipeline_parallel_size=pp_size)
        if host is not None:
            a["host"] = host
        if port is not None:
            a["port"] = port
        if n_nodes > 1:
            a.update(nnodes=n_nodes, node_rank=node_rank)
            if dist_init_addr:
                from ..utils.network import split_hostport

                h, p_ = split_hostport(dist_init_addr)            # (IPv6 literals with or without brackets)
                a.update(master_addr=h, master_port=str(p_))
            if node_rank > 0:
                a["headless"] = True
        return a

    @staticmethod
    def build_cmd(cfg: "vLLMConfig", tp_size: int = 1, pp_size: int = 1, module: str = "vllm.entrypoints.openai.api_server", **kw) -> list[str]:
        return server_cmd(module, vLLMConfig.build_args(cfg, tp_size, pp_size, **kw))


def server_cmd(module: str, args: dict) -> list[str]:
    """``python -m module --flag value ...``: booleans become bare flags (left out when false), ``None`` is left out,
    lists repeat their values after the flag."""
    import sys

    cmd = [sys.executable, "-m", module]
    for k, v in args.items():
        flag = "--" + k.replace("_", "-")
        if v is None or v is False or v == "":
            continue
        if v is True:
            cmd.append(flag)
        elif isinstance(v, (list, tuple)):
            cmd += [flag] + [str(x) for x in v]
        elif isinstance(v, dict):
            import json

            cmd += [flag, json.dumps(v)]
        else:
            cmd += [flag, str(v)]
    return cmd


@dataclass
class SGLangConfig:
    model_path: str = ""
    random_seed: int = 1
    skip_tokenizer_init: bool = False
    disable_cuda_graph: bool = False
    disable_radix_cache: bool = True
    enable_nccl_nvls: bool = False
    attention_backend: Optional[str] = None
    max_running_requests: Optional[int] = None
    chunked_prefill_size: Optional[int] = -1
    max_prefill_tokens: int = 32768
    schedule_policy: str = "lpm"
    page_size: int = 1
    cpu_offload_gb: int = 0
    dtype: str = "bfloat16"
    kv_cache_dtype: str = "auto"
    context_length: Optional[int] = 32768
    mem_fraction_static: Optional[float] = 0.9
    log_level: str = "warning"
    enable_metrics: bool = True
    decode_log_interval: int = 1
    enable_multithread_load: bool = False
    enable_return_routed_experts: bool = False
    enable_lora: Optional[bool] = None
    max_lora_rank: Optional[int] = None
    extra: dict = field(default_factory=dict)   # server flags of the reference's backend, accepted and kept
    __allow_extra__ = True

    @staticmethod
    def build_args(cfg: "SGLangConfig", tp_size: int = 1, base_gpu_id: int = 0, host: Optional[str] = None, port: Optional[int] = None,
                   dist_init_addr: Optional[str] = None, n_nodes: int = 1, node_rank: int = 0, pp_size: int = 1) -> dict:
        """Flags of ``sglang.launch_server`` for this configuration (reference: ``areal/api/cli_args.py:2258-2330``)."""
        a = {k: v for k, v in dataclasses.asdict(cfg).items() if k != "extra"}
        a.update(cfg.extra or {})
        a.update(tokenizer_path=cfg.model_path, tokenizer_mode="auto", load_format="auto", trust_remote_code=True, device="cuda",
                 is_embedding=False, tp_size=tp_size, pp_size=pp_size, base_gpu_id=base_gpu_id, nnodes=n_nodes, node_rank=node_rank,
                 dist_init_addr=dist_init_addr)
        if host is not None:
            a["host"] = host
        if port is not None:
            a["port"] = port
        return a

    @staticmethod
    def build_cmd(cfg: "SGLangConfig", tp_size: int = 1, base_gpu_id: int = 0, module: str = "sglang.launch_server", **kw) -> list[str]:
        return server_cmd(module, SGLangConfig.build_args(cfg, tp_size, base_gpu_id, **kw))


@dataclass
class NativeInferConfig:
    """Options of this framework's own rollout engine (paged KV, continuous batching)."""

    page_size: int = 64
    max_running_requests: int = 256
    max_prefill_tokens: int = 16384
    context_length: int = 32768
    mem_fraction_static: float = 0.85
    # Colocated engines: size the KV pool as (free memory - reserve_free_gb) instead of a fraction, so
    # the trainer sharing the GPU keeps a known amount for its activations. 0 = use the fraction.
    reserve_free_gb: float = 0.0
    # KV pool in pausable memory (addresses survive while the physical pages leave the GPU): offload() then
    # really returns the pool's memory to the device and onload() takes it back without re-capturing CUDA graphs
    pausable_kv_cache: bool = False
    kv_cache_dtype: str = "bfloat16"
    use_cuda_graph: bool = True
    weight_dtype: str = "bfloat16"  # or float8_e4m3fn (block-scaled)
    random_seed: int = 1
    share_trainer_weights: bool = True  # colocated mode: read the trainer's parameters in place
    num_pages: Optional[int] = None     # fixed KV page count (default: sized from free memory)
    # In-flight weight updates: False = running requests are interrupted and re-prefilled under
    # the new weights (what a server that flushes its cache does); True = they keep their KV
    # cache and simply continue, every token tagged with the version that sampled it.
    retain_kv_on_weight_update: bool = False
    # KV pages of a request: False = taken as the sequence grows (a page at a time; when the pool runs
    # dry the most recently admitted request is pre-empted: it returns what it has and its client
    # resubmits it, so its prefix is prefetched again); True = all pages for prompt + max_new_tokens are
    # reserved at admission (no pre-emption ever, but long budgets keep most of the pool idle).
    reserve_full_length: bool = False
    # Requests with an identical prompt (the samples of a GRPO group, retries) share the prompt's full KV
    # pages and the logits of its last token: the prompt is prefetched once per weight version.
    enable_prefix_sharing: bool = False


@dataclass
class OpenAIProxyConfig:
    mode: str = "inline"  # inline | subproc | online
    tool_call_parser: str = "qwen25"
    reasoning_parser: str = "qwen3"
    chat_template_type: str = "hf"
    engine_max_tokens: Optional[int] = None
    export_style: str = "individual"  # individual | concat
    subproc_max_workers: int = 4
    turn_discount: float = 1.0
    session_timeout_seconds: int = 3600
    admin_api_key: str = "areal-admin-key"


AgentConfig = OpenAIProxyConfig


@dataclass
class InferenceEngineConfig:
    experiment_name: Optional[str] = None
    trial_name: Optional[str] = None
    fileroot: Optional[str] = None
    max_concurrent_rollouts: Optional[int] = None
    queue_size: Optional[int] = None
    consumer_batch_size: int = 1
    max_head_offpolicyness: int = 0
    # The admission formula bounds how far rollout may run AHEAD of the trainer; an episode that
    # finishes long after its cohort (a straggler) is still trained when it arrives, at whatever age
    # it then has (the reference behaves the same). True: a training batch is not formed while an
    # episode that would exceed the bound in the NEXT batch is still running, so no trained token is
    # older than max_head_offpolicyness versions, at the price of waiting for stragglers.
    strict_staleness: bool = False
    enable_rollout_tracing: bool = False
    deterministic_sampling: bool = False
    check_trajectory_format: bool = False
    schedule_policy: str = "round_robin"
    routing_strategy: str = "round_robin"
    tokenizer_path: str = ""
    dump_to_file: bool = False
    setup_timeout: float = 300.0
    request_timeout: float = 3600.0
    request_retries: int = 3
    serialize_group_samples: bool = False
    workers_ready_timeout: float = 600.0
    lora_name: str = ""
    model: str = "default"
    poll_interval: float = 0.05
    admin_api_key: str = "areal-admin-key"
    api_url: str = ""
    provider_api_key: str = ""
    pause_grace_period: float = 0.0
    scheduling_spec: list[SchedulingSpec] = field(default_factory=lambda: [SchedulingSpec(gpu=1)])
    scheduling_strategy: SchedulingStrategy = field(default_factory=SchedulingStrategy)
    backend: str = ""
    use_lora: bool = False
    agent: OpenAIProxyConfig = field(default_factory=OpenAIProxyConfig)
    openai: Optional[OpenAIProxyConfig] = None
    return_routed_experts: bool = False
    _version: str = "v1"


@dataclass
class _Timer:
    experiment_name: str = ""
    trial_name: str = ""
    fileroot: str = ""
    freq_epochs: Optional[int] = None
    freq_steps: Optional[int] = None
    freq_secs: Optional[int] = None


@dataclass
class EvaluatorConfig(_Timer):
    eval_before_train: bool = False


@dataclass
class SaverConfig(_Timer):
    mode: str = "auto"  # auto | sync | async
    max_pinned_gb: float = 17.5


@dataclass
class RecoverConfig(_Timer):
    mode: str = "disabled"  # on | auto | off | disabled
    retries: int = 3
    no_save_optim: bool = False
    no_load_optim: bool = False


@dataclass
class WandBConfig:
    mode: str = "disabled"
    wandb_base_url: str = ""
    wandb_api_key: str = ""
    entity: Optional[str] = None
    project: Optional[str] = None
    name: Optional[str] = None
    job_type: Optional[str] = None
    group: Optional[str] = None
    notes: Optional[str] = None
    tags: Optional[list[str]] = None
    config: Optional[dict] = None
    id_suffix: Optional[str] = "train"


@dataclass
class SwanlabConfig:
    project: Optional[str] = None
    name: Optional[str] = None
    config: Optional[dict] = None
    logdir: Optional[str] = None
    mode: Optional[str] = "disabled"
    api_key: Optional[str] = None


@dataclass
class TensorBoardConfig:
    path: Optional[str] = None


@dataclass
class TrackioConfig:
    mode: str = "disabled"            # disabled | online | local
    project: Optional[str] = None     # defaults to the experiment name
    name: Optional[str] = None        # defaults to the trial name
    space_id: Optional[str] = None    # Hugging Face Space that also receives the metrics

    def __post_init__(self):
        if self.mode not in ("disabled", "online", "local"):
            raise ValueError(f"trackio.mode must be disabled, online or local, got '{self.mode}'")


@dataclass
class StatsLoggerConfig:
    experiment_name: str = ""
    trial_name: str = ""
    fileroot: str = ""
    wandb: WandBConfig = field(default_factory=WandBConfig)
    swanlab: SwanlabConfig = field(default_factory=SwanlabConfig)
    tensorboard: TensorBoardConfig = field(default_factory=TensorBoardConfig)
    trackio: TrackioConfig = field(default_factory=TrackioConfig)
    jsonl: bool = True  # always-on local sink


@dataclass
class SessionTracerConfig:
    enabled: bool = False
    flush_threshold: int = 256


@dataclass
class MemoryProfilerConfig:
    enabled: bool = False
    profile_steps: list[int] = field(default_factory=list)
    max_entries: int = 100000


@dataclass
class PerfTracerConfig:
    experiment_name: str = ""
    trial_name: str = ""
    fileroot: str = ""
    enabled: bool = False
    save_interval: int = 1
    profile_steps: Optional[list[int]] = None
    session_tracer: SessionTracerConfig = field(default_factory=SessionTracerConfig)


@dataclass
class NameResolveConfig:
    type: str = "nfs"  # memory | nfs | etcd3 | ray
    nfs_record_root: str = "/tmp/areal/name_resolve"
    etcd3_addr: str = "localhost:2379"
    ray_actor_name: str = "ray_kv_store"


@dataclass
class ClusterSpecConfig:
    name_resolve: NameResolveConfig = field(default_factory=NameResolveConfig)
    cluster_name: str = "local"
    fileroot: str = "/tmp/areal/experiments"
    n_nodes: int = 1
    n_gpus_per_node: int = 8


@dataclass
class SchedulerConfig:
    type: Optional[str] = None  # local | ray | slurm | null (SPMD launch)
    endpoint: str = "http://localhost:8081"
    deploy_mode: str = "separation"
    functioncall_service_domain: str = "http://localhost:8080"
    reward_functioncall_config: dict = field(default_factory=dict)
    reward_model_path: str = ""
    reward_model_service_url: str = "http://localhost:30000/classify"


@dataclass
class DatasetConfig:
    path: str = ""
    type: str = ""
    batch_size: int = 1
    shuffle: bool = True
    pin_memory: bool = False
    num_workers: int = 0
    drop_last: bool = True
    max_length: Optional[int] = None


_DatasetConfig = DatasetConfig


@dataclass
class LauncherConfig:
    inference_server_cpus_per_gpu: int = 4
    inference_server_mem_per_gpu: int = 32768
    trainer_cpus_per_gpu: int = 4
    trainer_mem_per_gpu: int = 32768
    inference_server_env_vars: str = ""
    trainer_env_vars: str = ""


@dataclass
class BaseExperimentConfig:
    post_exit_hook: Optional[str] = None      # shell command (LOG_DIR set) or `module:function` run by the launcher after the job ended
    experiment_name: str = "default-experiment"
    trial_name: str = "trial0"
    cluster: ClusterSpecConfig = field(default_factory=ClusterSpecConfig)
    allocation_mode: str = ""
    seed: int = 1
    enable_offload: bool = False
    total_train_epochs: int = 1
    total_train_steps: Optional[int] = None
    total_train_n_seqs: Optional[int] = None
    tokenizer_path: str = ""
    train_dataset: DatasetConfig = field(default_factory=DatasetConfig)
    valid_dataset: Optional[DatasetConfig] = None
    saver: SaverConfig = field(default_factory=SaverConfig)
    evaluator: EvaluatorConfig = field(default_factory=EvaluatorConfig)
    stats_logger: StatsLoggerConfig = field(default_factory=StatsLoggerConfig)
    perf_tracer: Optional[PerfTracerConfig] = None
    memory_profiler: MemoryProfilerConfig = field(default_factory=MemoryProfilerConfig)
    recover: RecoverConfig = field(default_factory=RecoverConfig)
    sglang: SGLangConfig = field(default_factory=SGLangConfig)
    vllm: vLLMConfig = field(default_factory=vLLMConfig)
    native_infer: NativeInferConfig = field(default_factory=NativeInferConfig)
    launcher: LauncherConfig = field(default_factory=LauncherConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)


@dataclass
class SFTConfig(BaseExperimentConfig):
    actor: TrainEngineConfig = field(default_factory=TrainEngineConfig)
    model: Optional[TrainEngineConfig] = None  # legacy alias of ``actor``


@dataclass
class RWConfig(BaseExperimentConfig):
    actor: TrainEngineConfig = field(default_factory=TrainEngineConfig)
    model: Optional[TrainEngineConfig] = None


@dataclass
class DPOConfig(BaseExperimentConfig):
    actor: TrainEngineConfig = field(default_factory=TrainEngineConfig)
    ref: Optional[TrainEngineConfig] = None
    beta: float = 0.1
    loss_type: str = "sigmoid"  # sigmoid | ipo


@dataclass
class PPOConfig(BaseExperimentConfig):
    async_training: bool = True
    gconfig: GenerationHyperparameters = field(default_factory=GenerationHyperparameters)
    eval_gconfig: Optional[GenerationHyperparameters] = None
    rollout: InferenceEngineConfig = field(default_factory=InferenceEngineConfig)
    actor: PPOActorConfig = field(default_factory=PPOActorConfig)
    ref: Optional[PPOActorConfig] = None
    critic: Optional[PPOCriticConfig] = None
    teacher: Optional[TeacherConfig] = None
    dynamic_bs: bool = False


@dataclass
class GRPOConfig(PPOConfig):
    pass


# --------------------------------------------------------------------------- loader
class ConfigError(ValueError):
    pass


_INTERP = re.compile(r"\$\{([^}]+)\}")


def _lookup(root: dict, dotted: str):
    cur: Any = root
    for part in dotted.split("."):
        if isinstance(cur, dict) and part in cur:
            cur = cur[part]
        elif isinstance(cur, list) and part.isdigit() and int(part) < len(cur):
            cur = cur[int(part)]
        else:
            raise ConfigError(f"interpolation key '{dotted}' not found")
    return cur


def _resolve(node, root, depth=0):
    if depth > 32:
        raise ConfigError("interpolation cycle")
    if isinstance(node, dict):
        return {k: _resolve(v, root, depth) for k, v in node.items()}
    if isinstance(node, list):
        return [_resolve(v, root, depth) for v in node]
    if isinstance(node, str):
        m = _INTERP.fullmatch(node.strip())
        if m:  # whole-value reference keeps the referenced type
            key = m.group(1).strip()
            if key.startswith("oc.env:") or key.startswith("env:"):
                name, _, dflt = key.split(":", 1)[1].partition(",")
                return os.environ.get(name.strip(), dflt.strip() or None)
            return _resolve(_lookup(root, key), root, depth + 1)
        if "${" in node:
            return _INTERP.sub(lambda mm: str(_resolve(_lookup(root, mm.group(1).strip()), root, depth + 1)), node)
    return node


def _parse_scalar(text: str):
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def _set_dotted(tree: dict, dotted: str, value, create: bool) -> None:
    parts = dotted.split(".")
    cur = tree
    for p in parts[:-1]:
        if isinstance(cur, list):
            cur = cur[int(p)]
            continue
        if p not in cur or cur[p] is None:
            cur[p] = {}
        cur = cur[p]
    last = parts[-1]
    if isinstance(cur, list):
        cur[int(last)] = value
    else:
        cur[last] = value


def _strip_optional(tp):
    origin = get_origin(tp)
    if origin is Union or origin is types.UnionType:
        args = [a for a in get_args(tp) if a is not type(None)]
        if len(args) == 1:
            return args[0], True
        return tp, True
    return tp, False


def _coerce(value, tp, path: str):
    tp, optional = _strip_optional(tp)
    if value is None:
        return None
    origin = get_origin(tp)
    if is_dataclass(tp):
        if is_dataclass(value):
            return value
        if not isinstance(value, dict):
            raise ConfigError(f"{path}: expected a mapping for {tp.__name__}, got {type(value).__name__}")
        return _merge_into_dataclass(tp, value, path)
    if origin in (list, typing.List):
        (sub,) = get_args(tp) or (Any,)
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"{path}: expected a list")
        return [_coerce(v, sub, f"{path}[{i}]") for i, v in enumerate(value)]
    if origin in (dict, typing.Dict):
        if not isinstance(value, dict):
            raise ConfigError(f"{path}: expected a mapping")
        return dict(value)
    if tp is Any or origin is Union or origin is types.UnionType or origin is typing.Literal:
        return value
    if tp is bool:
        if isinstance(value, bool):
            return value
        if isinstance(value, str) and value.lower() in ("true", "false"):
            return value.lower() == "true"
        raise ConfigError(f"{path}: expected bool, got {value!r}")
    if tp is int:
        if isinstance(value, bool):
            raise ConfigError(f"{path}: expected int, got bool")
        if isinstance(value, int):
            return value
        if isinstance(value, float) and value.is_integer():
            return int(value)
        if isinstance(value, str):
            try:
                return int(float(value)) if "e" in value.lower() else int(value)
            except ValueError:
                pass
        raise ConfigError(f"{path}: expected int, got {value!r}")
    if tp is float:
        if isinstance(value, (int, float)) and not isinstance(value, bool):
            return float(value)
        if isinstance(value, str):
            try:
                return float(value)
            except ValueError:
                pass
        raise ConfigError(f"{path}: expected float, got {value!r}")
    if tp is str:
        return value if isinstance(value, str) else str(value)
    return value


def _merge_into_dataclass(cls, data: dict, path: str = "", strict: bool = True):
    hints = get_type_hints(cls)
    known = {f.name: f for f in fields(cls)}
    kwargs = {}
    extra_ok = getattr(cls, "__allow_extra__", False) and "extra" in known
    extra: dict = {}
    for key, val in data.items():
        if key not in known:
            if extra_ok:      # tunables of a backend this framework replaces: kept, not interpreted
                extra[key] = val
                continue
            if not strict:
                continue
            raise ConfigError(f"unknown config key '{path + '.' if path else ''}{key}' for {cls.__name__}")
        kwargs[key] = _coerce(val, hints[key], f"{path + '.' if path else ''}{key}")
    if extra:
        kwargs["extra"] = {**kwargs.get("extra", {}), **extra}
    try:
        return cls(**kwargs)
    except (TypeError, ValueError) as e:
        raise ConfigError(f"{path or cls.__name__}: {e}") from e


def to_structured_cfg(raw: dict, config_cls, strict: bool = True):
    """Resolves ``${...}`` references and builds the typed dataclass tree. ``strict=False``
    ignores unknown TOP-LEVEL keys (a launcher reads the shared part of any experiment config)."""
    resolved = _resolve(raw, raw)
    return _merge_into_dataclass(config_cls, resolved, strict=strict)


def parse_cli_args(argv: list[str]):
    """Returns ``(raw_mapping, config_file)`` from ``--config file.yaml k=v +k=v ...``."""
    ap = argparse.ArgumentParser(add_help=True)
    ap.add_argument("--config", type=str, default=None, help="YAML experiment config")
    ap.add_argument("overrides", nargs="*", help="key=value overrides (dotted keys; +key adds)")
    args, unknown = ap.parse_known_args(argv)
    raw: dict = {}
    cfg_file = None
    if args.config:
        cfg_file = Path(args.config).expanduser().resolve()
        if not cfg_file.exists():
            raise ConfigError(f"config file {cfg_file} not found")
        raw = yaml.safe_load(cfg_file.read_text()) or {}
    for ov in list(args.overrides) + [u for u in unknown if "=" in u]:
        if "=" not in ov:
            raise ConfigError(f"override '{ov}' is not key=value")
        key, _, val = ov.partition("=")
        create = key.startswith("+")
        key = key.lstrip("+").strip()
        _set_dotted(raw, key, _parse_scalar(val), create)
    return raw, cfg_file


def config_to_dict(cfg) -> dict:
    return asdict(cfg)


def save_config(cfg, log_dir: str) -> str:
    os.makedirs(log_dir, exist_ok=True)
    path = os.path.join(log_dir, "config.yaml")
    with open(path, "w") as f:
        yaml.safe_dump(config_to_dict(cfg), f, sort_keys=False)
    return path


def get_log_dir(cfg: BaseExperimentConfig) -> str:
    import getpass

    return os.path.join(cfg.cluster.fileroot, "logs", getpass.getuser(), cfg.experiment_name, cfg.trial_name)


def load_expr_config(argv: list[str], config_cls):
    """Parses ``argv`` and returns ``(config, config_file)``; the merged config is saved to
    the experiment's log directory like the reference does (cli_args.py:3544-3568)."""
    raw, cfg_file = parse_cli_args(argv)
    cfg = to_structured_cfg(raw, config_cls)
    try:
        save_config(cfg, get_log_dir(cfg))
    except OSError:
        pass
    return cfg, str(cfg_file) if cfg_file else None
