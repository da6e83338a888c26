"""The training engine: a :class:`~areal_b200.models.decoder.CausalLM` on packed micro-batches
with ZeRO-style sharded optimisation over data-parallel (and Ulysses sequence-parallel)
ranks, implementing the :class:`~areal_b200.api.engine_api.TrainEngine` contract.

Call flow of ``train_batch`` (reference: ``areal/engine/fsdp_engine.py:774``,
``_prepare_mb_list`` :1883, ``_compute_logprobs_and_loss`` :2147, ``optimizer_step`` :696):

  split by token budget -> pad to pages -> global loss weight (all-reduce) ->
  per micro-batch: forward, fused LM-head logprob/entropy, user loss, scaled backward
  (weight gradients accumulate in fp32 ``main_grad``) ->
  gradient reduce-scatter -> global norm / clip -> sharded AdamW -> parameter all-gather.

Algorithm-specific engines (PPO actor / critic, SFT, RW, DPO) are thin mix-ins at the bottom,
mirroring ``FSDPPPOActor`` etc. (fsdp_engine.py:2257-2476).
"""
from __future__ import annotations

import math
import os
import time
from datetime import timedelta
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist

from ..api.alloc_mode import FSDPParallelStrategy, ModelAllocation, ParallelStrategy
from ..api.cli_args import MicroBatchSpec, TrainEngineConfig
from ..api.engine_api import InferenceEngine, TrainEngine
from ..api.io_struct import FinetuneSpec, SaveLoadMeta, WeightUpdateMeta
from ..models import hf_io
from ..models.config import ModelConfig, preset
from ..models.decoder import CausalLM, PackedBatch, build_model
from ..utils import data as D
from ..utils import logging as alog
from ..utils import stats_tracker
from .flat_params import FlatParamStore
from .optimizer import ShardedAdamW

logger = alog.getLogger("train_engine")

DIST_TIMEOUT_S = 7200


def _dtype_of(name: str):
    return {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[name]


class _GatherOverSP(torch.autograd.Function):
    """Concatenates the sequence-parallel ranks' slices of a per-token tensor. Every rank then
    evaluates the SAME loss on whole sequences; in backward a rank keeps only the gradient of its
    own slice (the other slices are the other ranks' business), so the parameter gradients summed
    over the group are those of the loss counted once. Role of ``_sp_all_gather`` in the reference
    (areal/engine/fsdp_engine.py:2057-2142)."""

    @staticmethod
    def forward(ctx, x, group, rank, world):
        ctx.rank, ctx.n = rank, x.shape[0]
        x = x.contiguous()
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x, group=group)
        return torch.cat(parts, dim=0)

    @staticmethod
    def backward(ctx, g):
        return g[ctx.rank * ctx.n:(ctx.rank + 1) * ctx.n].contiguous(), None, None, None


class B200TrainEngine(TrainEngine):
    def __init__(self, config: TrainEngineConfig):
        self.config = config
        self.model: Optional[CausalLM] = None
        self.model_config: Optional[ModelConfig] = None
        self.store: Optional[FlatParamStore] = None
        self.optimizer: Optional[ShardedAdamW] = None
        self.parallel: Optional[ParallelStrategy] = None
        self.device = torch.device("cpu")
        self.rank = 0
        self.world_size = 1
        self._version = 0
        self._dp_group = None
        self._sp_group = None
        self._cpu_group = None
        self._own_pg = False
        self.rollout_engine: Optional[InferenceEngine] = None
        self.weight_update_meta: Optional[WeightUpdateMeta] = None
        self._initialized = False
        self._weight_pusher = None
        self._grad_reducer = None
        self.last_step_stats: dict = {}
        self.d2h_bytes = 0          # bytes of results this engine read back from the device (losses, log-probs, optimizer status)
        self._err_poll = None

    # ------------------------------------------------------------------ process groups
    def create_process_group(self, parallel_strategy: Optional[ParallelStrategy] = None):
        use_cuda = torch.cuda.is_available() and os.environ.get("AREAL_FORCE_CPU", "0") != "1"
        if parallel_strategy is None and self.config.backend:
            parallel_strategy = ModelAllocation.from_str(self.config.backend).parallel
        self.parallel = parallel_strategy or FSDPParallelStrategy()
        env_world = int(os.environ.get("WORLD_SIZE", "1"))
        if not dist.is_initialized() and env_world > 1:
            backend = "nccl" if use_cuda else "gloo"
            if use_cuda:
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dist.init_process_group(backend=backend, timeout=timedelta(seconds=DIST_TIMEOUT_S))
            self._own_pg = True
        if dist.is_initialized():
            self.rank, self.world_size = dist.get_rank(), dist.get_world_size()
        if use_cuda:
            self.device = torch.device("cuda", torch.cuda.current_device())
        p = self.parallel
        if getattr(self, "_train_ranks", None) is None:
            self._train_ranks = list(range(self.world_size))
        n = len(self._train_ranks)
        if p.world_size != n:
            if p.world_size == 1 and n > 1:  # bare config: everything data-parallel
                self.parallel = p = FSDPParallelStrategy(data_parallel_size=n)
            else:
                raise ValueError(f"parallel strategy {p} needs {p.world_size} ranks, engine has {n}")
        self.pp_size = p.pp_size
        self.pp_rank = 0
        self._pp_group = self._pp_cpu_group = None
        self.sp_size, self.dp_size, self.tp_size = p.cp_size, p.dp_size, p.tp_size
        sp, tp, dp = self.sp_size, self.tp_size, self.dp_size
        # rank layout inside the trainer ranks: index = (d * sp + s) * tp + t  (tp fastest)
        self.local_index = self._train_ranks.index(self.rank) if self.rank in self._train_ranks else -1
        li = max(self.local_index, 0)
        if self.pp_size > 1:
            return self._create_pp_groups(li, use_cuda)
        self.tp_rank = li % tp
        self.sp_rank = (li // tp) % sp
        self.dp_rank = li // (tp * sp)
        self._tp_group = None
        self._mp_group = None      # context + tensor parallel peers of one data-parallel rank
        self._all_train_group = None
        tr = self._train_ranks

        def gid(d, s_, t):
            return tr[(d * sp + s_) * tp + t]
        preset = getattr(self, "_preset_groups", None)
        if preset is not None:
            # groups were created collectively by every rank of a trainer / rollout split
            self._shard_group = preset.get("shard") if n > 1 else None
            self._sp_group = preset.get("sp")
            self._dp_group = preset.get("dp")
            self._cpu_group = preset.get("cpu") if n > 1 else None
            self._tp_group = preset.get("tp")
            self._mp_group = preset.get("mp", self._sp_group)
            self._all_train_group = self._shard_group
        elif dist.is_initialized() and n > 1:
            whole = n == self.world_size
            self._all_train_group = dist.group.WORLD if whole else dist.new_group(tr)
            # shard groups: ranks that hold the same tensor-parallel slice
            if tp == 1:
                self._shard_group = self._all_train_group
            else:
                for t in range(tp):
                    ranks = [gid(d, s_, t) for d in range(dp) for s_ in range(sp)]
                    g = dist.new_group(ranks) if len(ranks) > 1 else None
                    if t == self.tp_rank:
                        self._shard_group = g
            for d in range(dp):
                for t in range(tp):
                    ranks = [gid(d, s_, t) for s_ in range(sp)]
                    g = dist.new_group(ranks) if sp > 1 else None
                    if d == self.dp_rank and t == self.tp_rank:
                        self._sp_group = g
            for s_ in range(sp):
                for t in range(tp):
                    ranks = [gid(d, s_, t) for d in range(dp)]
                    g = dist.new_group(ranks) if dp > 1 else None
                    if s_ == self.sp_rank and t == self.tp_rank:
                        self._dp_group = g
            for d in range(dp):
                for s_ in range(sp):
                    ranks = [gid(d, s_, t) for t in range(tp)]
                    g = dist.new_group(ranks) if tp > 1 else None
                    if d == self.dp_rank and s_ == self.sp_rank:
                        self._tp_group = g
            if tp > 1 and sp > 1:
                for d in range(dp):
                    ranks = [gid(d, s_, t) for s_ in range(sp) for t in range(tp)]
                    g = dist.new_group(ranks)
                    if d == self.dp_rank:
                        self._mp_group = g
            else:
                self._mp_group = self._tp_group if tp > 1 else self._sp_group
            self._cpu_group = dist.new_group(tr, backend="gloo") if use_cuda else self._all_train_group
            # statistics are reduced over ranks that saw different tokens only
            self._stats_group = self._cpu_group
            if tp > 1:
                for t in range(tp):
                    ranks = [gid(d, s_, t) for d in range(dp) for s_ in range(sp)]
                    g = dist.new_group(ranks, backend="gloo") if len(ranks) > 1 else None
                    if t == self.tp_rank:
                        self._stats_group = g
            # warm the groups up so the first real collective does not pay connection setup
            t_ = torch.zeros(1, device=self.device)
            dist.all_reduce(t_, group=self._all_train_group)
        else:
            self._shard_group = None
        if not hasattr(self, "_stats_group"):
            self._stats_group = self._cpu_group
        if sp > 1 and tp == 1:
            # sequence-parallel peers evaluate the loss on the same whole micro-batches, so their
            # statistics are copies: only the heads of the data-parallel replicas are reduced
            if preset is not None:
                self._stats_group = preset.get("stats") if self.sp_rank == 0 else None
            elif dist.is_initialized() and n > 1:
                heads = [gid(d, 0, 0) for d in range(dp)]
                g = dist.new_group(heads, backend="gloo") if (dp > 1 and use_cuda) else (dist.new_group(heads) if dp > 1 else None)
                self._stats_group = g if self.sp_rank == 0 else None
        self.ep_size = getattr(p, "ep_size", 1) or 1
        self.ep_rank, self._ep_group, self._edp_group = 0, None, None
        if self.ep_size > 1:
            ep = self.ep_size
            self.etp_size = int(getattr(p, "etp_size", tp) or tp) if tp > 1 else 1
            if sp > 1 or preset is not None:
                raise NotImplementedError("expert parallelism folds into data (and tensor) parallelism: no sequence parallelism, no trainer-rollout split")
            if self.etp_size not in (1, tp):
                raise NotImplementedError(f"expert tensor parallelism must equal the attention tensor parallelism ({tp}) or 1, got {self.etp_size}")
            if self.etp_size == tp:
                # experts are sliced over the tensor-parallel group like a dense MLP and spread over consecutive
                # data-parallel ranks: an EP group holds the ranks of one tensor-parallel slice
                if dp % ep:
                    raise ValueError(f"ep={ep} must divide dp={dp}")
                self.ep_rank = self.dp_rank % ep
                for t in range(tp):
                    for blk in range(dp // ep):
                        g = dist.new_group([gid(blk * ep + e, 0, t) for e in range(ep)])
                        if blk == self.dp_rank // ep and t == self.tp_rank:
                            self._ep_group = g
                    for e in range(ep):                           # replicas of the same experts: their gradients are summed
                        ranks = [gid(blk * ep + e, 0, t) for blk in range(dp // ep)]
                        g = dist.new_group(ranks) if len(ranks) > 1 else None
                        if e == self.ep_rank and t == self.tp_rank:
                            self._edp_group = g
                self._edp_index, self._n_edp = self.dp_rank // ep, dp // ep
                self._export_member = self.dp_rank < ep
            else:
                # whole experts spread over data x tensor ranks (attention keeps its tensor split): the tensor-parallel
                # peers of a replica hold the same tokens, so each routes its own 1 / tp of them
                flat = dp * tp
                if flat % ep:
                    raise ValueError(f"ep={ep} must divide dp * tp = {flat}")
                me = self.dp_rank * tp + self.tp_rank
                self.ep_rank = me % ep
                for blk in range(flat // ep):
                    g = dist.new_group([tr[blk * ep + e] for e in range(ep)])
                    if blk == me // ep:
                        self._ep_group = g
                for e in range(ep):
                    ranks = [tr[blk * ep + e] for blk in range(flat // ep)]
                    g = dist.new_group(ranks) if len(ranks) > 1 else None
                    if e == self.ep_rank:
                        self._edp_group = g
                self._edp_index, self._n_edp = me // ep, flat // ep
                import math

                self._export_member = me < math.lcm(ep, tp)       # whole EP groups and whole TP groups: an export gathers over both
        return self

    def _create_pp_groups(self, li: int, use_cuda: bool):
        """Pipeline x data x tensor parallel layout: index = (stage * dp + d) * tp + t (stages outermost, tensor-parallel
        peers adjacent). Every (stage, tensor slice) shards its optimizer state over its own data-parallel ranks; the
        ranks of one pipeline (all stages and slices of one ``d``) see the same data. Activations travel between the
        ranks that hold the same slice of neighbouring stages: with plain tensor parallelism every slice holds the whole
        hidden state, so no exchange crosses slices."""
        pp, dp, tp, tr = self.pp_size, self.dp_size, self.tp_size, self._train_ranks
        if self.sp_size > 1:
            raise NotImplementedError("pipeline parallelism combines with data and tensor parallelism (no sequence parallelism inside a stage)")
        if getattr(self, "_preset_groups", None) is not None:
            raise NotImplementedError("pipeline parallelism inside a trainer / rollout split")
        self.tp_rank, self.dp_rank, self.pp_rank = li % tp, (li // tp) % dp, li // (tp * dp)
        self.sp_rank = 0
        self._tp_group = self._sp_group = None

        def gid(s_, d, t):
            return tr[(s_ * dp + d) * tp + t]
        self._all_train_group = dist.group.WORLD if len(tr) == self.world_size else dist.new_group(tr)
        self._shard_group = self._dp_group = None
        for s_ in range(pp):
            for t in range(tp):
                ranks = [gid(s_, d, t) for d in range(dp)]
                g = dist.new_group(ranks) if dp > 1 else None
                if s_ == self.pp_rank and t == self.tp_rank:
                    self._shard_group = self._dp_group = g
        for d in range(dp):
            for t in range(tp):
                ranks = [gid(s_, d, t) for s_ in range(pp)]
                g = dist.new_group(ranks)
                gc = dist.new_group(ranks, backend="gloo") if use_cuda else g
                if d == self.dp_rank and t == self.tp_rank:
                    self._pp_group, self._pp_cpu_group = g, gc
        self._mp_group = self._pp_group
        if tp > 1:
            for s_ in range(pp):
                for d in range(dp):
                    g = dist.new_group([gid(s_, d, t) for t in range(tp)])
                    if s_ == self.pp_rank and d == self.dp_rank:
                        self._tp_group = g
            for d in range(dp):                                  # every stage and slice of one replica
                g = dist.new_group([gid(s_, d, t) for s_ in range(pp) for t in range(tp)])
                if d == self.dp_rank:
                    self._mp_group = g
        self._cpu_group = dist.new_group(tr, backend="gloo") if use_cuda else self._all_train_group
        # losses and statistics exist only on the ranks that hold the last stage: the last pipeline rank, or rank 0
        # under the V-shaped placement of the ZBV schedule (two chunks per rank, down the ranks and back up); tensor-
        # parallel peers hold copies, so each slice reduces over its own data-parallel peers
        sched = str(getattr(self.config.archon, "pp_schedule", "1F1B")).lower()
        self._pp_loss_rank = 0 if sched in ("zbv", "zbvzerobubble") else pp - 1
        self._stats_group = None
        for t in range(tp):
            last = [gid(self._pp_loss_rank, d, t) for d in range(dp)]
            g = dist.new_group(last, backend="gloo") if dp > 1 else None
            if self.pp_rank == self._pp_loss_rank and t == self.tp_rank:
                self._stats_group = g
        self.ep_size = getattr(self.parallel, "ep_size", 1) or 1
        self.ep_rank, self._ep_group, self._edp_group = 0, None, None
        if self.ep_size > 1:
            # experts of a stage's MoE layers spread over consecutive data-parallel ranks of that stage
            ep = self.ep_size
            if tp > 1 or dp % ep:
                raise NotImplementedError(f"expert parallelism inside pipeline stages: ep={ep} must divide dp={dp}, no tensor parallelism")
            self.etp_size = 1
            self.ep_rank = self.dp_rank % ep
            for s_ in range(pp):
                for blk in range(dp // ep):
                    g = dist.new_group([gid(s_, blk * ep + e, 0) for e in range(ep)])
                    if s_ == self.pp_rank and blk == self.dp_rank // ep:
                        self._ep_group = g
                for e in range(ep):
                    ranks = [gid(s_, blk * ep + e, 0) for blk in range(dp // ep)]
                    g = dist.new_group(ranks) if len(ranks) > 1 else None
                    if s_ == self.pp_rank and e == self.ep_rank:
                        self._edp_group = g
            self._edp_index, self._n_edp = self.dp_rank // ep, dp // ep
            self._export_member = self.dp_rank < ep
        t_ = torch.zeros(1, device=self.device)
        dist.all_reduce(t_, group=self._all_train_group)
        return self

    def set_train_ranks(self, ranks: list[int], groups: Optional[dict] = None):
        """Restricts the engine to a subset of the global ranks (trainer / rollout split).
        ``groups``: process groups created collectively by all ranks (keys shard, dp, sp, cpu)."""
        self._train_ranks = list(ranks)
        self._preset_groups = groups

    # ------------------------------------------------------------------ init
    def initialize(self, addr: Optional[str] = None, ft_spec: Optional[FinetuneSpec] = None,
                   model_config: Optional[ModelConfig] = None, **kwargs):
        cfg = self.config
        if self.parallel is None:
            self.create_process_group()
        dtype = _dtype_of(cfg.dtype)
        if not self.device.type == "cuda" and dtype != torch.float32:
            dtype = torch.float32  # CPU reference path computes in fp32
        if model_config is None:
            if cfg.model_config:
                mc = dict(cfg.model_config)
                model_config = preset(mc.pop("preset"), **mc) if "preset" in mc else ModelConfig(**mc)
            elif cfg.path and os.path.isdir(cfg.path):
                model_config = ModelConfig.from_pretrained(cfg.path)
            else:
                raise ValueError("no model architecture: give model_config, config.model_config or a checkpoint path")
        if cfg.is_critic:
            model_config.is_critic = True
            model_config.tie_word_embeddings = False
        self.model_config = model_config
        seed = kwargs.get("seed", 1)
        t0 = time.time()
        tp = getattr(self, "tp_size", 1)
        if getattr(model_config, "is_hybrid", False) and tp > 1 and (getattr(self, "sp_size", 1) > 1 or bool(cfg.fsdp.tp_sequence_parallel)):
            raise NotImplementedError("linear-attention (hybrid) models: tensor parallelism does not combine with sequence parallelism")
        if getattr(model_config, "is_hybrid", False) and getattr(cfg.fsdp, "context_parallel", "ulysses") != "ulysses" and getattr(self, "sp_size", 1) > 1:
            raise NotImplementedError("hybrid models split sequences by heads (Ulysses); the delta rule needs whole sequences")
        has_ckpt = (not cfg.init_from_scratch and cfg.path and os.path.isdir(cfg.path)
                    and any(f.endswith(".safetensors") for f in os.listdir(cfg.path)))
        if getattr(self, "pp_size", 1) > 1:
            from ..parallel.pp import PipelineRunner, PipelineStage

            if model_config.is_vlm or cfg.use_lora:
                raise NotImplementedError("pipeline parallelism with vision-language models / LoRA")
            loader = (lambda full: hf_io.load_model_hf(full, cfg.path, strict=not cfg.is_critic)) if has_ckpt else None
            self.local_model_config = model_config
            vpp = max(int(getattr(self.parallel, "virtual_pipeline_parallel_size", 0) or 0), int(cfg.megatron.virtual_pipeline_parallel_size or 1), 1)
            sched_name = str(getattr(cfg.archon, "pp_schedule", "1F1B"))
            zbv = sched_name.lower() in ("zbv", "zbvzerobubble")
            if getattr(self, "ep_size", 1) > 1 and (zbv or vpp > 1 or sched_name.lower() in ("interleaved1f1b", "interleavedzerobubble")):
                raise NotImplementedError("expert parallelism inside pipeline stages runs the one-chunk schedules (1F1B, GPipe, ZBH1)")
            if zbv or vpp > 1 or sched_name.lower() in ("interleaved1f1b", "interleavedzerobubble"):
                # virtual stages: several model chunks per rank, interleaved 1F1B on the timetable runner; ZBV places
                # its two chunks in a V (first and last stage on rank 0) and orders the operations greedily
                from ..parallel.pp import InterleavedStages, ScheduledPipelineRunner

                vpp = 2 if zbv else max(vpp, 2)
                self.model = InterleavedStages(model_config, self.pp_rank, self.pp_size, vpp, dtype=dtype, device=self.device, seed=seed,
                                               init_full=loader, placement="v" if zbv else "loop", tp=tp, tp_rank=self.tp_rank)
                self._pp_runner = ScheduledPipelineRunner(self.model, self._pp_group,
                                                          "ZBV" if zbv else
                                                          "GPipe" if sched_name.lower() == "gpipe" else
                                                          "InterleavedZeroBubble" if "zero" in sched_name.lower() or sched_name.lower() == "zbh1"
                                                          else "Interleaved1F1B")
            else:
                self.model = PipelineStage(model_config, self.pp_rank, self.pp_size, dtype=dtype, device=self.device, seed=seed, init_full=loader,
                                           tp=tp, tp_rank=self.tp_rank)
                # zero-bubble names of the reference map to the split-backward 1F1B (input gradients sent on first,
                # weight gradients in the wait that follows); the V-shaped variant (ZBV) is the branch above
                sched = {"1f1b": "1F1B", "gpipe": "GPipe", "zbh1": "ZBH1", "zerobubble": "ZBH1"}.get(sched_name.lower(), "1F1B")
                self._pp_runner = PipelineRunner(self.model, self._pp_group, schedule=sched)
            if tp > 1:
                from ..parallel import tp as TP

                if model_config.is_moe:
                    raise NotImplementedError("pipeline x tensor parallelism covers dense models")
                TP.install_tp(self.model, self._tp_group, tp, self.tp_rank)
            if self.device.type == "cuda":
                torch.cuda.empty_cache()
        elif tp > 1:
            # every rank materialises the full weights once (same seed / same checkpoint), keeps
            # its slice and drops the rest
            from ..parallel import tp as TP

            full = build_model(model_config, dtype=dtype, device=self.device, seed=seed)
            if has_ckpt:
                hf_io.load_model_hf(full, cfg.path, strict=not cfg.is_critic)
            xtp = getattr(self, "ep_size", 1) == 1 or getattr(self, "etp_size", 1) == tp      # experts sliced over the TP group too
            self.local_model_config = TP.local_config(model_config, tp, expert_tp=xtp)
            self.model = build_model(self.local_model_config, dtype=dtype, device=self.device, seed=seed)
            TP.load_sharded_from_full(self.model, model_config, {n_: p_.detach() for n_, p_ in full.named_parameters()}, tp, self.tp_rank,
                                      expert_tp=xtp)
            tp_sp = bool(cfg.fsdp.tp_sequence_parallel) and not model_config.is_moe
            fused_tp = None
            if tp_sp and self.device.type == "cuda" and cfg.fsdp.fuse_tp_projections and model_config.head_dim in (64, 128):
                from ..parallel.tp_fused import FusedTPLinear

                unit = 128 * tp
                max_t = (max(int(cfg.mb_spec.max_tokens_per_mb or 0), unit) + unit - 1) // unit * unit
                lc = self.local_model_config
                widest = max(model_config.hidden_size, 2 * lc.intermediate_size, (lc.num_heads + 2 * lc.num_kv_heads) * lc.head_dim)
                fused_tp = FusedTPLinear(self._tp_group, self.device, max_t // tp, widest, widest)
            self._tp_fused = fused_tp
            TP.install_tp(self.model, self._tp_group, tp, self.tp_rank, sequence_parallel=tp_sp, fused=fused_tp, expert_tp=xtp)
            del full
            if self.device.type == "cuda":
                torch.cuda.empty_cache()
        else:
            self.local_model_config = model_config
            # sharded parameters with memory_efficient_load: the model is built on the host and only shards reach the device
            on_host = bool(getattr(cfg.fsdp, "shard_parameters", False)) and bool(cfg.fsdp.memory_efficient_load)
            self.model = build_model(model_config, dtype=dtype, device="cpu" if on_host else self.device, seed=seed)
            if has_ckpt:
                hf_io.load_model_hf(self.model, cfg.path, strict=not cfg.is_critic)
        f8 = cfg.archon.fp8 if cfg.archon.fp8.enabled else cfg.megatron.fp8
        if f8.enabled and f8.include_dense and hasattr(self.model, "set_fp8"):
            if tp > 1:
                raise NotImplementedError("fp8 projections with tensor parallelism")
            self.model.set_fp8(True)
        self._expert_param_names: list[str] = []
        if getattr(self, "ep_size", 1) > 1:
            from ..parallel.ep import shard_experts

            if not model_config.is_moe:
                raise ValueError("expert parallelism needs a mixture-of-experts model")
            fused_ep = (self.device.type == "cuda" and (cfg.archon.fuse_ep_dispatch or cfg.megatron.moe_enable_deepep)
                        and os.environ.get("AREAL_EP_FUSED", "1") != "0" and tp == 1 and getattr(self, "pp_size", 1) == 1)
            self._expert_param_names = shard_experts(self.model, self.ep_rank, self.ep_size, self._ep_group, fused=fused_ep,
                                                     device=self.device)
        self.model.gradient_checkpointing = cfg.gradient_checkpointing
        ac = getattr(cfg.archon, "ac_mode", "selective") if not cfg.gradient_checkpointing else "full"
        if getattr(cfg, "activation_checkpointing", None):
            ac = cfg.activation_checkpointing
        if ac in ("selective", "memory_budget") and not cfg.gradient_checkpointing and getattr(cfg, "activation_checkpointing", None) \
                and getattr(self, "pp_size", 1) == 1:
            self.model.set_activation_checkpointing(ac, getattr(cfg, "activation_memory_budget", 0.5))
        self.use_lora = bool(cfg.use_lora) and cfg.optimizer is not None
        if self.use_lora:
            if tp > 1:
                raise NotImplementedError("LoRA with tensor parallelism")
            from ..models.lora import apply_lora

            apply_lora(self.model, cfg.lora_rank, cfg.lora_alpha, cfg.target_modules or None, seed=seed)
        sp = self.sp_size
        # ranks that hold the same tensor-parallel slice shard its optimizer state (ZeRO)
        self._shard_ranks = [self._train_ranks[(d * sp + s_) * tp + self.tp_rank] for d in range(self.dp_size) for s_ in range(sp)] \
            if self.local_index >= 0 else list(self._train_ranks)
        if getattr(self, "pp_size", 1) > 1:
            self._shard_ranks = [self._train_ranks[(self.pp_rank * self.dp_size + d) * tp + self.tp_rank] for d in range(self.dp_size)]
        n_shards = len(self._shard_ranks) if self._shard_group is not None else 1
        shard_rank = (self.dp_rank * sp + self.sp_rank) if n_shards > 1 else 0
        on_gpu = self.device.type == "cuda"
        fused = n_shards > 1 and on_gpu and cfg.fsdp.fuse_reduce_scatter_adamw
        # the parameter buffer may be peer-mapped over a wider group (trainer + rollout ranks)
        psg = kwargs.get("param_symm_group")
        psg_ranks = kwargs.get("param_symm_ranks")
        alloc_g = (lambda n, dt, d: self._symmetric_alloc(n, dt, d, self._shard_group, self._shard_ranks)) if fused else None
        if psg is not None and on_gpu:
            alloc_p = lambda n, dt, d: self._symmetric_alloc(n, dt, d, psg, psg_ranks)
        else:
            alloc_p = alloc_g
        alloc = alloc_g
        self.expert_store = self.expert_optimizer = None
        if self._expert_param_names:
            # experts differ between the ranks of an EP group: their own flat space, sharded over
            # the ranks that hold the SAME experts; everything else is sharded over all ranks
            fused, alloc_g, alloc_p, alloc = False, None, None, None
            expert = set(self._expert_param_names)
            self.expert_store = FlatParamStore(self.model, self._n_edp, self._edp_index, torch.float32,
                                               with_grads=cfg.optimizer is not None, include=lambda n: n in expert)
        _expert_set = frozenset(self._expert_param_names)
        dense_only = (lambda n: n not in _expert_set) if _expert_set else None
        self._z3 = None
        if bool(getattr(cfg.fsdp, "shard_parameters", False)):
            # ZeRO-3: parameters and gradients sharded as well, decoder layers materialised one at a time
            if getattr(self, "pp_size", 1) > 1 or getattr(self, "ep_size", 1) > 1 or self.use_lora or (tp > 1 and bool(cfg.fsdp.tp_sequence_parallel)):
                raise NotImplementedError("fsdp.shard_parameters covers data / sequence / tensor parallel models (no pp / ep, LoRA or "
                                          "sequence-parallel residual stream); an image tower stays resident with the embedding for a micro-batch")
            from .sharded_params import ShardedParamStore

            fused, alloc = False, None
            self.store = self._z3 = ShardedParamStore(self.model, n_shards, shard_rank, self._shard_group if n_shards > 1 else None,
                                                      self._shard_ranks if n_shards > 1 else None, torch.float32,
                                                      with_grads=cfg.optimizer is not None, device=self.device)
            self.model.param_units = self.store
            if tp > 1:
                # every TP slice shards its own weights over its data-parallel ranks; partial gradients of replicated
                # parameters are summed over the TP group before a unit's gradients leave for their owners
                from ..parallel import tp as TP

                partial = TP.partial_grad_names(self.model)

                def sum_partial(names, params, group=self._tp_group):
                    for n_, p_ in zip(names, params):
                        if n_ in partial and getattr(p_, "main_grad", None) is not None:
                            dist.all_reduce(p_.main_grad, group=group)
                self.store.grad_hook = sum_partial
        else:
            self.store = FlatParamStore(self.model, n_shards, shard_rank, torch.float32, alloc_param=alloc_p, alloc_grad=alloc_g,
                                        with_grads=cfg.optimizer is not None, only_trainable=self.use_lora, include=dense_only)
        if on_gpu:
            torch.cuda.empty_cache()        # the parameters' first home (before the flat buffer) goes back to the driver
        if n_shards > 1:
            # identical initial weights on every rank of the shard group
            if self._z3 is None:
                dist.broadcast(self.store.flat_param, src=self._shard_ranks[0], group=self._shard_group)
        if tp > 1 and cfg.optimizer is not None:
            self._replicated_ranges = self._find_replicated_ranges()
        if getattr(self, "pp_size", 1) > 1 and cfg.optimizer is not None:
            # the last stage's copy of a tied embedding must not count twice in the global norm
            self._tp_replicated_ranges = self._replicated_ranges if tp > 1 else []
            self._replicated_ranges = []
            m = self.model
            if m.is_last and not m.is_first and m.embed_tokens is not None and m.lm_head is None and not model_config.is_critic:
                lo, hi = self.store.shard_range
                tied = [n for n in self.store.names if n.endswith("embed_tokens")][-1]   # the last stage's copy
                off, numel = self.store.locate(tied)
                a, b = max(off, lo), min(off + numel, hi)
                if a < b:
                    self._replicated_ranges.append((a - lo, b - lo))
        if cfg.optimizer is not None:
            total = ft_spec.total_train_steps if ft_spec is not None else 1
            self.optimizer = ShardedAdamW(self.store, cfg.optimizer, total_steps=total, group=self._shard_group)
            if self.expert_store is not None:
                self.expert_optimizer = ShardedAdamW(self.expert_store, cfg.optimizer, total_steps=total, group=self._edp_group)
        if model_config.is_vlm and ((tp > 1 and (self.sp_size > 1 or getattr(self, "pp_size", 1) > 1 or bool(cfg.fsdp.tp_sequence_parallel)))
                                    or (self.sp_size > 1 and getattr(cfg.fsdp, "context_parallel", "ulysses") != "ulysses")):
            raise NotImplementedError("vision-language models run with data parallelism plus either Ulysses sequence parallelism or plain "
                                      "tensor parallelism of the language model (the image tower stays whole; no zig-zag / pipeline split)")
        self._cp_zigzag = self.sp_size > 1 and getattr(cfg.fsdp, "context_parallel", "ulysses") == "zigzag"
        self._zz_perm = None
        if getattr(cfg.fsdp, "context_parallel", "ulysses") not in ("ulysses", "zigzag"):
            raise ValueError("fsdp.context_parallel must be ulysses or zigzag")
        if self._cp_zigzag:
            self._sp_fused = None
            if tp > 1 or getattr(self, "pp_size", 1) > 1:
                raise NotImplementedError("zig-zag context parallelism combines with data parallelism only")
        elif self.sp_size > 1:
            from ..parallel.ulysses import install_ulysses

            install_ulysses(self.model, self._sp_group, self.sp_size, self.sp_rank)
            if model_config.is_vlm:
                if getattr(cfg.fsdp, "shard_vision_across_sp", True):
                    self.model.vision_sp = (self._sp_group, self.sp_size, self.sp_rank)    # pictures split over the group too
            self._sp_fused = None
            mc = model_config
            if (on_gpu and cfg.fsdp.fuse_ulysses_projections and not self.use_lora and tp == 1 and self.sp_size <= 8 and not getattr(mc, "is_hybrid", False) and not mc.is_vlm
                    and mc.num_heads % sp == 0 and mc.num_kv_heads % sp == 0 and not mc.attention_bias and mc.head_dim in (64, 128)
                    and ((mc.num_heads + 2 * mc.num_kv_heads) // sp * mc.head_dim) % 64 == 0):
                from ..parallel.tp_fused import FusedUlyssesLinear
                from ..parallel.ulysses import install_fused_ulysses

                unit = 128 * sp
                max_t = (max(int(cfg.mb_spec.max_tokens_per_mb or 0), unit) + unit - 1) // unit * unit
                cols = max(mc.hidden_size, (mc.num_heads + 2 * mc.num_kv_heads) * mc.head_dim)
                self._sp_fused = FusedUlyssesLinear(self._sp_group, self.device, max_t // sp, cols)
                install_fused_ulysses(self.model, self._sp_fused)
        if alloc is not None:
            from ..parallel.fused_zero import FusedGradReducer

            mc = 0
            if cfg.fsdp.reduce_in_switch or os.environ.get("AREAL_NVLS_REDUCE", "0") == "1":
                # in-switch reduction (NVLS) when the symmetric allocation came with a multicast mapping
                mc = int(getattr(self._symm_handles[self.store.flat_grad.data_ptr()][0], "multicast_ptr", 0) or 0)
                logger.info("gradient reduce-scatter through the NVLink switch: %s", "on" if mc else "no multicast mapping, peer loads")
            self._grad_reducer = FusedGradReducer(self.store, self._shard_group,
                                                  self.peer_ptrs(self.store.flat_grad, self._shard_ranks),
                                                  self.peer_ptrs(self.store.flat_param, self._shard_ranks), grad_multicast_ptr=mc)
        self._initialized = True
        logger.info("initialised %s: %.2fB params, dtype %s, dp=%d sp=%d, %.1fs", model_config.arch,
                    model_config.num_params() / 1e9, dtype, self.dp_size, self.sp_size, time.time() - t0)
        return self

    def _find_replicated_ranges(self) -> list[tuple[int, int]]:
        """Ranges (relative to this rank's gradient shard) that belong to parameters every
        tensor-parallel rank holds in full: they count once in the global gradient norm."""
        from ..parallel.tp import replicated_parameter_names

        lo, hi = self.store.shard_range
        out = []
        for name in replicated_parameter_names(self.model):
            off, numel = self.store.locate(name)
            a, b = max(off, lo), min(off + numel, hi)
            if a < b:
                out.append((a - lo, b - lo))
        return out

    _symm_handles: dict = {}

    def _symmetric_alloc(self, n: int, dtype, device, group, group_ranks):
        """Allocates a buffer that every rank of ``group`` can address (peer pointers) for the
        fused reduce-scatter / parameter write-back / weight-push kernels."""
        from ..parallel.symm import symm_empty

        t, hdl = symm_empty(n, dtype, device, group)
        t.zero_()
        self._symm_handles = dict(self._symm_handles)
        self._symm_handles[t.data_ptr()] = (hdl, list(group_ranks))
        return t

    def peer_ptrs(self, tensor: torch.Tensor, global_ranks: list[int]) -> list[int]:
        """Addresses (in this process) of the peers' copies of a symmetric buffer."""
        hdl, ranks = self._symm_handles[tensor.data_ptr()]
        ptrs = list(hdl.buffer_ptrs)
        return [ptrs[ranks.index(r)] for r in global_ranks]

    def destroy(self):
        self.model = None
        self.store = None
        self.optimizer = None
        if self._own_pg and dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass
        self._initialized = False

    # ------------------------------------------------------------------ topology
    @property
    def data_parallel_group(self):
        return self._dp_group

    @property
    def data_parallel_rank(self) -> int:
        return self.dp_rank

    @property
    def data_parallel_world_size(self) -> int:
        return self.dp_size

    def current_data_parallel_head(self) -> int:
        if getattr(self, "pp_size", 1) > 1:
            return self._train_ranks[self.dp_rank * getattr(self, "tp_size", 1)]          # first stage (first slice) of this rank's pipeline
        return self._train_ranks[self.dp_rank * self.sp_size * getattr(self, "tp_size", 1)]

    def is_data_parallel_head(self) -> bool:
        return self.sp_rank == 0 and getattr(self, "tp_rank", 0) == 0 and getattr(self, "pp_rank", 0) == 0

    @property
    def pipeline_parallel_group(self):
        return getattr(self, "_pp_group", None)

    def is_pipeline_last_stage(self) -> bool:
        return getattr(self, "pp_size", 1) == 1 or self.pp_rank == getattr(self, "_pp_loss_rank", self.pp_size - 1)

    @property
    def context_and_model_parallel_group(self):
        return self._mp_group if getattr(self, "_mp_group", None) is not None else self._sp_group

    @property
    def tensor_parallel_group(self):
        return getattr(self, "_tp_group", None)

    @property
    def cpu_group(self):
        return self._cpu_group

    # ------------------------------------------------------------------ modes / versions
    def train(self, mode: bool = True):
        self.model.train(mode)
        return self

    def set_version(self, version: int):
        self._version = version

    def get_version(self) -> int:
        return self._version

    # ------------------------------------------------------------------ micro-batches
    def _align(self) -> int:
        base = D.N_TOKENS_PER_PAGE if self.device.type == "cuda" else 1
        if getattr(self, "_sp_fused", None) is not None:
            return max(base, 128 * self.sp_size)   # the fused projections work on 128-row blocks per rank
        if getattr(self.model, "tp_sequence_parallel", False):
            import math

            return math.lcm(base, (128 if getattr(self, "_tp_fused", None) is not None else 1) * self.tp_size)
        return base * self.sp_size if self.sp_size > 1 and base % self.sp_size else max(base, self.sp_size)

    def _prepare_mb_list(self, input_: dict[str, Any]) -> D.MicroBatchList:
        assert "attention_mask" in input_ and "input_ids" in input_, "expected a padded batch"
        input_ = D.amend_position_ids(dict(input_))
        spec = self.config.mb_spec
        if getattr(self, "pp_size", 1) > 1 and getattr(self.model, "n_chunks", 1) > 1 and spec.n_mbs_divisor % self.pp_size:
            import dataclasses
            import math as _math

            # interleaved 1F1B walks the micro-batches in groups of the pipeline size
            spec = dataclasses.replace(spec, n_mbs_divisor=_math.lcm(max(1, spec.n_mbs_divisor), self.pp_size))
        mbl = D.split_padded_tensor_dict_into_mb_list(input_, spec, group=self._cpu_group if self.dp_size > 1 else None)
        D.pad_mb_list(mbl, pad_to_maximum=self.config.pad_to_maximum, max_tokens=self.config.mb_spec.max_tokens_per_mb,
                      align=self._align())
        return mbl

    def _mb_to_device(self, mb: dict[str, Any]) -> dict[str, Any]:
        out = {}
        for k, v in mb.items():
            if torch.is_tensor(v):
                if v.device != self.device:
                    v = v.pin_memory() if (self.device.type == "cuda" and not v.is_pinned() and v.numel() > 0) else v
                    v = v.to(self.device, non_blocking=True)
                out[k] = v
            else:
                out[k] = v
        return out

    def _forward_mb(self, mb: dict[str, Any]):
        """Runs the model on one padded packed micro-batch (already on the device). Returns
        hidden states for the local sequence-parallel slice plus the matching labels."""
        ids = mb["input_ids"].to(torch.int32) if self.device.type == "cuda" else mb["input_ids"].long()
        cu = mb["cu_seqlens"]
        T = ids.shape[0]
        pos = mb.get("position_ids")
        if pos is None or pos.shape[0] != T:
            pos = D.positions_from_cu_seqlens(cu, T)
        labels = torch.roll(ids, shifts=-1, dims=0)
        pb = PackedBatch(cu, pos, T, int(mb.get("max_seqlen", 0)))
        if getattr(self.config, "enable_tree_training", False):
            # prefix sharing: sequences of the micro-batch that start alike (the samples of a group share their
            # prompt) are merged into a trie, every distinct (prefix, token) runs through the layers once, and
            # the per-token hidden states are read back from the trie nodes (reference:
            # areal/engine/fsdp_engine.py tree-training branch over areal/models/tree_attn/*)
            if self.sp_size > 1 or getattr(self, "pp_size", 1) > 1 or getattr(self, "tp_size", 1) > 1:
                raise NotImplementedError("tree training runs with data parallelism only")
            from ..models.tree_attn import tree_hidden_for_packed_batch

            hidden, saving = tree_hidden_for_packed_batch(self.model, ids, cu, pad_to=self._align())
            self._tree_saving = saving
            stats_tracker.scalar(tree_token_saving=saving)
            return hidden, labels, slice(0, T)
        if self.sp_size > 1 and self._cp_zigzag:
            return self._forward_mb_zigzag(ids, labels, cu, T)
        if self.sp_size == 1 and getattr(self.model, "tp_sequence_parallel", False):
            # the layers keep this rank's rows of the residual stream; attention sees all tokens (its heads)
            chunk = T // self.tp_size
            sl = slice(self.tp_rank * chunk, (self.tp_rank + 1) * chunk)
            hidden = self.model.forward_hidden(ids[sl], pb)
            return hidden, labels[sl], sl
        if self.sp_size > 1:
            chunk = T // self.sp_size
            sl = slice(self.sp_rank * chunk, (self.sp_rank + 1) * chunk)
            pb_local = PackedBatch(cu, pos[sl], T, pb.max_seqlen)
            pb_local.tile_info = pb.tile_info
            pb_local.full_position_ids = pb.position_ids
            if getattr(self.model.cfg, "is_vlm", False):
                from ..models.vlm import collect_multi_modal

                mm = collect_multi_modal(mb.get("multi_modal_input"))
                if mm is not None:
                    mm = {k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in mm.items()}
                hidden = self.model.forward_hidden(ids, pb_local, mm=mm, row_slice=sl)
            else:
                hidden = self.model.forward_hidden(ids[sl], pb_local)
            return hidden, labels[sl], sl
        if getattr(self.model.cfg, "is_vlm", False):
            from ..models.vlm import collect_multi_modal

            mm = collect_multi_modal(mb.get("multi_modal_input"))
            if mm is not None:
                mm = {k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in mm.items()}
            hidden = self.model.forward_hidden(ids, pb, mm=mm)
        else:
            hidden = self.model.forward_hidden(ids, pb)
        return hidden, labels, slice(0, T)

    def _forward_mb_zigzag(self, ids, labels, cu, T):
        """Context parallelism by sequence chunks: every sequence is cut into ``2 * cp`` chunks, this rank runs the
        layers on chunks ``r`` and ``2 cp - 1 - r`` of every sequence and attends to the gathered keys / values chunk
        pair by chunk pair (``parallel/cp.py``). Per-token outputs are gathered and put back into the packed order
        by :meth:`_sp_gather`, so the loss sees whole sequences exactly as under Ulysses."""
        import math

        from ..parallel import cp as CP

        sp, r = self.sp_size, self.sp_rank
        cu_host = cu.cpu()
        src, pos_l, local_lens = CP.zigzag_indices(cu_host, sp, r)
        T_local = int(src.numel())
        srcd = src.to(self.device)
        pad = srcd < 0
        ids_l = ids[srcd.clamp(min=0)].masked_fill(pad, 0)
        labels_l = labels[srcd.clamp(min=0)].masked_fill(pad, 0)
        cu_l = torch.tensor([0] + list(torch.tensor(local_lens).cumsum(0)), dtype=torch.int32, device=self.device)
        pb_l = PackedBatch(cu_l, pos_l.to(self.device).int(), T_local, max(CP.padded_lengths(cu_host, sp)))
        scale = 1.0 / math.sqrt(self.model.cfg.head_dim)
        group = self._sp_group

        def attn(q, k, v):
            return CP.cp_attention(q, k, v, cu_host, sp, r, group, scale)
        hidden = self.model.forward_hidden(ids_l, pb_l, attn_fns=[attn] * len(self.model.layers))
        perm = torch.full((T,), -1, dtype=torch.long)
        for peer in range(sp):
            s_p = src if peer == r else CP.zigzag_indices(cu_host, sp, peer)[0]
            ok = s_p >= 0
            perm[s_p[ok]] = (peer * T_local + torch.arange(T_local))[ok]
        self._zz_perm = perm.to(self.device)
        return hidden, labels_l, slice(0, T_local)

    # ------------------------------------------------------------------ train / eval / forward
    def optimizer_zero_grad(self):
        self.store.zero_grad()
        if getattr(self, "expert_store", None) is not None:
            self.expert_store.zero_grad()

    def forward_backward_batch(self, mb_list: D.MicroBatchList, process_output_fn: Callable, forward_only: bool = False):
        """Runs every micro-batch; ``process_output_fn(hidden, labels, mb, pad_len, sl)`` returns a
        loss (training) or an output (forward only)."""
        if getattr(self, "pp_size", 1) > 1:
            return self._pp_forward_backward(mb_list, process_output_fn, forward_only)
        outs = []
        z3 = getattr(self, "_z3", None)
        for mb, pad in zip(mb_list.padded_mbs, mb_list.padding_lengths):
            mbd = self._mb_to_device(mb)
            if z3 is not None:
                z3.begin(train=not forward_only)     # embedding / head stay for the micro-batch, layers come and go
            try:
                if forward_only:
                    with torch.no_grad():
                        hidden, labels, sl = self._forward_mb(mbd)
                        outs.append(process_output_fn(hidden, labels, mbd, pad, sl))
                else:
                    hidden, labels, sl = self._forward_mb(mbd)
                    loss = process_output_fn(hidden, labels, mbd, pad, sl)
                    aux = self.model.aux_loss()
                    if aux is not None:
                        loss = loss + aux
                    loss.backward()
                    outs.append(loss.detach())
            finally:
                if z3 is not None:
                    z3.end(train=not forward_only)
        return outs

    def _pp_forward_backward(self, mb_list: D.MicroBatchList, process_output_fn: Callable, forward_only: bool):
        """Micro-batches through this rank's pipeline (every stage holds the same micro-batches).
        Losses / outputs exist on the last stage; the other stages return ``[]``."""
        mbs = []
        for mb, pad in zip(mb_list.padded_mbs, mb_list.padding_lengths):
            mbd = self._mb_to_device(mb)
            ids = mbd["input_ids"].to(torch.int32) if self.device.type == "cuda" else mbd["input_ids"].long()
            T = ids.shape[0]
            pos = mbd.get("position_ids")
            if pos is None or pos.shape[0] != T:
                pos = D.positions_from_cu_seqlens(mbd["cu_seqlens"], T)
            mbs.append(dict(input_ids=ids, pb=PackedBatch(mbd["cu_seqlens"], pos, T, int(mbd.get("max_seqlen", 0))),
                            labels=torch.roll(ids, shifts=-1, dims=0), mbd=mbd, pad=pad))

        def last_stage(hidden, mb):
            out = process_output_fn(hidden, mb["labels"], mb["mbd"], mb["pad"], slice(0, mb["input_ids"].shape[0]))
            if not forward_only:
                aux = self.model.aux_loss()
                if aux is not None:
                    out = out + aux
            return out

        return self._pp_runner.run(mbs, last_stage, forward_only=forward_only)

    def _pp_share(self, outs: list):
        """Results of the last pipeline stage made known to every stage of this pipeline."""
        if getattr(self, "pp_size", 1) == 1:
            return outs
        box = [outs if self.is_pipeline_last_stage() else None]
        tp = getattr(self, "tp_size", 1)
        src = self._train_ranks[(getattr(self, "_pp_loss_rank", self.pp_size - 1) * self.dp_size + self.dp_rank) * tp + getattr(self, "tp_rank", 0)]
        dist.broadcast_object_list(box, src=src, group=self._pp_cpu_group)
        return box[0]

    def _slice_mb(self, mb: dict[str, Any], sl: slice, pad: int) -> dict[str, Any]:
        """Per-token fields restricted to the local sequence-parallel slice."""
        T = mb["input_ids"].shape[0]
        out = {}
        for k, v in mb.items():
            if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == T and k != "cu_seqlens":
                out[k] = v[sl]
            else:
                out[k] = v
        return out

    def _row_split(self):
        """(group, size, rank) over which a micro-batch's tokens are split by rows: the Ulysses / context-parallel
        group, or the tensor-parallel group when its residual stream is sequence parallel; size 1 otherwise."""
        if self.sp_size > 1:
            return self._sp_group, self.sp_size, self.sp_rank
        if getattr(self.model, "tp_sequence_parallel", False):
            return self._tp_group, self.tp_size, self.tp_rank
        return None, 1, 0

    def _sp_gather(self, t: torch.Tensor) -> torch.Tensor:
        g, n, r = self._row_split()
        if self.sp_size <= 1 and n > 1:
            return _GatherOverSP.apply(t, g, r, n)
        if self.sp_size <= 1:
            return t
        full = _GatherOverSP.apply(t, self._sp_group, self.sp_rank, self.sp_size)
        return self._sp_restore(full)

    def _sp_restore(self, full: torch.Tensor) -> torch.Tensor:
        """Rank-major concatenation of the ranks' local outputs -> packed order of the micro-batch (the identity
        under Ulysses, whose ranks hold consecutive slices)."""
        if getattr(self, "_cp_zigzag", False) and self._zz_perm is not None:
            return full.index_select(0, self._zz_perm)
        return full

    def _actor_outputs(self, hidden, labels, temperature=None):
        t = self.config.temperature if temperature is None else temperature
        return self.model.logprobs_entropy(hidden, labels, t, chunk=max(256, self.config.logprobs_chunk_size))

    def train_batch(self, input_: dict[str, Any], loss_fn: Callable[..., torch.Tensor],
                    loss_weight_fn: Callable[[dict[str, Any]], torch.Tensor]) -> dict[str, float]:
        assert self.optimizer is not None, "engine was initialised without an optimizer"
        self.model.train()
        self.optimizer_zero_grad()
        mbl = self._prepare_mb_list(input_)
        weights = [float(loss_weight_fn(mb)) for mb in mbl.mbs]
        total_w = torch.tensor([sum(weights)], dtype=torch.float64)
        if self.dp_size > 1:
            tw = total_w.to(self.device) if self.device.type == "cuda" and dist.get_backend(self._dp_group) == "nccl" else total_w
            dist.all_reduce(tw, group=self._dp_group)
            total_w = tw.cpu()
        total_weight = float(total_w[0])
        if total_weight <= 0:
            raise ValueError("total loss weight is zero: nothing to train on")
        it = iter(weights)

        def process(hidden, labels, mb, pad, sl):
            w = next(it)
            # sequence-parallel ranks gather the per-token outputs and evaluate the loss on the WHOLE
            # micro-batch (sequence-level losses, pair sums and sorts need whole sequences)
            if self.config.is_critic:
                loss = loss_fn(self._sp_gather(self.model.values(hidden)), mb)
            else:
                logp, ent = self._actor_outputs(hidden, labels)
                loss = loss_fn(self._sp_gather(logp), self._sp_gather(ent), mb)
            # sum over data-parallel ranks of (w_mb / W_total) * mean-loss_mb == global weighted mean
            return loss * (w / total_weight)

        losses = self.forward_backward_batch(mbl, process)
        stats = self.optimizer_step()
        stats["loss"] = float(torch.stack(losses).sum()) if losses else 0.0
        self.d2h_bytes += 4
        if getattr(self, "pp_size", 1) > 1:
            stats["loss"] = float(self._pp_runner.broadcast_loss(torch.tensor(stats["loss"])))
        return stats

    def optimizer_step(self) -> dict[str, float]:
        hook = getattr(self, "before_optimizer_step", None)
        if hook is not None:
            hook()
        self.store.fold_autograd_grads()
        if getattr(self, "expert_store", None) is not None:
            return self._ep_optimizer_step()
        opt = self.optimizer
        tp = getattr(self, "tp_size", 1)
        if getattr(self, "_z3", None) is not None:
            # gradients were reduced to their owners unit by unit during the backward; the updated shard stays put
            pre = None
            if tp > 1:
                g32 = self.store.grad_shard.float()
                rep = sum((g32[a:b].pow(2).sum() for a, b in self._replicated_ranges), torch.zeros((), device=self.device))
                pre = (g32.pow(2).sum() - rep + rep / tp).reshape(1)        # replicated parameters count once over the TP group
                dist.all_reduce(pre, group=self._all_train_group)
            res = opt.step(self.store.grad_shard, precomputed_sumsq=pre)
            if self.model.cfg.is_moe and self.model.cfg.router_bias_update_rate > 0:
                for layer in self.model.layers:
                    upd = getattr(layer.mlp, "update_expert_bias", None)
                    if upd is not None:
                        upd(self._shard_group)
            st = self._read_step_state(res["state"])
            self.last_step_stats = dict(update_successful=float(st[2]), grad_norm=float(st[3]), lr=float(res["lr"]))
            return dict(self.last_step_stats)
        tp = getattr(self, "tp_size", 1)
        if tp > 1:
            from ..parallel.tp import allreduce_replicated_grads

            allreduce_replicated_grads(self.model, self._tp_group)
        pp = getattr(self, "pp_size", 1)
        fused = (self._grad_reducer is not None and not opt.sgd and not opt.bf16_state and not opt.offload
                 and tp == 1 and pp == 1)
        if self._shard_group is not None:
            if fused:
                gshard = self._grad_reducer.reduce_scatter(opt.state)
            elif self._grad_reducer is not None:
                gshard = self._grad_reducer.reduce_scatter()
            else:
                if dist.get_backend(self._shard_group) == "nccl":
                    gshard = torch.empty_like(self.store.grad_shard)
                    dist.reduce_scatter_tensor(gshard, self.store.flat_grad, group=self._shard_group)
                else:
                    dist.all_reduce(self.store.flat_grad, group=self._shard_group)
                    gshard = self.store.grad_shard
        else:
            gshard = self.store.grad_shard
        if fused:
            from ..ops import functional as OF

            OF.clip_coef_(opt.state, float(opt.cfg.gradient_clipping or 0.0), 1.0)
            opt.step_count += 1
            lr = opt.current_lr()
            self._grad_reducer.adamw_and_all_gather(opt, opt.state, lr)
            res = {"state": opt.state, "lr": lr}
        else:
            pre = None
            if pp > 1:
                # global norm^2 = sum over every stage's shards; a tied embedding's second copy is left out
                pre = torch.zeros(1, dtype=torch.float32, device=self.device)
                g32 = gshard.float()
                zero = torch.zeros((), device=self.device)
                if tp > 1:
                    # parameters that every tensor-parallel slice holds in full count once (1 / tp from each slice); the
                    # tied copy is left out first, whether sliced or not
                    keep = torch.ones_like(g32)
                    for a, b in self._tp_replicated_ranges:
                        keep[a:b] = 1.0 / tp
                    for a, b in self._replicated_ranges:
                        keep[a:b] = 0.0
                    pre[0] = (g32.pow(2) * keep).sum()
                else:
                    pre[0] = g32.pow(2).sum() - sum((g32[a:b].pow(2).sum() for a, b in self._replicated_ranges), zero)
                dist.all_reduce(pre, group=self._all_train_group)
            elif tp > 1:
                # global norm^2 = sum over TP ranks of the sliced parameters' part + the replicated
                # parameters' part counted once
                pre = torch.zeros(1, dtype=torch.float32, device=self.device)
                g32 = gshard.float()
                tot = g32.pow(2).sum()
                rep = sum((g32[a:b].pow(2).sum() for a, b in self._replicated_ranges), torch.zeros((), device=self.device))
                pre[0] = tot - rep + rep / tp
                dist.all_reduce(pre, group=self._all_train_group)
            res = opt.step(gshard, precomputed_sumsq=pre)
            if self._shard_group is not None:
                if self._grad_reducer is not None:
                    self._grad_reducer.all_gather_params()
                else:
                    dist.all_gather_into_tensor(self.store.flat_param, self.store.param_shard.clone(), group=self._shard_group)
        if self.model.cfg.is_moe and self.model.cfg.router_bias_update_rate > 0:
            # auxiliary-loss-free balancing: selection biases follow the expert load of this step
            for layer in self.model.layers:
                upd = getattr(layer.mlp, "update_expert_bias", None)
                if upd is not None:
                    upd(self._shard_group)
        st = self._read_step_state(res["state"])
        self.last_step_stats = dict(update_successful=float(st[2]), grad_norm=float(st[3]), lr=float(res["lr"]))
        return dict(self.last_step_stats)

    def _read_step_state(self, state: torch.Tensor) -> list:
        """The optimizer's 4-float status, read at the one host synchronisation of the step. The
        device error word travels with it: a bounded wait that gave up anywhere in this step (a peer
        that never signalled, a lost copy) means gradients or parameters may be incomplete. Every
        trainer rank learns of it (MAX over the host group) and raises, so no rank carries on alone."""
        poll = None
        if self.device.type == "cuda":
            if self._err_poll is None:
                from ..ops import lib as oplib

                self._err_poll = oplib.ErrorPoller()
            poll = self._err_poll
            poll.enqueue()
        st = state.tolist()
        self.d2h_bytes += state.numel() * state.element_size()
        code = poll.value() if poll is not None else 0
        if self._cpu_group is not None and os.environ.get("AREAL_SKIP_ERROR_EXCHANGE", "0") != "1":
            t = torch.tensor([code], dtype=torch.int32)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self._cpu_group)
            code = max(code, int(t[0]))
        if code != 0:
            from ..ops import lib as oplib

            if poll is not None:
                poll.pending = False
            oplib.kernel_error()        # clear the local word
            raise oplib.KernelWaitTimeout(f"optimizer step: a device-side wait gave up on some trainer rank (code {code}: "
                                          f"{oplib.KERNEL_ERROR_NAMES.get(code, 'unknown')}); the step's update must not be used")
        if poll is not None:
            poll.pending = False
        return st

    def use_library_collectives(self, on: bool = True) -> None:
        """Switches this engine between its fused peer-memory kernels and the library-collective
        path at a step boundary (all trainer ranks must switch at the same step): NCCL
        reduce-scatter + all-gather around the optimizer, NCCL all-to-all around attention, NCCL
        broadcast for the weight update. Used to measure the fused path against that baseline."""
        if on:
            if getattr(self, "_fused_saved", None) is None:
                self._fused_saved = dict(reducer=self._grad_reducer, sp=getattr(self, "_sp_fused", None), pusher=self._weight_pusher)
            self._grad_reducer = None
            if getattr(self, "_sp_fused", None) is not None:
                from ..parallel.ulysses import install_fused_ulysses

                install_fused_ulysses(self.model, None)
            if self._weight_pusher is not None and hasattr(self.rollout_engine, "remote_ranks"):
                from ..parallel.weight_push import BroadcastWeightPusher

                old = self._weight_pusher
                new = BroadcastWeightPusher(self, self.rollout_engine, self.rollout_engine.wu_group)
                new.seq = old.seq
                self._weight_pusher = new
        elif getattr(self, "_fused_saved", None) is not None:
            sv = self._fused_saved
            self._grad_reducer = sv["reducer"]
            if sv["sp"] is not None:
                from ..parallel.ulysses import install_fused_ulysses

                install_fused_ulysses(self.model, sv["sp"])
            if sv["pusher"] is not None:
                sv["pusher"].seq = self._weight_pusher.seq
                self._weight_pusher = sv["pusher"]
            self._fused_saved = None

    def _reduce_scatter_flat(self, store, group):
        """Sum of ``store.flat_grad`` over ``group``; returns this rank's shard."""
        if group is None or dist.get_world_size(group) == 1:
            return store.grad_shard
        if dist.get_backend(group) == "nccl":
            out = torch.empty_like(store.grad_shard)
            dist.reduce_scatter_tensor(out, store.flat_grad, group=group)
            return out
        dist.all_reduce(store.flat_grad, group=group)
        return store.grad_shard

    @staticmethod
    def _all_gather_flat(store, group):
        if group is not None and dist.get_world_size(group) > 1:
            dist.all_gather_into_tensor(store.flat_param, store.param_shard.clone(), group=group)

    def _ep_optimizer_step(self) -> dict[str, float]:
        """Expert parallelism: the dense parameters' gradients are summed over all ranks, the
        experts' over the replicas of the same experts; one global norm clips both."""
        es = self.expert_store
        es.fold_autograd_grads()
        tp = getattr(self, "tp_size", 1)
        if tp > 1:
            from ..parallel.tp import allreduce_replicated_grads

            allreduce_replicated_grads(self.model, self._tp_group)
        g_dense = self._reduce_scatter_flat(self.store, self._shard_group)
        g_exp = self._reduce_scatter_flat(es, self._edp_group)
        d32 = g_dense.float()
        dense_sq = d32.pow(2).sum()
        if tp > 1:
            # parameters that every tensor-parallel rank holds in full count once; every expert element (whole or
            # sliced) lives in exactly one rank's shard
            rep = sum((d32[a:b].pow(2).sum() for a, b in self._replicated_ranges), torch.zeros((), device=self.device))
            dense_sq = dense_sq - rep + rep / tp
        elif getattr(self, "pp_size", 1) > 1:
            # the last stage's copy of a tied embedding is left out
            dense_sq = dense_sq - sum((d32[a:b].pow(2).sum() for a, b in self._replicated_ranges), torch.zeros((), device=self.device))
        pre = (dense_sq + g_exp.float().pow(2).sum()).reshape(1)
        if self._all_train_group is not None:
            dist.all_reduce(pre, group=self._all_train_group)     # every shard of either kind lives on exactly one rank
        res = self.optimizer.step(g_dense, precomputed_sumsq=pre)
        self.expert_optimizer.step(g_exp, precomputed_sumsq=pre)
        self._all_gather_flat(self.store, self._shard_group)
        self._all_gather_flat(es, self._edp_group)
        if self.model.cfg.router_bias_update_rate > 0:
            for layer in self.model.layers:
                upd = getattr(layer.mlp, "update_expert_bias", None)
                if upd is not None:
                    # whole experts under tensor-parallel attention: every rank counted its own share of the tokens
                    upd(self._all_train_group if tp > 1 and getattr(self, "etp_size", 1) != tp else self._shard_group)
        st = self._read_step_state(res["state"])
        self.last_step_stats = dict(update_successful=float(st[2]), grad_norm=float(st[3]), lr=float(res["lr"]))
        return dict(self.last_step_stats)

    def lr_scheduler_step(self):
        if self.optimizer is not None:
            self.optimizer.lr_scheduler_step()
        if getattr(self, "expert_optimizer", None) is not None:
            self.expert_optimizer.lr_scheduler_step()

    @torch.no_grad()
    def eval_batch(self, input_: dict[str, Any], loss_fn: Callable, loss_weight_fn: Callable) -> Optional[torch.Tensor]:
        self.model.eval()
        mbl = self._prepare_mb_list(input_)
        weights = [float(loss_weight_fn(mb)) for mb in mbl.mbs]
        it = iter(weights)

        def process(hidden, labels, mb, pad, sl):
            w = next(it)
            if self.config.is_critic:
                return loss_fn(self._sp_gather(self.model.values(hidden)), mb) * w
            logp, ent = self._actor_outputs(hidden, labels)
            return loss_fn(self._sp_gather(logp), self._sp_gather(ent), mb) * w

        outs = self._pp_share([o.float().cpu() for o in self.forward_backward_batch(mbl, process, forward_only=True)])
        tot = torch.stack([o.float().cpu() for o in outs]).sum().reshape(1).double()
        w = torch.tensor([sum(weights)], dtype=torch.float64)
        if self.dp_size > 1 and self._cpu_group is not None:
            both = torch.cat([tot, w])
            dist.all_reduce(both, group=self._cpu_group)
            tot, w = both[:1], both[1:]
        return (tot / w.clamp(min=1e-12)).float().squeeze(0)

    @torch.no_grad()
    def forward_batch(self, input_: dict[str, Any], output_seqlens: Optional[list[int]] = None,
                      aggregate_fn: Callable = torch.cat, output: str = "logprobs", temperature: Optional[float] = None):
        """Per-token outputs for a padded batch, returned as a padded ``[B, L]`` tensor in the
        input order. ``output``: logprobs | entropy | values | logprobs_entropy."""
        self.model.eval()
        mbl = self._prepare_mb_list(input_)
        B, L = input_["attention_mask"].shape

        def process(hidden, labels, mb, pad, sl):
            if self.config.is_critic or output == "values":
                v = self.model.values(hidden)
                res = (v,)
            else:
                logp, ent = self._actor_outputs(hidden, labels, temperature)
                res = (logp, ent) if output == "logprobs_entropy" else ((ent,) if output == "entropy" else (logp,))
            row_group, row_n, _ = self._row_split()
            if row_n > 1:
                full = []
                for r in res:
                    parts = [torch.empty_like(r) for _ in range(row_n)]
                    dist.all_gather(parts, r.contiguous(), group=row_group)
                    full.append(self._sp_restore(torch.cat(parts)))
                res = tuple(full)
            host = tuple(D.unpad_logits(r, pad).float().cpu() for r in res)
            self.d2h_bytes += sum(h.numel() * 4 for h in host)
            return host

        outs = self._pp_share(self.forward_backward_batch(mbl, process, forward_only=True))
        n_out = len(outs[0]) if outs else 1
        results = []
        for j in range(n_out):
            padded = torch.zeros(B, L, dtype=torch.float32)
            for g, o, mb in zip(mbl.groups, outs, mbl.mbs):
                cu = mb["cu_seqlens"].tolist()
                for k, i in enumerate(g):
                    n = cu[k + 1] - cu[k]
                    padded[i, :n] = o[j][cu[k]:cu[k + 1]]
            results.append(padded)
        return results[0] if n_out == 1 else tuple(results)

    # ------------------------------------------------------------------ save / load
    def save(self, meta: SaveLoadMeta):
        os.makedirs(meta.path, exist_ok=True)
        head = self.local_index <= 0
        if meta.weight_format == "hf" and getattr(self, "pp_size", 1) > 1:
            # the stages of the first pipeline write their own tensors; the head merges the index
            maps = [None] * self.pp_size
            if self.dp_rank == 0 or (getattr(self, "ep_size", 1) > 1 and self._export_member):
                named = list(self._pp_native_full())
                mine = {}
                if getattr(self, "tp_rank", 0) == 0 and self.dp_rank == 0:          # one writer per stage
                    mine = hf_io.save_hf_sharded(meta.path, self.model_config, hf_io.native_to_hf_tensors(self.model_config, named),
                                                 rank_tag=f"pp{self.pp_rank}", write_index=False)
                dist.all_gather_object(maps, mine, group=self._pp_cpu_group)
            if head:
                merged = {}
                for m_ in maps:
                    merged.update(m_)
                total = sum(os.path.getsize(os.path.join(meta.path, f)) for f in set(merged.values()))
                hf_io.write_hf_index(meta.path, merged, total)
                self.model_config.save_pretrained(meta.path)
                if meta.tokenizer is not None:
                    meta.tokenizer.save_pretrained(meta.path)
        elif meta.weight_format == "hf" and getattr(self, "_z3", None) is not None:
            # every rank takes part in the unit-by-unit gather; the head writes tensor by tensor
            named = self._z3_full_tensors()
            if head:
                hf_io.save_hf_sharded(meta.path, self.model_config, hf_io.native_to_hf_tensors(self.model_config, named))
                if meta.tokenizer is not None:
                    meta.tokenizer.save_pretrained(meta.path)
            else:
                for _ in named:
                    pass
        elif meta.weight_format == "hf" and getattr(self, "ep_size", 1) > 1:
            if self._export_member:                           # the first EP (and TP) groups gather their slices; the head writes
                named = self._ep_full_named_tensors()
                if head:
                    hf_io.save_hf_sharded(meta.path, self.model_config, hf_io.native_to_hf_tensors(self.model_config, named))
                    if meta.tokenizer is not None:
                        meta.tokenizer.save_pretrained(meta.path)
                else:
                    for _ in named:
                        pass
        elif meta.weight_format == "hf":
            if getattr(self, "tp_size", 1) > 1:
                # every tensor-parallel rank of the first data-parallel replica takes part in
                # the gather; the head writes full tensors one by one
                if self.dp_rank == 0 and self.sp_rank == 0:
                    named = self._gathered_full_tensors()
                    if head:
                        hf_io.save_hf_sharded(meta.path, self.model_config, hf_io.native_to_hf_tensors(self.model_config, named))
                    else:
                        for _ in named:
                            pass
            elif head and getattr(self, "use_lora", False):
                from ..models.lora import merge_lora_, save_adapter, unmerge_lora_

                save_adapter(self.model, os.path.join(meta.path, "adapter"), base_model_name_or_path=self.config.path)
                merge_lora_(self.model)       # the served checkpoint carries the adapters folded in
                try:
                    hf_io.save_model_hf(self.model, meta.path, skip=lambda n: "_lora_" in n)
                finally:
                    unmerge_lora_(self.model)
            elif head:
                hf_io.save_model_hf(self.model, meta.path)
            if head and meta.tokenizer is not None:
                meta.tokenizer.save_pretrained(meta.path)
        else:
            from ..ckpt.sharded import save_sharded

            save_sharded(self, meta.path, with_optim=meta.with_optim)
            return
        if meta.with_optim and self.optimizer is not None:
            torch.save(self.optimizer.state_dict(), os.path.join(meta.path, f"optim_rank{max(self.local_index, 0)}.pt"))
            if getattr(self, "expert_optimizer", None) is not None:
                torch.save(self.expert_optimizer.state_dict(), os.path.join(meta.path, f"optim_expert_rank{max(self.local_index, 0)}.pt"))
        if self._cpu_group is not None:
            dist.barrier(group=self._cpu_group)

    def _ep_full_named_tensors(self, to_cpu: bool = False):
        """(name, full tensor): expert stacks gathered over the EP group, tensor-parallel slices over the TP group
        (collectives of those groups: every rank of both must iterate)."""
        from ..parallel import tp as TP

        expert = set(self._expert_param_names)
        tp, xtp = getattr(self, "tp_size", 1), getattr(self, "etp_size", 1) == getattr(self, "tp_size", 1)
        for n_, p_ in self.model.named_parameters():
            t = p_.detach()
            if n_ in expert:
                parts = [torch.empty_like(t) for _ in range(self.ep_size)]
                dist.all_gather(parts, t.contiguous(), group=self._ep_group)
                t = torch.cat(parts, dim=0)
            if tp > 1 and (n_ not in expert or xtp):
                parts = [torch.empty_like(t) for _ in range(tp)]
                dist.all_gather(parts, t.contiguous(), group=self._tp_group)
                t = TP.unshard_tensors(self.model_config, n_, parts, expert_tp=xtp)
            yield n_, (t.to("cpu", copy=True) if to_cpu else t)

    def _z3_full_tensors(self):
        """(name, full tensor) under sharded parameters: gathered unit by unit over the shard group, then over the TP
        group when the model is tensor parallel (a collective of both groups)."""
        from ..parallel import tp as TP

        tp = getattr(self, "tp_size", 1)
        for n_, t in self._z3.full_tensors():
            if tp > 1:
                parts = [torch.empty_like(t) for _ in range(tp)]
                dist.all_gather(parts, t.contiguous(), group=self._tp_group)
                t = TP.unshard_tensors(self.model_config, n_, parts)
            yield n_, t

    def _pp_native_full(self, skip_tied_copy: bool = True):
        """(native name, full tensor) of this stage's parameters; tensor-parallel slices are gathered over the TP group
        first (then a collective of that group: all its ranks must iterate)."""
        from ..parallel import tp as TP

        tp = getattr(self, "tp_size", 1)
        expert = {self.model.native_name(n) for n in self._expert_param_names}
        for n_, p_ in self.model.named_native_parameters(skip_tied_copy=skip_tied_copy):
            t = p_.detach()
            if n_ in expert:                      # expert stacks: gathered over the stage's EP group
                parts = [torch.empty_like(t) for _ in range(self.ep_size)]
                dist.all_gather(parts, t.contiguous(), group=self._ep_group)
                t = torch.cat(parts, dim=0)
            if tp > 1:
                parts = [torch.empty_like(t) for _ in range(tp)]
                dist.all_gather(parts, t.contiguous(), group=self._tp_group)
                t = TP.unshard_tensors(self.model_config, n_, parts)
            yield n_, t

    def _gathered_full_tensors(self):
        """Yields (name, full tensor) for a tensor-parallel model; a collective over the TP group."""
        from ..parallel import tp as TP

        for n_, p_ in self.model.named_parameters():
            parts = [torch.empty_like(p_) for _ in range(self.tp_size)]
            dist.all_gather(parts, p_.detach().contiguous(), group=self._tp_group)
            yield n_, TP.unshard_tensors(self.model_config, n_, parts)

    def load(self, meta: SaveLoadMeta):
        if meta.weight_format == "hf" and getattr(self, "pp_size", 1) > 1:
            mine = {n: p for n, p in self.model.named_native_parameters(skip_tied_copy=False)}
            plan = hf_io.hf_to_native_plan(self.model_config)
            wanted = {hf for n in mine for hf, _, _ in plan[n]}
            tp_ = getattr(self, "tp_size", 1)
            ep_ = getattr(self, "ep_size", 1)
            if ep_ > 1:
                # full expert stacks staged per stage, this rank's experts kept
                expert = {self.model.native_name(n) for n in self._expert_param_names}
                shapes = {n: tuple(p.shape) for n, p in build_model(self.model_config, dtype=self.model.dtype, device="meta").named_parameters()}
                stage = {n: (torch.empty(shapes[n], dtype=p.dtype, device=p.device) if n in expert else p.data) for n, p in mine.items()}
                hf_io.load_hf_tensors_into(self.model_config, stage, ((k, t) for k, t in hf_io.iter_safetensors(meta.path) if k in wanted), strict=False)
                El = self.model_config.num_experts // ep_
                with torch.no_grad():
                    for n in expert:
                        mine[n].copy_(stage[n][self.ep_rank * El:(self.ep_rank + 1) * El])
                del stage
            elif tp_ > 1:
                # full-size staging tensors for this stage's names, sliced into the local parameters afterwards
                from ..parallel import tp as TP

                shapes = {n: tuple(p.shape) for n, p in build_model(self.model_config, dtype=self.model.dtype, device="meta").named_parameters()}
                stage = {n: torch.empty(shapes[n], dtype=p.dtype, device=p.device) for n, p in mine.items()}
                hf_io.load_hf_tensors_into(self.model_config, stage, ((k, t) for k, t in hf_io.iter_safetensors(meta.path) if k in wanted), strict=False)
                with torch.no_grad():
                    for n, p in mine.items():
                        p.copy_(TP.shard_tensor(self.model_config, n, stage[n], tp_, self.tp_rank))
                del stage
            else:
                hf_io.load_hf_tensors_into(self.model_config, {n: p.data for n, p in mine.items()},
                                           ((k, t) for k, t in hf_io.iter_safetensors(meta.path) if k in wanted), strict=False)
        elif meta.weight_format == "hf" and getattr(self, "_z3", None) is not None:
            # tensors stream from the files; every rank keeps what falls into its shard
            tp_ = getattr(self, "tp_size", 1)
            if tp_ == 1:
                hf_io.load_hf_tensors_into(self.model_config, None, hf_io.iter_safetensors(meta.path), strict=not self.config.is_critic,
                                           writer=self._z3.write_piece)
            else:
                # pieces of a full tensor are collected until it is complete, then this rank's TP slice is kept
                from ..parallel import tp as TP

                shapes = {n: (tuple(p.shape), p.dtype) for n, p in build_model(self.model_config, dtype=self.model.dtype, device="meta").named_parameters()}
                plan = hf_io.hf_to_native_plan(self.model_config)
                staged: dict[str, list] = {}

                def collect(native, expert, rows, t):
                    ent = staged.setdefault(native, [torch.empty(shapes[native][0], dtype=shapes[native][1]), 0])
                    dst = ent[0] if expert is None else ent[0][expert]
                    (dst if rows is None else dst[rows[0]:rows[1]]).copy_(t.to(dst.dtype))
                    ent[1] += 1
                    if ent[1] == len(plan[native]):
                        self._z3.write_full(native, TP.shard_tensor(self.model_config, native, ent[0], tp_, self.tp_rank))
                        del staged[native]
                hf_io.load_hf_tensors_into(self.model_config, None, hf_io.iter_safetensors(meta.path), strict=not self.config.is_critic, writer=collect)
        elif meta.weight_format == "hf" and getattr(self, "ep_size", 1) > 1:
            full = build_model(self.model_config, dtype=self.model.dtype, device=self.device, seed=0)
            hf_io.load_model_hf(full, meta.path, strict=not self.config.is_critic)
            from ..parallel import tp as TP

            src = dict(full.named_parameters())
            El = self.model_config.num_experts // self.ep_size
            tp_, xtp = getattr(self, "tp_size", 1), getattr(self, "etp_size", 1) == getattr(self, "tp_size", 1)
            expert = set(self._expert_param_names)
            with torch.no_grad():
                for n_, p_ in self.model.named_parameters():
                    t = TP.shard_tensor(self.model_config, n_, src[n_].detach(), tp_, getattr(self, "tp_rank", 0), expert_tp=xtp)
                    p_.copy_(t[self.ep_rank * El:(self.ep_rank + 1) * El] if n_ in expert else t)
            del full, src
        elif meta.weight_format == "hf":
            if getattr(self, "tp_size", 1) > 1:
                from ..parallel import tp as TP

                full = build_model(self.model_config, dtype=self.model.dtype, device=self.device, seed=0)
                hf_io.load_model_hf(full, meta.path, strict=not self.config.is_critic)
                TP.load_sharded_from_full(self.model, self.model_config, {n_: p_.detach() for n_, p_ in full.named_parameters()},
                                          self.tp_size, self.tp_rank)
                del full
            else:
                hf_io.load_model_hf(self.model, meta.path, strict=not self.config.is_critic)
        else:
            from ..ckpt.sharded import load_sharded

            load_sharded(self, meta.path, with_optim=meta.with_optim)
            return
        if getattr(self, "expert_optimizer", None) is not None:
            self.expert_optimizer.resync_master()
            pe = os.path.join(meta.path, f"optim_expert_rank{max(self.local_index, 0)}.pt")
            if meta.with_optim and os.path.exists(pe):
                self.expert_optimizer.load_state_dict(torch.load(pe, map_location="cpu", weights_only=False))
        if self.optimizer is not None:
            self.optimizer.resync_master()
            p = os.path.join(meta.path, f"optim_rank{max(self.local_index, 0)}.pt")
            if meta.with_optim and os.path.exists(p):
                self.optimizer.load_state_dict(torch.load(p, map_location="cpu", weights_only=False))

    # ------------------------------------------------------------------ rollout coupling
    def connect_engine(self, engine: InferenceEngine, meta: WeightUpdateMeta):
        self.rollout_engine = engine
        self.weight_update_meta = meta
        from ..wsync.service import make_weight_pusher

        self._weight_pusher = make_weight_pusher(self, engine, meta)

    def update_weights(self, meta: Optional[WeightUpdateMeta] = None):
        meta = meta or self.weight_update_meta
        if self._weight_pusher is None:
            raise RuntimeError("connect_engine must be called before update_weights")
        return self._weight_pusher.push(meta)

    def _rollout_source(self):
        """The rollout engine itself, or (with context / tensor parallel peers that must see the
        same tokens) a coordinator that lets the data-parallel head roll out and broadcasts."""
        if self.sp_size * getattr(self, "tp_size", 1) * getattr(self, "pp_size", 1) > 1 and dist.is_initialized():
            from ..rollout.dist_rollout import DistRolloutCoordinator

            return DistRolloutCoordinator(self.rollout_engine, self, redistribute=False)
        return self.rollout_engine

    def rollout_batch(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None):
        return self._rollout_source().rollout_batch(data, workflow=workflow, workflow_kwargs=workflow_kwargs,
                                                    should_accept_fn=should_accept_fn)

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None, dynamic_bs=False):
        return self._rollout_source().prepare_batch(dataloader, workflow=workflow, workflow_kwargs=workflow_kwargs,
                                                    should_accept_fn=should_accept_fn, dynamic_bs=dynamic_bs)

    # ------------------------------------------------------------------ memory
    def offload(self):
        """Moves parameters / optimizer state to pinned host memory (time-sliced colocation)."""
        if self.device.type != "cuda" or getattr(self, "_offloaded", None):
            return
        self._offloaded = {}
        for name in ("master", "exp_avg", "exp_avg_sq"):
            if self.optimizer is not None:
                t = getattr(self.optimizer, name)
                self._offloaded[name] = t.to("cpu", non_blocking=False).pin_memory()
                setattr(self.optimizer, name, torch.empty(0, device=self.device))
        if getattr(self.store, "flat_grad", None) is not None:
            self._offloaded["grad_shape"] = self.store.flat_grad.numel()
        torch.cuda.empty_cache()

    def onload(self):
        off = getattr(self, "_offloaded", None)
        if not off:
            return
        for name in ("master", "exp_avg", "exp_avg_sq"):
            if name in off:
                setattr(self.optimizer, name, off[name].to(self.device, non_blocking=True))
        self._offloaded = None

    @torch.no_grad()
    def export_weights(self) -> dict[str, torch.Tensor]:
        """Host copies of the (replicated) parameters under their native names: the payload of
        the controller-mediated weight update for small models and CPU runs."""
        if getattr(self, "use_lora", False):
            from ..models.lora import merge_lora_, unmerge_lora_

            merge_lora_(self.model)
            try:
                return {n: p.detach().to("cpu", copy=True) for n, p in self.model.named_parameters() if "_lora_" not in n}
            finally:
                unmerge_lora_(self.model)
        if getattr(self, "_z3", None) is not None:
            return {n: t.to("cpu", copy=True) for n, t in self._z3_full_tensors()}
        if getattr(self, "ep_size", 1) > 1 and getattr(self, "pp_size", 1) == 1:
            return dict(self._ep_full_named_tensors(to_cpu=True))
        if getattr(self, "tp_size", 1) > 1 and getattr(self, "pp_size", 1) == 1:
            return {n: t.to("cpu", copy=True) for n, t in self._gathered_full_tensors()}
        if getattr(self, "pp_size", 1) > 1:
            # every stage contributes its own tensors; all stages end up with the full dictionary
            parts = [None] * self.pp_size
            mine = {n: t.to("cpu", copy=True) for n, t in self._pp_native_full()}
            dist.all_gather_object(parts, mine, group=self._pp_cpu_group)
            out = {}
            for d_ in parts:
                out.update(d_)
            return out
        return {n: p.detach().to("cpu", copy=True) for n, p in self.model.named_parameters()}

    def export_stats(self) -> dict[str, float]:
        # reduce over the trainer ranks only (rollout ranks of a split world do not take part)
        g = getattr(self, "_stats_group", self._cpu_group)
        return stats_tracker.export_all(reduce_group=g, distributed=g is not None)


FSDPEngine = B200TrainEngine  # the role FSDPEngine plays in the reference


# --------------------------------------------------------------------------- algorithm mix-ins
class B200PPOActor(B200TrainEngine):
    def __init__(self, config):
        super().__init__(config)
        from ..trainer.ppo.actor import PPOActor

        self.actor = PPOActor(config, self)

    @torch.no_grad()
    def compute_logp(self, *a, **k):
        return self.actor.compute_logp(*a, **k)

    @torch.no_grad()
    def compute_advantages(self, *a, **k):
        return self.actor.compute_advantages(*a, **k)

    def ppo_update(self, *a, **k):
        return self.actor.ppo_update(*a, **k)


class B200PPOCritic(B200TrainEngine):
    def __init__(self, config):
        super().__init__(config)
        from ..trainer.ppo.critic import PPOCritic

        self.critic = PPOCritic(config, self)

    @torch.no_grad()
    def compute_values(self, *a, **k):
        return self.critic.compute_values(*a, **k)

    def ppo_update(self, *a, **k):
        return self.critic.ppo_update(*a, **k)


class B200LMEngine(B200TrainEngine):
    def __init__(self, config):
        super().__init__(config)
        from ..trainer.sft.lm_engine import LMEngine

        self.lm_engine = LMEngine(self)

    def train_lm(self, data):
        return self.lm_engine.train_lm(data)

    def evaluate_lm(self, data):
        return self.lm_engine.evaluate_lm(data)


class B200RWEngine(B200TrainEngine):
    def __init__(self, config):
        config.is_critic = True
        super().__init__(config)
        from ..trainer.rw.rw_engine import RWEngine

        self.rw_engine = RWEngine(self)

    def train_rw(self, data):
        return self.rw_engine.train_rw(data)

    def evaluate_rw(self, data):
        return self.rw_engine.evaluate_rw(data)


class B200DPOEngine(B200TrainEngine):
    def __init__(self, config, beta: float = 0.1, loss_type: str = "sigmoid"):
        super().__init__(config)
        from ..trainer.dpo.dpo_engine import DPOEngine

        self.dpo_engine = DPOEngine(self, beta=beta, loss_type=loss_type)

    def train_dpo(self, data):
        return self.dpo_engine.train_dpo(data)

    def evaluate_dpo(self, data):
        return self.dpo_engine.evaluate_dpo(data)


FSDPPPOActor, FSDPPPOCritic, FSDPLMEngine, FSDPRWEngine, FSDPDPOEngine = (
    B200PPOActor, B200PPOCritic, B200LMEngine, B200RWEngine, B200DPOEngine)
