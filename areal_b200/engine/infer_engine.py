"""The rollout (inference) engine of this framework: continuous batching over a paged KV
cache, prefill with the varlen flash-attention kernel, decode with the paged-attention kernel
under CUDA graphs, fused sampling that returns per-token log-probs, abort / pause / resume
for weight hot-swap, and per-token weight-version tagging.

It implements :class:`~areal_b200.api.engine_api.InferenceEngine` in-process (one engine per
GPU / process) and takes the place of the SGLang / vLLM servers plus HTTP clients of the
reference (``areal/engine/sglang_remote.py``, ``areal/infra/remote_inf_engine.py``).
Interruptible generation follows ``remote_inf_engine.py:912-1083``: the client loop pins the
weight version before every (re)submission, an aborted request returns its partial output,
and the prefix (prompt + tokens so far) is prefetched again under the new weights.

On CPU tensors (tests, tiny models) the engine recomputes the full prefix every step with the
reference ops instead of using the paged cache; semantics are identical.
"""
from __future__ import annotations

import asyncio
import collections
import math
import threading
import time
import zlib
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Any, Optional

import numpy as np
import torch

from ..api.cli_args import InferenceEngineConfig, NativeInferConfig
from ..api.engine_api import InferenceEngine
from ..api.io_struct import ModelRequest, ModelResponse, ParamSpec, WeightUpdateMeta
from ..models.config import ModelConfig
from ..models.decoder import CausalLM, PackedBatch, build_model
from ..ops import functional as OF
from ..ops import lib as oplib
from ..utils import logging as alog

logger = alog.getLogger("infer_engine")

DECODE_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512)


@dataclass
class _Seq:
    rid: str
    tokens: list[int]                      # prompt + generated so far
    prompt_len: int
    max_new: int
    min_new: int
    temperature: float
    greedy: bool
    stop_ids: set
    ignore_eos: bool
    seed: int
    future: Any = None                     # (loop, asyncio future)
    out_tokens: list[int] = field(default_factory=list)
    out_logprobs: list[float] = field(default_factory=list)
    out_versions: list[int] = field(default_factory=list)
    row: int = -1                          # row of the static decode buffers while running
    pages: list[int] = field(default_factory=list)
    cached: int = 0                        # tokens whose KV is in the cache
    t_submit: float = 0.0
    t_first: float = 0.0
    aborted: bool = False
    top_p: float = 1.0
    top_k: int = 0
    stop_strs: tuple = ()                  # stop strings (need the request's tokenizer)
    tokenizer: Any = None
    stop_window: int = 16                  # tokens decoded per check
    mm: Any = None                         # vision-language request: {"pixel_values", "image_grid_thw"}
    rope_delta: int = 0                    # M-RoPE: rotary position of token i (after the prompt) = i + rope_delta
    hstate: Any = None                     # recurrent-state models: models.hybrid.SequenceState once the prompt is absorbed


class PagedKVCache:
    """K and V pages for all layers: ``[layers, 2, num_pages * page_size, Hkv, D]``."""

    def __init__(self, cfg: ModelConfig, num_pages: int, page_size: int, device, dtype, pausable: bool = False):
        self.page_size, self.num_pages = page_size, num_pages
        shape = (cfg.num_layers, 2, num_pages * page_size, cfg.num_kv_heads, cfg.head_dim)
        self.pausable = None
        if pausable:
            from ..ops import vmm

            if vmm.available():
                n = 1
                for d in shape:
                    n *= d
                self.pausable = vmm.PausableBuffer(n * torch.empty(0, dtype=dtype).element_size(), device, keep_contents=False)
                self.data = self.pausable.tensor(dtype, shape)
                self.data.zero_()
        if self.pausable is None:
            self.data = torch.zeros(*shape, device=device, dtype=dtype)
        self.free = list(range(num_pages - 1, -1, -1))
        self.ref = [0] * num_pages          # users of a page: its sequence, plus the prefix cache and other sequences when shared

    def alloc(self, n: int) -> Optional[list[int]]:
        if len(self.free) < n:
            return None
        out = self.free[-n:] if n else []
        if n:
            del self.free[-n:]
        for p in out:
            self.ref[p] = 1
        return out

    def share(self, pages: list[int]) -> None:
        for p in pages:
            self.ref[p] += 1

    def release(self, pages: list[int]) -> None:
        for p in pages:
            self.ref[p] -= 1
            if self.ref[p] <= 0:
                self.ref[p] = 0
                self.free.append(p)

    def pages_needed(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size


class NativeInferenceEngine(InferenceEngine):
    def __init__(self, config: Optional[InferenceEngineConfig] = None, infer_config: Optional[NativeInferConfig] = None,
                 model_config: Optional[ModelConfig] = None, model: Optional[CausalLM] = None, eos_token_id: Optional[int] = None,
                 tp_group=None, tp_control_group=None):
        """``tp_group``: ranks that hold one tensor-parallel replica together (attention heads and
        MLP columns split, embeddings replicated). Every rank of the group runs this engine; the
        group's first rank is the leader and the only one that accepts requests. The ranks move in
        lock-step: once per loop iteration they exchange a small control record (new requests,
        pause / stop flags) over ``tp_control_group`` (a gloo group of the same ranks; defaults to
        ``tp_group``), after which scheduling, paging and sampling are deterministic and identical
        everywhere."""
        self.tp_group, self.tp_control_group = tp_group, (tp_control_group if tp_control_group is not None else tp_group)
        self.tp_size = torch.distributed.get_world_size(tp_group) if tp_group is not None else 1
        self.tp_rank = torch.distributed.get_rank(tp_group) if tp_group is not None else 0
        self._inbox: collections.deque = collections.deque()
        self.config = config or InferenceEngineConfig()
        self.icfg = infer_config or NativeInferConfig()
        self.model_config = model_config or (model.cfg if model is not None else None)
        self.model = model
        self.eos_token_id = eos_token_id
        self._version = 0
        self._lock = threading.Lock()
        self._waiting: collections.deque[_Seq] = collections.deque()
        self._running: list[_Seq] = []
        self._gen_paused = threading.Event()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._executor = None
        self._graphs: dict[int, Any] = {}
        self._step = 0
        self._exc: Optional[BaseException] = None
        self._idle = threading.Event()
        self._idle.set()
        self.stats = collections.Counter()
        self._prefix: collections.OrderedDict = collections.OrderedDict()     # prompt bytes -> shared pages + last-token logits
        self.device = torch.device("cpu")
        self.cache: Optional[PagedKVCache] = None

    # ------------------------------------------------------------------ lifecycle
    def initialize(self, device=None, seed: int = 1, train_data_parallel_size: int = 1, model_path: Optional[str] = None,
                   start_executor: bool = True, **kwargs):
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        if self.model is None:
            if self.model_config is None:
                if not model_path:
                    raise ValueError("inference engine needs a model, a model_config or a model_path")
                self.model_config = ModelConfig.from_pretrained(model_path)
            dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            self.model = build_model(self.model_config, dtype=dtype, device=self.device, seed=seed)
            if model_path:
                from ..models import hf_io

                hf_io.load_model_hf(self.model, model_path)
            if self.tp_size > 1:
                self._shard_model_for_tp(dtype, seed)
        elif self.tp_size > 1 and not hasattr(self, "tp_exchange"):
            self._setup_tp_exchange()          # a ready-made tensor-parallel slice was handed in
        self.shared_model = kwargs.get("shared_model", False)
        if not self.shared_model:
            self.model.eval()
            for p in self.model.parameters():
                p.requires_grad_(False)
        # Layers with a recurrent state (gated delta rule) have no paged-cache decode kernel: such models
        # absorb a prompt with one packed forward that also returns the per-sequence state (rule state,
        # convolution tail, keys / values of the full-attention layers) and then advance one token per
        # step on that state (``_step_recurrent``).
        self._recompute_decode = bool(getattr(self.model_config, "is_hybrid", False))
        if self.device.type == "cuda" and not self._recompute_decode:
            self._init_cuda_state()
        elif self.device.type == "cuda":
            self.stream = torch.cuda.Stream(device=self.device)
        self._t_start = time.perf_counter()
        self._thread = threading.Thread(target=self._engine_main, name="infer-engine", daemon=True)
        self._thread.start()
        if start_executor:
            from ..rollout.executor import WorkflowExecutor

            self._executor = WorkflowExecutor(self.config, self, dp_world_size=train_data_parallel_size).initialize()
        return self

    def _shard_model_for_tp(self, dtype, seed):
        """Replaces the freshly built (or loaded) full model by this rank's tensor-parallel slice."""
        from ..parallel import tp as TP

        if self.model_config.is_vlm:
            raise NotImplementedError("tensor-parallel rollout of vision-language models")
        full, full_cfg = self.model, self.model_config
        self.full_model_config = full_cfg
        self.model_config = TP.local_config(full_cfg, self.tp_size)
        self.model = build_model(self.model_config, dtype=dtype, device=self.device, seed=seed)
        TP.load_sharded_from_full(self.model, full_cfg, {n: p.detach() for n, p in full.named_parameters()}, self.tp_size, self.tp_rank)
        TP.install_tp(self.model, self.tp_group, self.tp_size, self.tp_rank)
        del full
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
        self._setup_tp_exchange()

    def _setup_tp_exchange(self):
        """Dense models on CUDA: the sums over the tensor-parallel ranks run inside this library's
        own kernels over peer memory (``parallel/tp_decode.py``), so decode steps stay graph
        captured. Otherwise (CPU, MoE layers, ``AREAL_TP_FUSED=0``) the sums are library
        all-reduces and decode steps are replayed eagerly."""
        import os

        from ..parallel.tp_decode import TPDecodeExchange, install_tp_decode, supports_fused_tp

        self.tp_exchange = None
        if self.device.type != "cuda" or self.tp_size <= 1:
            return
        if os.environ.get("AREAL_TP_FUSED", "1") == "0" or not supports_fused_tp(self.model) or self.tp_size > 8:
            self.icfg.use_cuda_graph = False
            return
        ic = self.icfg
        max_rows = (max(ic.context_length, ic.max_prefill_tokens, ic.max_running_requests) + 255) // 128 * 128
        self.tp_exchange = TPDecodeExchange(self.tp_group, self.device, self.model_config.hidden_size, max_rows)
        install_tp_decode(self.model, self.tp_exchange)

    def _init_cuda_state(self):
        cfg, ic = self.model_config, self.icfg
        # blocks the caching allocator holds but nobody uses (e.g. the parameters' first home before a
        # trainer moved them into its flat buffer) would otherwise count as taken
        torch.cuda.empty_cache()
        free, total = torch.cuda.mem_get_info()
        per_page = cfg.num_layers * 2 * ic.page_size * cfg.num_kv_heads * cfg.head_dim * 2
        if getattr(ic, "reserve_free_gb", 0.0) > 0:
            budget = free - int(ic.reserve_free_gb * (1 << 30))
        else:
            budget = int(free * ic.mem_fraction_static) - (2 << 30)
        want = ic.max_running_requests * (ic.context_length // ic.page_size + 1)
        n_pages = max(16, min(want, budget // per_page))
        if getattr(ic, "num_pages", None):
            n_pages = ic.num_pages
        self.cache = PagedKVCache(cfg, n_pages, ic.page_size, self.device, torch.bfloat16,
                                  pausable=bool(getattr(ic, "pausable_kv_cache", False)))
        self.max_pages_per_seq = ic.context_length // ic.page_size + 1
        B = max(b for b in DECODE_BUCKETS if b <= max(1, ic.max_running_requests)) if ic.max_running_requests >= 1 else 1
        self.max_batch = B
        dev = self.device
        self.s_tokens = torch.zeros(B, dtype=torch.int32, device=dev)
        self.s_pos = torch.zeros(B, dtype=torch.int32, device=dev)
        self.s_slots = torch.full((B,), -1, dtype=torch.int32, device=dev)
        self.s_lens = torch.zeros(B, dtype=torch.int32, device=dev)
        self.s_pt = torch.zeros(B, self.max_pages_per_seq, dtype=torch.int32, device=dev)
        self.s_inv_temp = torch.ones(B, dtype=torch.float32, device=dev)
        self.s_greedy = torch.zeros(B, dtype=torch.int32, device=dev)
        self.s_seeds = torch.zeros(B, dtype=torch.int32, device=dev)
        self.s_out_tok = torch.zeros(B, dtype=torch.int32, device=dev)
        self.s_out_lp = torch.zeros(B, dtype=torch.float32, device=dev)
        # Host mirrors of the per-row decode state, packed in ONE pinned buffer so a decode
        # step costs one host-to-device copy: columns tokens|pos|slots|lens|greedy|seeds|
        # inv_temp(bits)|page table. Rows are stable while a sequence runs.
        self._ncol = 7 + self.max_pages_per_seq
        self.h_state = torch.zeros(B, self._ncol, dtype=torch.int32).pin_memory()
        self.d_state = torch.zeros(B, self._ncol, dtype=torch.int32, device=dev)
        hs = self.h_state.numpy()
        self.hn_tokens, self.hn_pos, self.hn_slots, self.hn_lens = hs[:, 0], hs[:, 1], hs[:, 2], hs[:, 3]
        self.hn_greedy, self.hn_seeds = hs[:, 4], hs[:, 5]
        self.hn_inv_temp = hs[:, 6].view(np.float32)
        self.hn_pt = hs[:, 7:]
        self.hn_slots[:] = -1
        self.hn_inv_temp[:] = 1.0
        self.h_out = torch.zeros(2, B, dtype=torch.int32).pin_memory()
        self.hn_out_tok = self.h_out.numpy()[0]
        self.hn_out_lp = self.h_out.numpy()[1].view(np.float32)
        self._row_seq: list = [None] * B
        self._rows_free = list(range(B - 1, -1, -1))   # pop() gives the lowest free row
        self.n_splits = 4
        self.s_part_o = torch.zeros(B * cfg.num_heads * self.n_splits * cfg.head_dim, dtype=torch.float32, device=dev)
        self.s_part_ml = torch.zeros(B * cfg.num_heads * self.n_splits * 2, dtype=torch.float32, device=dev)
        # higher priority than the default stream: when a trainer shares the GPU, the short decode
        # kernels get the SMs that free up first instead of queueing behind its long ones
        self.stream = torch.cuda.Stream(device=dev, priority=-1)
        self._err_poll = oplib.ErrorPoller()
        oplib.get_lib().ab2_runtime_init()
        logger.info("KV cache: %d pages x %d tokens (%.1f GB)", n_pages, ic.page_size, n_pages * per_page / 2 ** 30)

    def destroy(self):
        self._stop.set()
        if self._executor is not None:
            self._executor.destroy()
            self._executor = None
        if self._thread is not None:
            self._thread.join(timeout=10)
            self._thread = None
        self._graphs.clear()
        self.cache = None

    # ------------------------------------------------------------------ versions / weights
    def set_version(self, version: int) -> None:
        self._version = version

    def get_version(self) -> int:
        return self._version

    def pause_generation(self):
        """Aborts in-flight requests (they return their partial output) and holds the engine
        loop until ``continue_generation``."""
        self._gen_paused.set()
        self._idle.wait(timeout=60)

    def continue_generation(self):
        self._gen_paused.clear()

    def pause(self):
        if self._executor is not None:
            self._executor.pause()

    def resume(self):
        if self._executor is not None:
            self._executor.resume()

    def is_paused(self) -> bool:
        return self._executor.is_paused() if self._executor is not None else False

    @torch.no_grad()
    def update_weights_from_tensors(self, named_tensors, meta: Optional[WeightUpdateMeta] = None) -> Future:
        """Copies native-named tensors into the model (device-to-device or host-to-device)."""
        fut: Future = Future()
        params = dict(self.model.named_parameters())
        if isinstance(named_tensors, dict):
            named_tensors = named_tensors.items()
        for name, t in named_tensors:
            if self.tp_size > 1 and tuple(t.shape) != tuple(params[name].shape):
                from ..parallel import tp as TP

                t = TP.shard_tensor(self.full_model_config, name, t, self.tp_size, self.tp_rank)   # full tensor -> this rank's slice
            params[name].data.copy_(t.to(params[name].dtype), non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        if meta is not None and meta.version is not None:
            self.set_version(meta.version)
        fut.set_result(True)
        return fut

    @torch.no_grad()
    def export_weights(self) -> dict[str, torch.Tensor]:
        """Host copies of the parameters currently served (diagnostics, weight-sync checks)."""
        return {n: p.detach().to("cpu", copy=True) for n, p in self.model.named_parameters()}

    def update_weights_from_disk(self, meta: WeightUpdateMeta) -> Future:
        from ..models import hf_io

        fut: Future = Future()
        if self.tp_size > 1:
            from ..parallel import tp as TP

            full = build_model(self.full_model_config, dtype=self.model.dtype, device="cpu", seed=0)
            hf_io.load_model_hf(full, meta.path)
            TP.load_sharded_from_full(self.model, self.full_model_config, {n: p.detach() for n, p in full.named_parameters()},
                                      self.tp_size, self.tp_rank)
            del full
        else:
            hf_io.load_model_hf(self.model, meta.path)
        if meta.version is not None:
            self.set_version(meta.version)
        fut.set_result(True)
        return fut

    def init_weights_update_group(self, meta: WeightUpdateMeta) -> Future:
        fut: Future = Future()
        fut.set_result(True)
        return fut

    def update_weights_from_distributed(self, meta: WeightUpdateMeta, param_specs: list[ParamSpec]) -> Future:
        from ..wsync.service import receive_broadcast

        fut: Future = Future()
        receive_broadcast(self, meta, param_specs)
        fut.set_result(True)
        return fut

    def offload(self, tags=None):
        """Gives the KV pool's memory back to the device. With a pausable pool the addresses (and the
        CUDA graphs that point into them) survive; otherwise the pool and the graphs are dropped."""
        self.pause_generation()
        if self.cache is not None and self.cache.pausable is not None:
            self._abort_all_now()
            self._prefix.clear()
            self.cache.free = list(range(self.cache.num_pages - 1, -1, -1))
            self.cache.ref = [0] * self.cache.num_pages
            torch.cuda.synchronize(self.device)
            self.cache.pausable.pause()
            return
        self._graphs.clear()
        if self.cache is not None:
            self._saved_cache_shape = (self.cache.num_pages, self.cache.page_size)
            self.cache = None
            torch.cuda.empty_cache()

    def _abort_all_now(self):
        """Requests in flight lose their KV pages: they return what they have and their clients resubmit."""
        self._abort_all()

    def onload(self, tags=None):
        if self.cache is not None and self.cache.pausable is not None:
            if self.cache.pausable.paused:
                self.cache.pausable.resume()
                self.cache.data.zero_()
            self.continue_generation()
            return
        if self.cache is None and self.device.type == "cuda" and not self._recompute_decode:
            n, ps = self._saved_cache_shape
            self.cache = PagedKVCache(self.model_config, n, ps, self.device, torch.bfloat16)
        self.continue_generation()

    # ------------------------------------------------------------------ request API
    def _prepare_multi_modal(self, req: ModelRequest, prompt: list[int]):
        """Images of a vision-language request -> patches for the tower plus the M-RoPE offset of
        the tokens generated after the prompt. ``image_data`` entries may be PIL images, uint8
        arrays, raw bytes or base64 strings (optionally ``data:`` URLs); the prompt must already
        hold one placeholder token per merged patch (what the HF processor produces)."""
        images = getattr(req, "image_data", None)
        if not images or not getattr(self.model.cfg, "is_vlm", False):
            return None, 0
        from ..models.vision import mrope_position_ids, preprocess_images
        from ..utils.image import load_image

        pre = getattr(req, "metadata", None) or {}
        if isinstance(pre, dict) and pre.get("pixel_values") is not None:
            px, grid = torch.as_tensor(pre["pixel_values"]), torch.as_tensor(pre["image_grid_thw"]).view(-1, 3).long()
        else:
            px, grid = preprocess_images([load_image(im) for im in images], self.model.vcfg)
        cfg = self.model.cfg
        _, delta = mrope_position_ids(torch.tensor(prompt), grid, cfg.image_token_id, self.model.vcfg.spatial_merge_size, cfg.video_token_id)
        return {"pixel_values": px, "image_grid_thw": grid}, int(delta)

    async def agenerate(self, req: ModelRequest) -> ModelResponse:
        """Interruptible generation: loops over engine submissions until the request stops for
        a real reason; every segment is tagged with the weight version it ran under."""
        g = req.gconfig
        if self.tp_size > 1:
            if self.tp_rank != 0:
                raise RuntimeError("requests go to the leader (first rank) of a tensor-parallel replica")
            if g.stop:
                raise NotImplementedError("stop strings with a tensor-parallel replica (use stop_token_ids)")
        prompt = list(req.input_ids)
        budget = min(g.max_tokens - len(prompt), g.max_new_tokens)
        if budget <= 0:
            raise ValueError(f"prompt of {len(prompt)} tokens leaves no room under max_tokens={g.max_tokens}")
        out_tok: list[int] = []
        out_lp: list[float] = []
        out_ver: list[int] = []
        stop_reason = "abort"
        t0 = time.perf_counter()
        ttft = float("inf")
        tokens = prompt
        remaining = budget
        loop = asyncio.get_running_loop()
        mm, rope_delta = self._prepare_multi_modal(req, prompt)
        while stop_reason not in ("stop", "tool_calls", "length") and len(out_tok) < budget:
            while self._gen_paused.is_set():
                await asyncio.sleep(0.002)
            if self._exc is not None:
                raise RuntimeError("inference engine is dead") from self._exc
            version = self.get_version()
            fut = loop.create_future()
            seq = _Seq(rid=req.rid, tokens=list(tokens), prompt_len=len(tokens), max_new=remaining,
                       min_new=max(0, g.min_new_tokens - len(out_tok)), temperature=0.0 if g.greedy else g.temperature,
                       greedy=bool(g.greedy) or g.temperature == 0.0,
                       stop_ids=set(g.stop_token_ids or []), ignore_eos=g.ignore_eos,
                       # a request without its own seed: its id hashed with the engine's seed (``native_infer.random_seed``)
                       seed=(g.seed if g.seed is not None else zlib.crc32(req.rid.encode()) ^ (int(self.icfg.random_seed) * 0x9E3779B1)) & 0x7FFFFFFF,
                       future=(loop, fut),
                       t_submit=time.perf_counter(), top_p=g.top_p, top_k=0 if g.top_k >= 10 ** 7 else int(g.top_k),
                       mm=mm, rope_delta=rope_delta, stop_strs=tuple(g.stop or ()), tokenizer=getattr(req, "tokenizer", None),
                       stop_window=max(8, 2 * max((len(x) for x in (g.stop or [""])), default=0)))
            with self._lock:
                (self._inbox if self.tp_size > 1 else self._waiting).append(seq)
            seg_tokens, seg_lps, seg_vers, stop_reason, t_first = await fut
            if seg_tokens and ttft == float("inf"):
                ttft = t_first - t0
            out_tok += seg_tokens
            out_lp += seg_lps
            out_ver += seg_vers
            tokens = tokens + seg_tokens
            remaining -= len(seg_tokens)
        if stop_reason == "abort":
            stop_reason = "length"
        assert len(out_tok) == len(out_lp) == len(out_ver), "token / logprob / version streams diverged"
        lat = time.perf_counter() - t0
        return ModelResponse(input_tokens=prompt, output_tokens=out_tok, output_logprobs=out_lp, output_versions=out_ver,
                             stop_reason=stop_reason, latency=lat, ttft=ttft, tokenizer=req.tokenizer,
                             itl=[(lat - ttft) / max(1, len(out_tok) - 1)] if out_tok else [])

    def submit(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None, task_id=None, is_eval=False) -> int:
        return self._executor.submit(data, workflow, workflow_kwargs, should_accept_fn, task_id, is_eval)

    def wait(self, count, timeout=None, raise_timeout=True):
        return self._executor.wait(count, timeout, raise_timeout)

    def wait_for_task(self, task_id, timeout=None, raise_timeout=True):
        return self._executor.wait_for_task(task_id, timeout, raise_timeout)

    def rollout_batch(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None):
        return self._executor.rollout_batch(data, workflow, workflow_kwargs, should_accept_fn)

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None, dynamic_bs=False):
        return self._executor.prepare_batch(dataloader, workflow, workflow_kwargs, should_accept_fn, dynamic_bs)

    @property
    def workflow_executor(self):
        return self._executor

    # ------------------------------------------------------------------ engine loop
    def _engine_main(self):
        try:
            if self.device.type == "cuda":
                torch.cuda.set_device(self.device)
            while self.tp_size > 1 or not self._stop.is_set():      # a TP replica leaves the loop together (stop is exchanged)
                paused = self._gen_paused.is_set()
                if self.tp_size > 1:
                    paused, stop = self._tp_sync_control(paused)
                    if stop:
                        break
                if paused:
                    if not getattr(self.icfg, "retain_kv_on_weight_update", False):
                        self._abort_all()
                    self._idle.set()
                    time.sleep(0.001)
                    continue
                with self._lock:
                    has_work = bool(self._waiting) or bool(self._running)
                if not has_work:
                    self._idle.set()
                    time.sleep(0.0005)
                    continue
                self._idle.clear()
                t_busy = time.perf_counter()
                if self.device.type == "cuda" and self._recompute_decode:
                    with torch.cuda.stream(self.stream), torch.no_grad():
                        self._step_recurrent()
                elif self.device.type == "cuda":
                    with torch.cuda.stream(self.stream), torch.no_grad():
                        self._step_cuda()
                else:
                    with torch.no_grad():
                        self._step_recurrent() if self._recompute_decode else self._step_cpu()
                self.stats["busy_seconds"] += time.perf_counter() - t_busy
        except BaseException as e:  # surface to waiting clients
            import traceback

            logger.error("inference engine loop failed: %r\n%s", e, traceback.format_exc())
            self._exc = e
            self._fail_all(e)
            self._idle.set()
            # keep rejecting requests that were queued after the failure so no client hangs
            while not self._stop.is_set():
                self._fail_all(e)
                time.sleep(0.01)
        finally:
            self._idle.set()

    _SEQ_WIRE_FIELDS = ("rid", "tokens", "prompt_len", "max_new", "min_new", "temperature", "greedy", "stop_ids", "ignore_eos", "seed",
                        "top_p", "top_k", "rope_delta")

    def _tp_sync_control(self, paused: bool):
        """One exchange per loop iteration of a tensor-parallel replica: every rank reports its
        pause / stop flags, the leader adds the requests that arrived since the last exchange.
        Afterwards all ranks hold the same waiting queue and take the same branch."""
        import torch.distributed as dist

        mine = {"paused": paused, "stop": self._stop.is_set(), "new": None}
        fresh: list[_Seq] = []
        if self.tp_rank == 0:
            with self._lock:
                while self._inbox:
                    fresh.append(self._inbox.popleft())
            mine["new"] = [{k: getattr(q, k) for k in self._SEQ_WIRE_FIELDS} for q in fresh]
        box = [None] * self.tp_size
        dist.all_gather_object(box, mine, group=self.tp_control_group)
        arrivals = fresh if self.tp_rank == 0 else [_Seq(future=None, t_submit=time.perf_counter(), **d) for d in (box[0]["new"] or [])]
        if arrivals:
            with self._lock:
                self._waiting.extend(arrivals)
        return any(b["paused"] for b in box), any(b["stop"] for b in box)

    def _resolve(self, seq: _Seq, reason: str):
        res = (seq.out_tokens, seq.out_logprobs, seq.out_versions, reason, seq.t_first)
        if self.cache is not None and seq.pages:
            self.cache.release(seq.pages)
            seq.pages = []
        if seq.row >= 0:
            self._free_row(seq)
        if seq.future is None:          # follower of a tensor-parallel replica: the leader answers the client
            return
        loop, fut = seq.future

        def _set():
            if not fut.done():
                fut.set_result(res)
        loop.call_soon_threadsafe(_set)

    def _fail_all(self, e):
        with self._lock:
            seqs = list(self._waiting) + self._running
            self._waiting.clear()
            self._running = []
        for s in seqs:
            if s.future is None:
                continue
            loop, fut = s.future
            loop.call_soon_threadsafe(lambda f=fut: (not f.done()) and f.set_exception(RuntimeError(f"engine failed: {e!r}")))

    def _abort_all(self):
        with self._lock:
            seqs = list(self._waiting) + self._running
            self._waiting.clear()
            self._running = []
        for s in seqs:
            self.stats["aborted"] += 1
            self._resolve(s, "abort")

    def _finish_check(self, s: _Seq, tok: int) -> Optional[str]:
        n = len(s.out_tokens)
        if n >= s.min_new:
            if tok in s.stop_ids:
                return "stop"
            if not s.ignore_eos and self.eos_token_id is not None and tok == self.eos_token_id:
                return "stop"
            if s.stop_strs and s.tokenizer is not None:
                # stop strings are matched on the decoded tail (a string may span several tokens)
                tail = s.tokenizer.decode(s.out_tokens[-s.stop_window:])
                if any(st in tail for st in s.stop_strs):
                    return "stop"
        if n >= s.max_new:
            return "length"
        if len(s.tokens) >= self.icfg.context_length:
            return "length"
        return None

    # ---------------------------------------------------------------- CPU reference path
    def _step_cpu(self):
        with self._lock:
            while self._waiting and len(self._running) < self.icfg.max_running_requests:
                self._running.append(self._waiting.popleft())
            batch = list(self._running)
        if not batch:
            return
        lens = [len(s.tokens) for s in batch]
        ids = torch.tensor([t for s in batch for t in s.tokens], dtype=torch.long).to(self.device)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32).to(self.device)
        if any(s.mm is not None for s in batch):
            from ..models.vlm import collect_multi_modal

            hidden = self.model(ids, cu, max_seqlen=max(lens), mm=collect_multi_modal([s.mm for s in batch]))
        else:
            hidden = self.model(ids, cu, max_seqlen=max(lens))
        last = hidden[(cu[1:] - 1).long()]
        logits = self.model.logits(last).float().cpu()
        self._step += 1
        done = []
        for i, s in enumerate(batch):
            tok, lp = self._sample_cpu(logits[i], s)
            self._accept_token(s, tok, lp, done)
        self._retire(done)

    def _step_recurrent(self):
        """Models with carried state: new sequences are absorbed by one packed forward, running ones
        advance by one token on their state; both groups sample from the last position."""
        from ..models.hybrid import decode_states, prefill_states

        with self._lock:
            while self._waiting and len(self._running) < self.icfg.max_running_requests:
                self._running.append(self._waiting.popleft())
            batch = list(self._running)
        if not batch:
            return
        fresh = [s for s in batch if s.hstate is None]
        going = [s for s in batch if s.hstate is not None]
        rows, order = [], []
        if fresh:
            lens = [len(s.tokens) for s in fresh]
            ids = torch.tensor([t for s in fresh for t in s.tokens], dtype=torch.long).to(self.device)
            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32).to(self.device)
            hidden, states = prefill_states(self.model, ids, cu, max(lens))
            for s, st in zip(fresh, states):
                s.hstate = st
            rows.append(hidden[(cu[1:] - 1).long()])
            order += fresh
        if going:
            toks = torch.tensor([s.tokens[-1] for s in going], dtype=torch.long).to(self.device)
            rows.append(decode_states(self.model, toks, [s.hstate for s in going]))
            order += going
        logits = self.model.logits(torch.cat(rows, 0)).float().cpu()
        self._step += 1
        done = []
        for i, s in enumerate(order):
            tok, lp = self._sample_cpu(logits[i], s)
            self._accept_token(s, tok, lp, done)
        for s, _ in done:
            s.hstate = None
        self._retire(done)

    def _sample_cpu(self, logits: torch.Tensor, s: _Seq):
        if s.greedy:
            lp_all = torch.log_softmax(logits.float(), -1)
            tok = int(torch.argmax(lp_all))
            return tok, float(lp_all[tok])
        z = logits.float() / max(s.temperature, 1e-6)
        z = _apply_top_k_top_p(z, s.top_k, s.top_p)
        lp_all = torch.log_softmax(z, -1)
        gen = torch.Generator().manual_seed((s.seed * 1000003 + len(s.tokens)) & 0x7FFFFFFF)
        tok = int(torch.multinomial(lp_all.exp(), 1, generator=gen))
        return tok, float(lp_all[tok])

    def _accept_token(self, s: _Seq, tok: int, lp: float, done: list):
        if not s.out_tokens:
            s.t_first = time.perf_counter()
        s.out_tokens.append(tok)
        s.out_logprobs.append(lp)
        s.out_versions.append(self._version)
        s.tokens.append(tok)
        self.stats["generated_tokens"] += 1
        reason = self._finish_check(s, tok)
        if reason is not None:
            done.append((s, reason))

    def _retire(self, done):
        if not done:
            return
        gone = {id(s) for s, _ in done}
        with self._lock:
            self._running = [s for s in self._running if id(s) not in gone]
        for s, reason in done:
            self._resolve(s, reason)

    # ---------------------------------------------------------------- CUDA path
    def _step_cuda(self):
        cache = self.cache
        # ---- admission + prefill
        admitted: list[_Seq] = []
        reuse: list[tuple[_Seq, bytes]] = []       # sequences whose prompt is (or is about to be) in the prefix cache
        pending: dict = {}                         # prompts that a sequence of THIS batch prefetches
        sharing = bool(getattr(self.icfg, "enable_prefix_sharing", False))
        budget = self.icfg.max_prefill_tokens
        ps = cache.page_size
        full = bool(getattr(self.icfg, "reserve_full_length", False))
        with self._lock:
            while self._waiting and len(self._running) + len(admitted) + len(reuse) < self.max_batch:
                s = self._waiting[0]
                if full:
                    need = cache.pages_needed(min(len(s.tokens) + s.max_new, self.icfg.context_length))
                    headroom = 0
                else:
                    # pages for the prompt and the first generated token now, the rest as the sequence grows;
                    # a page per running sequence stays free so that growth rarely has to pre-empt
                    need = cache.pages_needed(min(len(s.tokens) + 1, self.icfg.context_length))
                    headroom = len(self._running) + len(admitted) + len(reuse) + 1
                key = self._prefix_key(s) if sharing else None
                hit = key is not None and (key in pending or self._prefix_lookup(key) is not None)
                if hit:
                    private = need - len(s.tokens) // ps
                    if not self._have_pages(private + headroom):
                        break
                    pages = self._alloc_pages(private)      # only the private part
                    if pages is None:
                        break
                    self._waiting.popleft()
                    s.pages = pages
                    reuse.append((s, key))
                    continue
                if len(s.tokens) > budget and admitted:
                    break
                if not self._have_pages(need + headroom):
                    break
                pages = self._alloc_pages(need)
                if pages is None:
                    break
                self._waiting.popleft()
                s.pages = pages
                admitted.append(s)
                budget -= len(s.tokens)
                if key is not None:
                    pending[key] = s
        done: list = []
        if admitted:
            self._prefill(admitted, done, remember=pending if sharing else None)
        started: list[_Seq] = []
        if reuse:
            # only the sequences that really started: one whose prefix entry was evicted meanwhile
            # went back to the waiting queue and must not also get a decode row
            started = self._start_from_prefix(reuse, done)
        if admitted or started:
            keep = [s for s in admitted + started if all(s is not d for d, _ in done)]
            for s in keep:
                self._assign_row(s)
            with self._lock:
                self._running.extend(keep)
        with self._lock:
            batch = list(self._running)
        if batch:
            # freshly prefilled sequences already hold their first token: they decode at once
            self._decode(batch, done)
        self._retire(done)

    def _layer_attn_fns(self, mode: str, **kw):
        cfg = self.model_config
        fns = []
        scale = 1.0 / math.sqrt(cfg.head_dim)
        L = oplib.get_lib()
        for li in range(cfg.num_layers):
            kc, vc = self.cache.data[li, 0], self.cache.data[li, 1]

            def fn(q, k, v, kc=kc, vc=vc):
                n = q.shape[0]
                rc = L.ab2_kv_append(k.data_ptr(), v.data_ptr(), kc.data_ptr(), vc.data_ptr(), kw["slots"].data_ptr(), n,
                                     cfg.num_kv_heads, cfg.head_dim, k.stride(0), v.stride(0), oplib.stream_ptr())
                oplib.check(rc, "ab2_kv_append")
                if mode == "prefill":
                    o, _ = OF.attention_fwd(q, k, v, kw["cu"], True, scale, kw["tile_info"])
                    return o
                # q may be the query part of the fused [q | k] buffer: rows q.stride(0) apart, heads dense
                assert q.stride(2) == 1 and q.stride(1) == cfg.head_dim
                o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
                rc = L.ab2_paged_decode_strided(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), kw["pt"].data_ptr(),
                                                kw["lens"].data_ptr(), self.s_part_o.data_ptr(), self.s_part_ml.data_ptr(),
                                                o.data_ptr(), n, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim,
                                                self.cache.page_size, self.max_pages_per_seq, self.n_splits, scale,
                                                q.stride(0), oplib.stream_ptr())
                oplib.check(rc, "ab2_paged_decode_strided")
                return o
            fns.append(fn)
        return fns

    def _slot_of(self, s: _Seq, pos: int) -> int:
        ps = self.cache.page_size
        return s.pages[pos // ps] * ps + pos % ps

    # ---- prefix sharing (identical prompts: GRPO groups, retries)
    @staticmethod
    def _prefix_key(s: _Seq) -> Optional[bytes]:
        return None if s.mm is not None else np.asarray(s.tokens, dtype=np.int32).tobytes()

    def _prefix_lookup(self, key: bytes):
        ent = self._prefix.get(key)
        if ent is None:
            return None
        if ent["version"] != self._version:            # computed under older weights
            self._prefix_drop(key)
            return None
        self._prefix.move_to_end(key)
        return ent

    def _prefix_drop(self, key: bytes) -> None:
        ent = self._prefix.pop(key, None)
        if ent is not None:
            self.cache.release(ent["pages"] + ([ent["tail_page"]] if ent["tail_page"] is not None else []))

    def _alloc_pages(self, n: int):
        """Page allocation that evicts least recently used prefix entries when the pool runs dry."""
        pages = self.cache.alloc(n)
        while pages is None and self._prefix:
            self._prefix_drop(next(iter(self._prefix)))
            pages = self.cache.alloc(n)
        return pages

    def _have_pages(self, n: int) -> bool:
        """True when ``n`` pages are free, or can be made free by dropping stored prompts."""
        if len(self.cache.free) >= n:
            return True
        spare = 0
        for ent in self._prefix.values():
            spare += sum(1 for p in ent["pages"] if self.cache.ref[p] == 1) + (ent["tail_page"] is not None)
            if len(self.cache.free) + spare >= n:
                return True
        return False

    def _grow_pages(self, seqs: list, done: list) -> list:
        """Before a decode step every sequence needs a page for the token it is about to cache. Takes
        them one at a time; when the pool is dry (stored prompts already dropped) the most recently
        admitted sequence other than the one in need is pre-empted: it leaves with what it has
        generated ("abort"), its client resubmits it and its prefix is prefetched again later."""
        ps = self.cache.page_size
        short = [s for s in seqs if len(s.pages) * ps < len(s.tokens)]
        if not short:
            return seqs
        gone = set()
        for s in short:
            if id(s) in gone:
                continue
            while len(s.pages) * ps < len(s.tokens):
                got = self._alloc_pages(1)
                if got is None:
                    victims = [v for v in seqs if id(v) not in gone and v is not s]
                    if not victims:
                        raise RuntimeError("KV page pool too small for a single sequence")
                    v = max(victims, key=lambda q: (q.t_submit, q.rid))
                    gone.add(id(v))
                    self.stats["preempted"] += 1
                    with self._lock:
                        self._running = [q for q in self._running if q is not v]
                    self._resolve(v, "abort")
                    continue
                s.pages.append(got[0])
                self.hn_pt[s.row, len(s.pages) - 1] = got[0]
        return [q for q in seqs if id(q) not in gone] if gone else seqs

    def _prefix_remember(self, key: bytes, s: _Seq, logits_row: torch.Tensor) -> None:
        ps = self.cache.page_size
        n = s.cached
        n_full, tail = n // ps, n % ps
        self._prefix_drop(key)                  # a stale entry of the same prompt gives its pages back first
        tail_page = None
        if tail:
            got = self.cache.alloc(1)
            if got is None:
                return
            tail_page = got[0]
            src = s.pages[n_full]
            self.cache.data[:, :, tail_page * ps: tail_page * ps + tail] = self.cache.data[:, :, src * ps: src * ps + tail]
        full = list(s.pages[:n_full])
        self.cache.share(full)
        self._prefix[key] = dict(pages=full, tail_page=tail_page, tail=tail, n=n, logits=logits_row.clone(), version=self._version)

    def _start_from_prefix(self, reuse: list, done: list) -> list:
        """Sequences whose whole prompt is cached: link the shared pages, copy the partial last page,
        sample the first token from the stored logits. No forward pass. Returns the sequences that
        started; the others (entry evicted since admission) are back at the head of the waiting queue."""
        ps = self.cache.page_size
        ready, rows = [], []
        for s, key in reuse:
            ent = self._prefix_lookup(key)
            if ent is None:                            # the sequence that was to prefetch it did not get to (eviction, failure)
                self.cache.release(s.pages)
                s.pages = []
                with self._lock:
                    self._waiting.appendleft(s)
                continue
            private = s.pages
            self.cache.share(ent["pages"])
            s.pages = list(ent["pages"]) + private
            if ent["tail"]:
                dst, src = private[0], ent["tail_page"]
                self.cache.data[:, :, dst * ps: dst * ps + ent["tail"]] = self.cache.data[:, :, src * ps: src * ps + ent["tail"]]
            s.cached = ent["n"]
            ready.append(s)
            rows.append(ent["logits"])
        if not ready:
            return ready
        toks, lps = self._sample_cuda(torch.stack(rows), ready)
        self.stats["prefix_hits"] += len(ready)
        self.stats["prefix_tokens_saved"] += sum(s.cached for s in ready)
        for s, tok, lp in zip(ready, toks, lps):
            self._accept_token(s, tok, lp, done)
        return ready

    def _prefill(self, seqs: list[_Seq], done: list, remember: Optional[dict] = None):
        dev = self.device
        lens = [len(s.tokens) for s in seqs]
        T = sum(lens)
        Tp = (T + 127) // 128 * 128
        ids = torch.zeros(Tp, dtype=torch.int32)
        pos = torch.zeros(Tp, dtype=torch.int32)
        slots = torch.full((Tp,), -1, dtype=torch.int32)
        off = 0
        for s, n in zip(seqs, lens):
            ids[off:off + n] = torch.tensor(s.tokens, dtype=torch.int32)
            pos[off:off + n] = torch.arange(n, dtype=torch.int32)
            ps = self.cache.page_size
            pg = torch.tensor(s.pages, dtype=torch.int32)
            ar = torch.arange(n, dtype=torch.int32)
            slots[off:off + n] = pg[(ar // ps).long()] * ps + ar % ps
            off += n
        cu_list = [0] + list(torch.tensor(lens).cumsum(0).tolist())
        if Tp > T:
            cu_list.append(Tp)
        cu = torch.tensor(cu_list, dtype=torch.int32)
        ids, pos, slots, cu = (t.pin_memory().to(dev, non_blocking=True) for t in (ids, pos, slots, cu))
        pb = PackedBatch(cu, pos, Tp, max(lens))
        fns = self._layer_attn_fns("prefill", slots=slots, cu=cu, tile_info=pb.tile_info)
        if any(s.mm is not None for s in seqs):
            from ..models.vlm import collect_multi_modal

            mm = collect_multi_modal([s.mm for s in seqs])
            mm = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in mm.items()}
            hidden = self.model.forward_hidden(ids, pb, attn_fns=fns, mm=mm)
        else:
            hidden = self.model.forward_hidden(ids, pb, attn_fns=fns)
        last_idx = torch.tensor([c - 1 for c in cu_list[1:len(seqs) + 1]], dtype=torch.long, device=dev)
        logits = self.model.logits(hidden[last_idx].contiguous())
        toks, lps = self._sample_cuda(logits, seqs)
        self.stats["prefill_tokens"] += T
        keys = {id(s): k for k, s in (remember or {}).items()}
        for i, (s, n, tok, lp) in enumerate(zip(seqs, lens, toks, lps)):
            s.cached = n
            if id(s) in keys:
                self._prefix_remember(keys[id(s)], s, logits[i])      # before the first token is appended to s.tokens
            self._accept_token(s, tok, lp, done)

    def _sample_rows(self, logits: torch.Tensor, n: int, inv_temp, greedy, seeds):
        """Launches the sampling kernel for ``n`` rows of ``logits`` with per-row parameters
        that already live on the device; results land in ``s_out_tok`` / ``s_out_lp``."""
        self._step += 1
        rc = oplib.get_lib().ab2_sample(logits.data_ptr(), logits.stride(0), n, logits.shape[1], inv_temp.data_ptr(),
                                        greedy.data_ptr(), seeds.data_ptr(), self._step & 0x7FFFFFFF,
                                        self.s_out_tok.data_ptr(), self.s_out_lp.data_ptr(), oplib.stream_ptr())
        oplib.check(rc, "ab2_sample")

    def _fetch_samples(self, n: int):
        """One device-to-host copy of the sampled tokens and logprobs (pinned), one sync."""
        self.h_out[0, :n].copy_(self.s_out_tok[:n], non_blocking=True)
        self.h_out[1, :n].copy_(self.s_out_lp[:n].view(torch.int32), non_blocking=True)
        self._err_poll.enqueue()            # the error word rides along with the step's only synchronisation
        torch.cuda.current_stream().synchronize()
        self._err_poll.check("rollout engine step")
        return self.hn_out_tok[:n].tolist(), self.hn_out_lp[:n].tolist()

    def _sample_cuda(self, logits: torch.Tensor, seqs: list[_Seq]):
        """Sampling for an ad-hoc list of sequences (prefill path)."""
        n = len(seqs)
        plain = all(s.top_p >= 1.0 and s.top_k <= 0 for s in seqs)
        if not plain:
            self._step += 1
            out_t, out_l = [], []
            lg = logits.float().cpu()
            for i, s in enumerate(seqs):
                t, l = self._sample_cpu(lg[i], s)
                out_t.append(t)
                out_l.append(l)
            return out_t, out_l
        inv_t = torch.tensor([1.0 if s.greedy else 1.0 / max(s.temperature, 1e-6) for s in seqs], dtype=torch.float32)
        gr = torch.tensor([int(s.greedy) for s in seqs], dtype=torch.int32)
        sd = torch.tensor([s.seed & 0x7FFFFFFF for s in seqs], dtype=torch.int32)
        self.s_inv_temp[:n].copy_(inv_t, non_blocking=True)
        self.s_greedy[:n].copy_(gr, non_blocking=True)
        self.s_seeds[:n].copy_(sd, non_blocking=True)
        self._sample_rows(logits, n, self.s_inv_temp, self.s_greedy, self.s_seeds)
        return self._fetch_samples(n)

    # ---- stable rows of the static decode buffers
    def _assign_row(self, s: _Seq):
        assert s.row < 0 and s.pages, "a sequence gets a decode row once, after its pages"
        r = self._rows_free.pop()
        s.row = r
        self._row_seq[r] = s
        self.hn_pt[r, :] = 0
        self.hn_pt[r, :len(s.pages)] = s.pages
        self.hn_greedy[r] = int(s.greedy)
        self.hn_seeds[r] = s.seed & 0x7FFFFFFF
        self.hn_inv_temp[r] = 1.0 if s.greedy else 1.0 / max(s.temperature, 1e-6)
        p = len(s.tokens) - 1              # position of the token the next decode step feeds
        self.hn_tokens[r] = s.tokens[-1]
        self.hn_pos[r] = p + s.rope_delta  # rotary position; the cache slot comes from hn_lens
        self.hn_lens[r] = p + 1

    def _free_row(self, s: _Seq):
        r = s.row
        s.row = -1
        if r < 0 or self._row_seq[r] is not s:
            return
        self._row_seq[r] = None
        self.hn_lens[r] = 0
        self.hn_slots[r] = -1
        self.hn_tokens[r] = 0
        self.hn_pos[r] = 0
        # keep the free list sorted descending so pop() returns the lowest row
        import bisect

        keys = [-x for x in self._rows_free]
        self._rows_free.insert(bisect.bisect_left(keys, -r), r)

    def _decode_forward(self, B: int) -> torch.Tensor:
        """One decode step over the static buffers (first B rows). Returns fp32 logits [B, V]."""
        st = self.d_state
        pb = PackedBatch.__new__(PackedBatch)
        pb.cu_seqlens = None
        pb.position_ids = st[:B, 1]
        pb.total_tokens, pb.max_seqlen, pb.tile_info = B, 1, None
        fns = self._layer_attn_fns("decode", slots=self.s_slots[:B], pt=self.s_pt[:B], lens=self.s_lens[:B])
        # strided columns of the packed state -> the contiguous buffers the kernels read
        self.s_tokens[:B].copy_(st[:B, 0])
        self.s_pos[:B].copy_(st[:B, 1])
        self.s_slots[:B].copy_(st[:B, 2])
        self.s_lens[:B].copy_(st[:B, 3])
        self.s_pt[:B].copy_(st[:B, 7:])
        pb.position_ids = self.s_pos[:B]
        hidden = self.model.forward_hidden(self.s_tokens[:B], pb, attn_fns=fns)
        return self.model.logits(hidden)

    def _decode(self, seqs: list[_Seq], done: list):
        """One decode step for every running row. Host work is vectorised over rows (numpy on
        the pinned mirror) and the step costs one H2D copy, one graph replay, the sampling
        launch and one D2H copy."""
        seqs = self._grow_pages(seqs, done)
        if not seqs:
            return
        hi = max(s.row for s in seqs) + 1
        B = min(next(b for b in DECODE_BUCKETS if b >= hi), self.max_batch)
        ps = self.cache.page_size
        active = self.hn_lens[:B] > 0
        pos = np.maximum(self.hn_lens[:B] - 1, 0)   # index of the fed token inside its sequence
        page = self.hn_pt[np.arange(B), np.minimum(pos // ps, self.max_pages_per_seq - 1)]
        self.hn_slots[:B] = np.where(active, page * ps + pos % ps, -1)
        self.d_state[:B].copy_(self.h_state[:B], non_blocking=True)
        if self.icfg.use_cuda_graph:
            g = self._graphs.get(B)
            if g is None:
                g = self._capture(B)
            graph, logits, n_kernels = g
            graph.replay()
            oplib.LAUNCHES["count"] += n_kernels
        else:
            logits = self._decode_forward(B)
        plain = all(s.top_p >= 1.0 and s.top_k <= 0 for s in seqs)
        if plain:
            st = self.d_state
            self.s_greedy[:B].copy_(st[:B, 4])
            self.s_seeds[:B].copy_(st[:B, 5])
            self.s_inv_temp[:B].copy_(st[:B, 6].view(torch.float32))
            self._sample_rows(logits, B, self.s_inv_temp, self.s_greedy, self.s_seeds)
            toks, lps = self._fetch_samples(B)
        else:
            self._step += 1
            lg = logits[:B].float().cpu()
            toks, lps = [0] * B, [0.0] * B
            for s in seqs:
                toks[s.row], lps[s.row] = self._sample_cpu(lg[s.row], s)
        self.stats["decode_steps"] += 1
        # advance the mirrors for the next step (vectorised), then per-sequence bookkeeping
        self.hn_tokens[:B] = np.where(active, np.asarray(toks, dtype=np.int32), 0)
        self.hn_pos[:B] += active
        self.hn_lens[:B] += active
        for s in seqs:
            r = s.row
            self._accept_token(s, toks[r], lps[r], done)

    def _capture(self, B: int):
        # warm-up outside capture (sets kernel attributes, allocates the error word)
        for _ in range(2):
            self._decode_forward(B)
        self.stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = oplib.launch_count()
        # thread_local: other threads (the colocated trainer) keep issuing CUDA work meanwhile
        with torch.cuda.graph(graph, stream=self.stream, capture_error_mode="thread_local"):
            logits = self._decode_forward(B)
        n_kernels = oplib.launch_count() - n0
        oplib.LAUNCHES["count"] = n0  # capture itself executes nothing
        self._graphs[B] = (graph, logits, n_kernels)
        return self._graphs[B]

    def export_stats(self) -> dict[str, float]:
        out = {f"infer/{k}": float(v) for k, v in self.stats.items()}
        out["infer/alive_seconds"] = time.perf_counter() - self._t_start
        return out


def _apply_top_k_top_p(z: torch.Tensor, top_k: int, top_p: float) -> torch.Tensor:
    if top_k and top_k > 0 and top_k < z.numel():
        kth = torch.topk(z, top_k).values[-1]
        z = torch.where(z < kth, torch.full_like(z, float("-inf")), z)
    if top_p < 1.0:
        sz, idx = torch.sort(z, descending=True)
        probs = torch.softmax(sz, -1)
        cum = torch.cumsum(probs, -1)
        remove = cum - probs > top_p
        sz = torch.where(remove, torch.full_like(sz, float("-inf")), sz)
        z = torch.full_like(z, float("-inf")).scatter(0, idx, sz)
    return z
