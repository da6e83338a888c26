"""Wire formats of the generation servers a :class:`RemoteInfEngine` can drive.

The engine's interruptible generation loop, server choice, retries and weight-update fan-out are the same for every
server; what differs is how a request is written and an answer read. A backend turns (prompt tokens, sampling options,
remaining budget) into an HTTP request and an HTTP answer into tokens / log-probs / versions / stop reason, and names the
control endpoints.

* ``native``: this repository's server (``areal_b200/engine/server.py``); answers carry per-token weight versions.
* ``sglang``: an SGLang server (``/generate`` with ``sampling_params``; tokens and log-probs come as
  ``meta_info.output_token_logprobs = [(logprob, token_id, text), ...]``).
* ``vllm``: a vLLM OpenAI-compatible server (``/v1/completions`` with a token-id prompt, ``return_tokens_as_token_ids``
  so that tokens come back as ``"token_id:N"``), with the pause / continue / weight-update routes of the reference's
  server extension.

Reference: ``areal/engine/sglang_remote.py:43-400``, ``areal/engine/vllm_remote.py:40-300`` (request builders and
response parsers of its ``RemoteInfEngine``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass
class HttpRequest:
    endpoint: str
    payload: dict = field(default_factory=dict)
    method: str = "POST"


@dataclass
class GenerationResult:
    tokens: list[int]
    logprobs: list[float]
    stop_reason: str                       # stop | length | abort | tool_calls
    versions: Optional[list[int]] = None   # per-token weight version when the server reports it


def _sampling(g, budget: int, done: int) -> dict:
    return {"max_new_tokens": budget - done, "min_new_tokens": max(0, g.min_new_tokens - done),
            "temperature": 0.0 if g.greedy else g.temperature, "top_p": g.top_p,
            "top_k": -1 if g.top_k >= 10 ** 7 else g.top_k, "stop_token_ids": g.stop_token_ids, "ignore_eos": g.ignore_eos}


class NativeBackend:
    name = "native"
    pause_endpoint, continue_endpoint, health_endpoint = "/pause_generation", "/continue_generation", "/health"
    offload_endpoint, onload_endpoint = "/release_memory_occupation", "/resume_memory_occupation"

    def build_generation(self, rid: str, tokens: list[int], g, budget: int, done: int) -> HttpRequest:
        sp = _sampling(g, budget, done)
        sp["seed"] = g.seed
        return HttpRequest("/generate", {"rid": rid, "input_ids": tokens, "return_logprob": True, "sampling_params": sp})

    def parse_generation(self, r: dict) -> GenerationResult:
        seg = r.get("output_ids", [])
        return GenerationResult(list(seg), list(r.get("output_logprobs", [0.0] * len(seg))), r["meta_info"]["finish_reason"]["type"],
                                r.get("output_versions"))

    def disk_update(self, meta) -> list[HttpRequest]:
        return [HttpRequest("/update_weights_from_disk", {"model_path": meta.path, "version": meta.version})]

    def init_group(self, meta, server_index: int, n_servers: int) -> HttpRequest:
        return HttpRequest("/init_weights_update_group", {
            "master_address": meta.nccl_master_address, "master_port": meta.nccl_master_port, "rank_offset": 1 + server_index,
            "world_size": n_servers + 1, "group_name": meta.nccl_group_name})

    def distributed_update(self, meta, specs) -> list[HttpRequest]:
        return [HttpRequest("/update_weights_from_distributed", {
            "names": [p.name for p in specs], "dtypes": [p.dtype for p in specs], "shapes": [list(p.shape) for p in specs],
            "group_name": meta.nccl_group_name, "version": meta.version})]

    def set_version(self, version: int) -> Optional[HttpRequest]:
        return HttpRequest("/set_version", {"version": version})


class SGLangBackend(NativeBackend):
    name = "sglang"

    def build_generation(self, rid: str, tokens: list[int], g, budget: int, done: int) -> HttpRequest:
        sp = _sampling(g, budget, done)
        sp["skip_special_tokens"] = getattr(g, "skip_special_tokens", True)
        sp["frequency_penalty"] = getattr(g, "frequency_penalty", 0.0)
        if getattr(g, "stop", None):
            sp["stop"] = list(g.stop)
        if g.seed is not None:
            sp["sampling_seed"] = g.seed
        return HttpRequest("/generate", {"rid": rid, "input_ids": tokens, "sampling_params": sp, "return_logprob": True, "stream": False})

    def parse_generation(self, r: dict) -> GenerationResult:
        meta = r["meta_info"]
        fin = meta["finish_reason"]
        if fin["type"] == "abort" and str(fin.get("message", "")).startswith("Abort before prefill"):
            return GenerationResult([], [], "abort")
        pairs = meta.get("output_token_logprobs") or []
        return GenerationResult([int(x[1]) for x in pairs], [float(x[0]) for x in pairs], fin["type"])

    def set_version(self, version: int) -> Optional[HttpRequest]:
        return None                              # the server has no notion of it: the client tags tokens itself


class VLLMBackend(NativeBackend):
    name = "vllm"
    pause_endpoint, continue_endpoint = "/areal_pause_generation", "/areal_continue_generation"
    offload_endpoint, onload_endpoint = "/sleep", "/wake_up"

    def build_generation(self, rid: str, tokens: list[int], g, budget: int, done: int) -> HttpRequest:
        p = {"prompt": tokens, "max_tokens": budget - done, "min_tokens": max(0, g.min_new_tokens - done),
             "temperature": 0.0 if g.greedy else g.temperature, "top_p": g.top_p, "top_k": -1 if g.top_k >= 10 ** 7 else g.top_k,
             "stop_token_ids": g.stop_token_ids, "ignore_eos": g.ignore_eos, "frequency_penalty": getattr(g, "frequency_penalty", 0.0),
             "return_tokens_as_token_ids": True, "logprobs": 0, "stream": False, "request_id": rid}
        if getattr(g, "stop", None):
            p["stop"] = list(g.stop)
        if g.seed is not None:
            p["seed"] = g.seed
        return HttpRequest("/v1/completions", p)

    def parse_generation(self, r: dict) -> GenerationResult:
        ch = r["choices"][0]
        lp = ch.get("logprobs") or {}
        toks = []
        for t in lp.get("tokens", []):
            if not (isinstance(t, str) and t.startswith("token_id:")):
                raise ValueError("the vLLM server must run with return_tokens_as_token_ids (got a text token)")
            toks.append(int(t[len("token_id:"):]))
        fin = ch.get("finish_reason") or "abort"
        return GenerationResult(toks, [float(x) for x in lp.get("token_logprobs", [])], {"stop": "stop", "length": "length"}.get(fin, "abort"))

    def disk_update(self, meta) -> list[HttpRequest]:
        return [HttpRequest("/areal_update_weights", {"model_path": meta.path, "version": meta.version})]

    def init_group(self, meta, server_index: int, n_servers: int) -> HttpRequest:
        r = super().init_group(meta, server_index, n_servers)
        return HttpRequest("/areal_init_weights_update_group", r.payload)

    def distributed_update(self, meta, specs) -> list[HttpRequest]:
        body = super().distributed_update(meta, specs)[0].payload
        return [HttpRequest("/areal_set_update_weight_meta", body), HttpRequest("/areal_update_weights_xccl", {})]

    def set_version(self, version: int) -> Optional[HttpRequest]:
        return None


BACKENDS: dict[str, Any] = {"native": NativeBackend, "sglang": SGLangBackend, "vllm": VLLMBackend, "": NativeBackend}


def get_backend(name: Optional[str]):
    try:
        return BACKENDS[(name or "").lower()]()
    except KeyError:
        raise ValueError(f"unknown generation-server backend '{name}' (native, sglang, vllm)") from None
