"""HTTP server around :class:`NativeInferenceEngine` — the process a remote rollout client
talks to (the role SGLang / vLLM servers play for the reference; request shapes follow
``areal/engine/sglang_remote.py:54-392``).

    python -m areal_b200.engine.server --model-path /ckpt --port 30000 [--preset qwen3-8b]

Routes (JSON):
    GET  /health, /get_model_info, /get_version
    POST /generate {rid, input_ids, sampling_params{max_new_tokens, temperature, top_p, top_k,
                    stop_token_ids, ignore_eos, min_new_tokens}, return_logprob}
         -> {output_ids, output_logprobs, output_versions, meta_info{finish_reason{type}, ...}}
    POST /pause_generation, /continue_generation, /abort_request {rid?}, /flush_cache
    POST /update_weights_from_disk {model_path, version?}
    POST /init_weights_update_group {...}, /update_weights_from_distributed {names, dtypes, shapes, version?}
    POST /release_memory_occupation, /resume_memory_occupation
    POST /set_version {version}
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Optional

from ..api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeInferConfig
from ..api.io_struct import ModelRequest, ParamSpec, WeightUpdateMeta
from ..utils import logging as alog
from ..utils import name_resolve, names
from ..utils.network import find_free_ports, gethostip

logger = alog.getLogger("infer_server")


def gconfig_from_sampling_params(sp: dict) -> GenerationHyperparameters:
    t = float(sp.get("temperature", 1.0))
    return GenerationHyperparameters(
        n_samples=1, max_new_tokens=int(sp.get("max_new_tokens", 128)), min_new_tokens=int(sp.get("min_new_tokens", 0)),
        max_tokens=int(sp.get("max_tokens", 1 << 30)), greedy=t == 0.0 or bool(sp.get("greedy", False)), temperature=t if t > 0 else 1.0,
        top_p=float(sp.get("top_p", 1.0)), top_k=int(sp.get("top_k", -1)) if int(sp.get("top_k", -1)) > 0 else int(1e8),
        stop_token_ids=list(sp.get("stop_token_ids") or []), ignore_eos=bool(sp.get("ignore_eos", False)),
        seed=sp.get("seed"))


class InferenceServer:
    def __init__(self, engine, host: str = "127.0.0.1", port: Optional[int] = None):
        self.engine = engine
        self.host, self.port = host, port or find_free_ports(1)[0]
        self._loop = asyncio.new_event_loop()
        self._loop_thread = threading.Thread(target=self._loop.run_forever, daemon=True, name="infer-server-loop")
        self._srv: Optional[ThreadingHTTPServer] = None
        self._inflight: dict[str, Any] = {}
        self._lock = threading.Lock()

    @property
    def address(self) -> str:
        return f"{self.host}:{self.port}"

    def _generate(self, body: dict) -> dict:
        req = ModelRequest(rid=body.get("rid") or os.urandom(8).hex(), input_ids=list(body["input_ids"]),
                           gconfig=gconfig_from_sampling_params(body.get("sampling_params") or {}))
        req.gconfig.max_tokens = max(req.gconfig.max_tokens, len(req.input_ids) + req.gconfig.max_new_tokens)
        fut = asyncio.run_coroutine_threadsafe(self.engine.agenerate(req), self._loop)
        with self._lock:
            self._inflight[req.rid] = fut
        try:
            r = fut.result()
        finally:
            with self._lock:
                self._inflight.pop(req.rid, None)
        return {"output_ids": r.output_tokens, "output_logprobs": r.output_logprobs, "output_versions": r.output_versions,
                "meta_info": {"finish_reason": {"type": r.stop_reason}, "prompt_tokens": r.input_len,
                              "completion_tokens": r.output_len, "latency": r.latency, "ttft": r.ttft}}

    def _dispatch(self, path: str, body: dict) -> dict:
        e = self.engine
        if path == "/generate":
            return self._generate(body)
        if path == "/pause_generation":
            e.pause_generation()
            return {"success": True}
        if path == "/continue_generation":
            e.continue_generation()
            return {"success": True}
        if path == "/abort_request":
            rid = body.get("rid")
            with self._lock:
                futs = [f for k, f in self._inflight.items() if rid in (None, "", k)]
            for f in futs:
                f.cancel()
            return {"success": True, "aborted": len(futs)}
        if path == "/flush_cache":
            return {"success": True}
        if path == "/update_weights_from_disk":
            meta = WeightUpdateMeta(type="disk", path=body["model_path"], version=body.get("version"))
            e.update_weights_from_disk(meta).result()
            return {"success": True, "message": "ok", "version": e.get_version()}
        if path == "/init_weights_update_group":
            meta = WeightUpdateMeta(type="xccl", nccl_master_address=body.get("master_address", "127.0.0.1"),
                                    nccl_master_port=int(body.get("master_port", 29500)),
                                    nccl_group_name=body.get("group_name", "update_weight_group"))
            meta.rank_offset = int(body.get("rank_offset", 1))      # type: ignore[attr-defined]
            meta.world_size = int(body.get("world_size", 2))        # type: ignore[attr-defined]
            e.init_weights_update_group(meta).result()
            return {"success": True}
        if path == "/update_weights_from_distributed":
            specs = [ParamSpec(n, tuple(s), d) for n, d, s in zip(body["names"], body["dtypes"], body["shapes"])]
            meta = WeightUpdateMeta(type="xccl", version=body.get("version"), nccl_group_name=body.get("group_name", "update_weight_group"))
            e.update_weights_from_distributed(meta, specs).result()
            return {"success": True}
        if path == "/release_memory_occupation":
            e.offload(body.get("tags"))
            return {"success": True}
        if path == "/resume_memory_occupation":
            e.onload(body.get("tags"))
            return {"success": True}
        if path == "/set_version":
            e.set_version(int(body["version"]))
            return {"success": True}
        raise KeyError(path)

    def start(self):
        self._loop_thread.start()
        srv = self

        class H(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def _reply(self, code: int, obj):
                b = json.dumps(obj).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(b)))
                self.end_headers()
                self.wfile.write(b)

            def do_GET(self):
                e = srv.engine
                if self.path == "/health" or self.path == "/health_generate":
                    return self._reply(200, {"status": "ok"})
                if self.path == "/get_version":
                    return self._reply(200, {"version": e.get_version()})
                if self.path == "/get_model_info":
                    mc = e.model_config
                    return self._reply(200, {"arch": mc.arch, "vocab_size": mc.vocab_size, "num_layers": mc.num_layers,
                                             "version": e.get_version(), "stats": e.export_stats()})
                self._reply(404, {"error": "unknown route"})

            def do_POST(self):
                n = int(self.headers.get("Content-Length", "0"))
                try:
                    body = json.loads(self.rfile.read(n)) if n else {}
                    self._reply(200, srv._dispatch(self.path.split("?")[0], body))
                except KeyError as ex:
                    self._reply(404, {"error": f"unknown route or missing field {ex}"})
                except (asyncio.CancelledError, cf_CancelledError):
                    self._reply(200, {"output_ids": [], "output_logprobs": [], "output_versions": [],
                                      "meta_info": {"finish_reason": {"type": "abort"}}})
                except Exception as ex:
                    logger.error("request %s failed: %r", self.path, ex)
                    self._reply(500, {"error": repr(ex)})

        self._srv = ThreadingHTTPServer((self.host if self.host != gethostip() else "0.0.0.0", self.port), H)
        self._srv.daemon_threads = True
        self._srv.request_queue_size = 1024
        threading.Thread(target=self._srv.serve_forever, daemon=True, name="infer-server").start()
        logger.info("inference server listening on %s", self.address)
        return self

    def stop(self):
        if self._srv is not None:
            self._srv.shutdown()
            self._srv.server_close()
            self._srv = None
        self._loop.call_soon_threadsafe(self._loop.stop)


from concurrent.futures import CancelledError as cf_CancelledError  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-path", default="")
    ap.add_argument("--preset", default="")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--max-running-requests", type=int, default=256)
    ap.add_argument("--context-length", type=int, default=32768)
    ap.add_argument("--mem-fraction-static", type=float, default=0.85)
    ap.add_argument("--experiment-name", default="")
    ap.add_argument("--trial-name", default="")
    ap.add_argument("--server-index", type=int, default=0)
    ap.add_argument("--seed", type=int, default=1)
    a = ap.parse_args(argv)
    from ..models.config import preset
    from .infer_engine import NativeInferenceEngine

    mc = preset(a.preset) if a.preset else None
    eng = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=a.max_running_requests,
                                                                           context_length=a.context_length,
                                                                           mem_fraction_static=a.mem_fraction_static),
                                model_config=mc)
    eng.initialize(model_path=a.model_path or None, seed=a.seed, start_executor=False)
    srv = InferenceServer(eng, a.host, a.port or None).start()
    if a.experiment_name:
        name_resolve.add_subentry(names.gen_servers(a.experiment_name, a.trial_name), srv.address)
    print(f"INFER_SERVER_READY {srv.address}", flush=True)
    try:
        threading.Event().wait()
    except KeyboardInterrupt:
        pass
    srv.stop()
    eng.destroy()


if __name__ == "__main__":
    main()
