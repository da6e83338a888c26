"""Data proxy: one per inference worker. Owns the RL sessions that run on that worker: every
session is an :class:`ArealOpenAI` client over the worker's engine; chat completions are
recorded token by token, rewards are attached, finished sessions are exported as training
trajectories. Also forwards pause / continue / version / memory control to the engine.
Reference: ``areal/v2/inference_service/data_proxy/{app.py, session.py}``."""
from __future__ import annotations

import asyncio
import secrets
import threading
import time
from typing import Any, Optional

from ...api.cli_args import GenerationHyperparameters
from ...openai.client import ArealOpenAI
from ..common import HTTPError, JsonService


class Session:
    def __init__(self, client: ArealOpenAI, task_id: Optional[str]):
        self.client, self.task_id = client, task_id
        self.created = self.last_used = time.time()
        self.finished = False


class DataProxy:
    def __init__(self, engine, tokenizer, gconfig: Optional[GenerationHyperparameters] = None, host: str = "127.0.0.1",
                 port: Optional[int] = None, session_timeout: float = 3600.0, chat_template_type: str = "hf"):
        self.engine, self.tokenizer, self.gconfig = engine, tokenizer, gconfig or GenerationHyperparameters()
        self.chat_template_type = chat_template_type
        self.session_timeout = session_timeout
        self.sessions: dict[str, Session] = {}
        self.ready: list[tuple[str, Session]] = []          # finished sessions waiting for export
        self._lock = threading.Lock()
        self._loop = asyncio.new_event_loop()
        threading.Thread(target=self._loop.run_forever, daemon=True, name="data-proxy-loop").start()
        self.svc = JsonService("data_proxy", host, port)
        self._install()

    # ------------------------------------------------------------------ helpers
    def _get(self, key: Optional[str]) -> Session:
        with self._lock:
            s = self.sessions.get(key or "")
        if s is None:
            raise HTTPError(401, "unknown session key")
        if s.finished:
            raise HTTPError(409, "session already finished")
        s.last_used = time.time()
        return s

    def _run(self, coro):
        return asyncio.run_coroutine_threadsafe(coro, self._loop).result()

    def gc(self) -> int:
        """Drops sessions idle for longer than the timeout."""
        now = time.time()
        with self._lock:
            dead = [k for k, s in self.sessions.items() if now - s.last_used > self.session_timeout]
            for k in dead:
                del self.sessions[k]
        return len(dead)

    # ------------------------------------------------------------------ routes
    def _install(self):
        svc = self.svc

        @svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "sessions": len(self.sessions), "ready": len(self.ready), "version": self.engine.get_version()}

        @svc.route("POST", "/rl/start_session")
        def start(body, ctx):
            key = "sk-sess-" + secrets.token_hex(16)
            cl = ArealOpenAI(self.engine, self.tokenizer, gconfig=self.gconfig, chat_template_type=self.chat_template_type)
            with self._lock:
                self.sessions[key] = Session(cl, body.get("task_id"))
            return {"session_id": key, "api_key": key}

        @svc.route("POST", "/v1/chat/completions")
        @svc.route("POST", "/chat/completions")
        def chat(body, ctx):
            s = self._get(ctx.api_key)
            kw = {k: body[k] for k in ("messages", "model", "temperature", "top_p", "max_tokens", "max_completion_tokens", "stop",
                                        "tools", "tool_choice", "frequency_penalty", "extra_body", "metadata") if k in body}
            comp = self._run(s.client.chat.completions.create(**kw))
            if body.get("stream"):
                # the completion is recorded whole (the trajectory needs it); the client gets it as chunk events
                from ...openai.proxy import chat_completion_chunks
                from ..common import SSE

                return SSE(list(chat_completion_chunks(comp)) + ["[DONE]"])
            return comp.to_dict()

        @svc.route("POST", "/v1/messages")
        def messages(body, ctx):
            # Anthropic Messages shape over the same recorded chat call (system prompt, content blocks, tools translated both ways)
            from ...openai.proxy import anthropic_message_events, anthropic_to_openai, openai_to_anthropic
            from ..common import SSE

            s = self._get(ctx.api_key)
            kw = {k: v for k, v in anthropic_to_openai(body).items() if v is not None}
            msg = openai_to_anthropic(self._run(s.client.chat.completions.create(**kw)))
            return SSE(list(anthropic_message_events(msg))) if body.get("stream") else msg

        @svc.route("POST", "/v1/responses")
        def responses(body, ctx):
            s = self._get(ctx.api_key)
            kw = {k: body[k] for k in ("input", "instructions", "model", "max_output_tokens", "temperature", "top_p", "tools") if k in body}
            r = self._run(s.client.responses.create(**kw))
            u = r.usage
            return {"id": r.id, "object": "response", "created_at": r.created_at, "model": r.model, "status": "completed", "output": r.output,
                    "output_text": r.output_text, "usage": {"input_tokens": u.prompt_tokens, "output_tokens": u.completion_tokens,
                                                            "total_tokens": u.total_tokens}}

        # tokenizer service: agents and evaluators that count or cut tokens use the policy's own tokenizer without
        # loading it (reference: areal/v2/inference_service/data_proxy/tokenizer_proxy.py)
        @svc.route("POST", "/tokenize")
        def tokenize(body, ctx):
            if "messages" in body:
                ids = self.tokenizer.apply_chat_template(body["messages"], tokenize=True, add_generation_prompt=bool(body.get("add_generation_prompt", True)))
            else:
                ids = self.tokenizer.encode(body["text"])
            ids = [int(i) for i in ids]
            return {"input_ids": ids, "count": len(ids)}

        @svc.route("POST", "/detokenize")
        def detokenize(body, ctx):
            return {"text": self.tokenizer.decode([int(i) for i in body["input_ids"]])}

        @svc.route("POST", "/rl/set_reward")
        def set_reward(body, ctx):
            s = self._get(ctx.api_key)
            if body.get("interaction_id"):
                s.client.set_reward(body["interaction_id"], float(body["reward"]))
            else:
                s.client.set_last_reward(float(body["reward"]))
            return {"ok": True}

        @svc.route("POST", "/rl/end_session")
        def end(body, ctx):
            s = self._get(ctx.api_key)
            s.finished = True
            with self._lock:
                self.sessions.pop(ctx.api_key, None)
                self.ready.append((ctx.api_key, s))
            return {"ok": True, "interactions": len(s.client._cache)}

        @svc.route("POST", "/export_trajectories")
        def export(body, ctx):
            style, discount = body.get("style", "individual"), body.get("discount", 1.0)
            with self._lock:
                take, self.ready = self.ready[: int(body.get("max_sessions", 1 << 30))], self.ready[int(body.get("max_sessions", 1 << 30)):]
            out = []
            for key, s in take:
                inter = s.client.export_interactions(style, discount)
                tds = [v.to_tensor_dict() for v in inter.values() if v.has_tensor_data]
                out.append({"session_id": key, "task_id": s.task_id,
                            "trajectories": [{k: (t[0].tolist() if t.dim() == 2 else t.tolist()) for k, t in td.items()} for td in tds]})
            return {"sessions": out}

        @svc.route("POST", "/pause_generation")
        def pause(body, ctx):
            self.engine.pause_generation()
            return {"ok": True}

        @svc.route("POST", "/continue_generation")
        def cont(body, ctx):
            self.engine.continue_generation()
            return {"ok": True}

        @svc.route("POST", "/set_version")
        def set_version(body, ctx):
            self.engine.set_version(int(body["version"]))
            return {"ok": True}

        @svc.route("POST", "/update_weights_from_http")
        def update_http(body, ctx):
            # pulls the trainer's weight dictionary (torch.save bytes) and hands it to the engine; the caller has paused
            # generation, or the engine swaps at its next step boundary
            import io

            import torch

            from ..common import fetch_bytes

            named = torch.load(io.BytesIO(fetch_bytes(body["url"], timeout=float(body.get("timeout_s", 600)))), map_location="cpu", weights_only=True)
            res = self.engine.update_weights_from_tensors(named)
            if hasattr(res, "result"):
                res.result()
            if body.get("version") is not None:
                self.engine.set_version(int(body["version"]))
            return {"ok": True, "tensors": len(named)}

        @svc.route("POST", "/release_memory")
        def release(body, ctx):
            self.engine.offload(body.get("tags"))
            return {"ok": True}

        @svc.route("POST", "/resume_memory")
        def resume(body, ctx):
            self.engine.onload(body.get("tags"))
            return {"ok": True}

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()
        self._loop.call_soon_threadsafe(self._loop.stop)

    @property
    def address(self) -> str:
        return self.svc.address
