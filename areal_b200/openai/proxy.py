"""HTTP front of the OpenAI-compatible client for agents that only speak HTTP.

Each episode opens a session (``start_session`` → key); the agent uses the key as its API key
against ``{base_url}/chat/completions``; rewards arrive with ``POST /rl/set_reward`` and the
episode is closed by ``POST /rl/end_session``; trajectories leave through
``POST /rl/export_trajectories``. Anthropic-style ``/v1/messages`` requests are translated to
chat completions. Reference: ``areal/experimental/openai/proxy/*`` (session keys, FastAPI
routes) and the gateway routes of ``areal/v2/inference_service/gateway/app.py``.

The server is stdlib-only (``ThreadingHTTPServer``); model calls are executed on one
background asyncio loop shared by all sessions.
"""
from __future__ import annotations

import asyncio
import json
import queue
import secrets
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Optional

from ..utils import logging as alog
from ..utils.network import find_free_ports
from .client import ArealOpenAI

logger = alog.getLogger("openai_proxy")


def anthropic_to_openai(body: dict) -> dict:
    """Translates a ``/v1/messages`` request into chat-completions arguments."""
    msgs: list[dict] = []
    sys_ = body.get("system")
    if sys_:
        if isinstance(sys_, list):
            sys_ = "".join(p.get("text", "") for p in sys_)
        msgs.append({"role": "system", "content": sys_})
    for m in body.get("messages", []):
        c = m.get("content")
        if isinstance(c, list):
            text, tool_results = [], []
            for p in c:
                if p.get("type") == "text":
                    text.append(p.get("text", ""))
                elif p.get("type") == "tool_result":
                    tr = p.get("content")
                    if isinstance(tr, list):
                        tr = "".join(q.get("text", "") for q in tr)
                    tool_results.append({"role": "tool", "tool_call_id": p.get("tool_use_id"), "content": tr or ""})
                elif p.get("type") == "tool_use":
                    msgs.append({"role": "assistant", "content": "", "tool_calls": [
                        {"id": p.get("id"), "type": "function", "function": {"name": p.get("name"), "arguments": json.dumps(p.get("input", {}))}}]})
            msgs.extend(tool_results)
            if text:
                msgs.append({"role": m.get("role", "user"), "content": "".join(text)})
        else:
            msgs.append({"role": m.get("role", "user"), "content": c or ""})
    tools = [{"type": "function", "function": {"name": t["name"], "description": t.get("description", ""),
                                               "parameters": t.get("input_schema", {})}} for t in body.get("tools", [])] or None
    return {"messages": msgs, "max_completion_tokens": body.get("max_tokens"), "temperature": body.get("temperature"),
            "top_p": body.get("top_p"), "tools": tools, "stop": body.get("stop_sequences")}


def openai_to_anthropic(comp) -> dict:
    m = comp.choices[0].message
    content: list[dict] = []
    if m.content:
        content.append({"type": "text", "text": m.content})
    for t in m.tool_calls or []:
        content.append({"type": "tool_use", "id": t.id, "name": t.function.name, "input": json.loads(t.function.arguments or "{}")})
    stop = {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use"}.get(comp.choices[0].finish_reason, "end_turn")
    return {"id": comp.id, "type": "message", "role": "assistant", "model": comp.model, "content": content, "stop_reason": stop,
            "usage": {"input_tokens": comp.usage.prompt_tokens, "output_tokens": comp.usage.completion_tokens}}


def chat_completion_chunks(comp, piece_chars: int = 64):
    """Server-sent-event payloads of a finished completion in the ``chat.completion.chunk`` wire
    format: a role delta, content (and reasoning) deltas of at most ``piece_chars`` characters,
    one delta per tool call, then the finish reason with the usage. The model call itself is not
    incremental (the trajectory is recorded whole), so the stream starts once generation ended."""
    base = {"id": comp.id, "object": "chat.completion.chunk", "created": comp.created, "model": comp.model}
    m = comp.choices[0].message

    def ev(delta: dict, finish=None, **extra) -> dict:
        return {**base, "choices": [{"index": 0, "delta": delta, "finish_reason": finish}], **extra}

    yield ev({"role": "assistant", "content": ""})
    for field, text in (("reasoning_content", m.reasoning_content), ("content", m.content)):
        for i in range(0, len(text or ""), piece_chars):
            yield ev({field: text[i:i + piece_chars]})
    for i, t in enumerate(m.tool_calls or []):
        yield ev({"tool_calls": [{"index": i, "id": t.id, "type": "function",
                                  "function": {"name": t.function.name, "arguments": t.function.arguments}}]})
    u = comp.usage
    yield ev({}, comp.choices[0].finish_reason,
             usage={"prompt_tokens": u.prompt_tokens, "completion_tokens": u.completion_tokens, "total_tokens": u.total_tokens})


def anthropic_message_events(msg: dict, piece_chars: int = 64):
    """(event name, payload) pairs of the ``/v1/messages`` streaming protocol for a finished message."""
    head = {k: v for k, v in msg.items() if k not in ("content", "stop_reason")}
    yield "message_start", {"type": "message_start", "message": {**head, "content": [], "stop_reason": None}}
    for i, blk in enumerate(msg["content"]):
        if blk["type"] == "text":
            yield "content_block_start", {"type": "content_block_start", "index": i, "content_block": {"type": "text", "text": ""}}
            for j in range(0, len(blk["text"]), piece_chars):
                yield "content_block_delta", {"type": "content_block_delta", "index": i,
                                              "delta": {"type": "text_delta", "text": blk["text"][j:j + piece_chars]}}
        else:
            yield "content_block_start", {"type": "content_block_start", "index": i,
                                          "content_block": {"type": "tool_use", "id": blk["id"], "name": blk["name"], "input": {}}}
            yield "content_block_delta", {"type": "content_block_delta", "index": i,
                                          "delta": {"type": "input_json_delta", "partial_json": json.dumps(blk["input"])}}
        yield "content_block_stop", {"type": "content_block_stop", "index": i}
    yield "message_delta", {"type": "message_delta", "delta": {"stop_reason": msg["stop_reason"]},
                            "usage": {"output_tokens": msg["usage"]["output_tokens"]}}
    yield "message_stop", {"type": "message_stop"}


class _Session:
    def __init__(self, client: ArealOpenAI):
        self.client = client
        self.created = time.time()
        self.ended = False
        self.final_reward: Optional[float] = None


class OpenAIProxyServer:
    def __init__(self, engine=None, tokenizer=None, gconfig=None, host: str = "127.0.0.1", port: Optional[int] = None,
                 admin_key: Optional[str] = None, chat_template_type: str = "hf"):
        self.engine, self.tokenizer, self.gconfig = engine, tokenizer, gconfig
        self.chat_template_type = chat_template_type
        self.host, self.port = host, port or find_free_ports(1)[0]
        self.admin_key = admin_key
        self._sessions: dict[str, _Session] = {}
        self._lock = threading.Lock()
        # online training: sessions opened over HTTP by an outside user are queued here when that user ends them
        self._external: set[str] = set()
        self._completed: "queue.Queue[str]" = queue.Queue()
        self._loop = asyncio.new_event_loop()
        self._loop_thread = threading.Thread(target=self._loop.run_forever, daemon=True, name="openai-proxy-loop")
        self._srv: Optional[ThreadingHTTPServer] = None

    @property
    def base_url(self) -> str:
        return f"http://{self.host}:{self.port}/v1"

    # ---- sessions
    def start_session(self, client: Optional[ArealOpenAI] = None) -> str:
        if client is None:
            client = ArealOpenAI(self.engine, self.tokenizer, gconfig=self.gconfig, chat_template_type=self.chat_template_type)
        key = "sk-sess-" + secrets.token_hex(16)
        with self._lock:
            self._sessions[key] = _Session(client)
        return key

    def end_session(self, key: str) -> None:
        with self._lock:
            s = self._sessions.get(key)
            done = s is not None and not s.ended and key in self._external
            if s is not None:
                s.ended = True
        if done:
            self._completed.put(key)

    def wait_for_completed_session(self, timeout: Optional[float] = None) -> Optional[str]:
        """Blocks until an outside user has finished a session it opened through ``/rl/start_session`` (start ->
        chat -> set_reward -> end_session); returns that session's key, ``None`` on timeout. The caller pops and exports
        it. Reference: the wait-for-session route of ``areal/experimental/openai/proxy/proxy_gateway.py`` used by
        ``online_agent.py``."""
        try:
            return self._completed.get(timeout=timeout)
        except queue.Empty:
            return None

    def pop_session(self, key: str) -> Optional[_Session]:
        with self._lock:
            self._external.discard(key)
            return self._sessions.pop(key, None)

    def _session(self, key: Optional[str]) -> _Session:
        with self._lock:
            s = self._sessions.get(key or "")
        if s is None:
            raise PermissionError("unknown session key")
        if s.ended:
            raise PermissionError("session already ended")
        return s

    def _run(self, coro):
        return asyncio.run_coroutine_threadsafe(coro, self._loop).result()

    # ---- HTTP
    def start(self):
        self._loop_thread.start()
        proxy = self

        class H(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def _key(self) -> Optional[str]:
                a = self.headers.get("Authorization", "")
                if a.lower().startswith("bearer "):
                    return a[7:].strip()
                return self.headers.get("x-api-key")

            def _reply(self, code: int, obj: Any):
                body = json.dumps(obj).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def _stream(self, events):
                """Server-sent events over chunked transfer encoding; ``events`` yields payload dicts or
                (event name, payload) pairs; a bare string is sent as is (the ``[DONE]`` sentinel)."""
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Transfer-Encoding", "chunked")
                self.end_headers()
                for e in events:
                    if isinstance(e, tuple):
                        data = f"event: {e[0]}\ndata: {json.dumps(e[1])}\n\n"
                    else:
                        data = f"data: {e if isinstance(e, str) else json.dumps(e)}\n\n"
                    raw = data.encode()
                    self.wfile.write(f"{len(raw):x}\r\n".encode() + raw + b"\r\n")
                    self.wfile.flush()
                self.wfile.write(b"0\r\n\r\n")

            def do_GET(self):
                if self.path in ("/health", "/v1/health"):
                    return self._reply(200, {"status": "ok", "sessions": len(proxy._sessions)})
                if self.path in ("/v1/models", "/models"):
                    return self._reply(200, {"object": "list", "data": [{"id": "default", "object": "model"}]})
                self._reply(404, {"error": "unknown route"})

            def do_POST(self):
                n = int(self.headers.get("Content-Length", "0"))
                try:
                    body = json.loads(self.rfile.read(n)) if n else {}
                    path = self.path.split("?")[0].rstrip("/")
                    if path.endswith("/chat/completions"):
                        s = proxy._session(self._key())
                        kw = {k: body[k] for k in ("messages", "model", "temperature", "top_p", "max_tokens", "max_completion_tokens",
                                                    "stop", "tools", "tool_choice", "frequency_penalty", "extra_body", "metadata") if k in body}
                        comp = proxy._run(s.client.chat.completions.create(**kw))
                        if body.get("stream"):
                            return self._stream(list(chat_completion_chunks(comp)) + ["[DONE]"])
                        return self._reply(200, comp.to_dict())
                    if path.endswith("/responses"):
                        s = proxy._session(self._key())
                        kw = {k: body[k] for k in ("input", "instructions", "model", "max_output_tokens", "temperature", "top_p",
                                                    "tools") if k in body}
                        r = proxy._run(s.client.responses.create(**kw))
                        u = r.usage
                        return self._reply(200, {"id": r.id, "object": "response", "created_at": r.created_at, "model": r.model,
                                                 "status": "completed", "output": r.output, "output_text": r.output_text,
                                                 "usage": {"input_tokens": u.prompt_tokens, "output_tokens": u.completion_tokens,
                                                           "total_tokens": u.total_tokens}})
                    if path.endswith("/v1/messages") or path == "/messages":
                        s = proxy._session(self._key())
                        kw = {k: v for k, v in anthropic_to_openai(body).items() if v is not None}
                        comp = proxy._run(s.client.chat.completions.create(**kw))
                        if body.get("stream"):
                            return self._stream(anthropic_message_events(openai_to_anthropic(comp)))
                        return self._reply(200, openai_to_anthropic(comp))
                    if path == "/rl/start_session":
                        if proxy.admin_key and self._key() != proxy.admin_key:
                            raise PermissionError("admin key required")
                        key = proxy.start_session()
                        with proxy._lock:
                            proxy._external.add(key)
                        return self._reply(200, {"api_key": key, "base_url": proxy.base_url})
                    if path == "/rl/set_reward":
                        s = proxy._session(self._key())
                        if body.get("interaction_id"):
                            s.client.set_reward(body["interaction_id"], float(body["reward"]))
                        else:
                            s.client.set_last_reward(float(body["reward"]))
                        return self._reply(200, {"ok": True})
                    if path == "/rl/end_session":
                        proxy.end_session(self._key())
                        return self._reply(200, {"ok": True})
                    if path == "/rl/export_trajectories":
                        key = body.get("api_key") or self._key()
                        s = proxy.pop_session(key)
                        if s is None:
                            raise PermissionError("unknown session key")
                        inter = s.client.export_interactions(body.get("style", "individual"), body.get("discount"))
                        out = {}
                        for cid, it in inter.items():
                            td = it.to_tensor_dict()
                            out[cid] = {k: v[0].tolist() if v.dim() == 2 else v.tolist() for k, v in td.items()}
                        return self._reply(200, {"interactions": out})
                    self._reply(404, {"error": "unknown route"})
                except PermissionError as e:
                    self._reply(401, {"error": str(e)})
                except (KeyError, ValueError, TypeError, NotImplementedError) as e:
                    self._reply(400, {"error": repr(e)})
                except Exception as e:  # engine failure
                    logger.error("proxy request failed: %r", e)
                    self._reply(500, {"error": repr(e)})

        self._srv = ThreadingHTTPServer((self.host, self.port), H)
        self._srv.daemon_threads = True
        threading.Thread(target=self._srv.serve_forever, daemon=True, name="openai-proxy").start()
        return self

    def stop(self):
        if self._srv is not None:
            self._srv.shutdown()
            self._srv.server_close()
            self._srv = None
        self._loop.call_soon_threadsafe(self._loop.stop)


class HostedProxy:
    """An :class:`OpenAIProxyServer` created inside an RPC worker over an engine that the worker already hosts
    (agents reach the rollout engine of that worker over HTTP; the trajectories stay on the worker until they
    are exported). The role of the reference's forked proxy rollout server
    (``areal/infra/controller/rollout_controller.py:406-471``); here the engine lives in the worker process, so
    the proxy is a set of threads beside it instead of a second process."""

    def __init__(self, engine_name: str, tokenizer: str, tokenizer_kwargs: Optional[dict] = None, gconfig: Optional[dict] = None,
                 admin_key: Optional[str] = None, host: str = "127.0.0.1", chat_template_type: str = "hf"):
        from ..api.cli_args import GenerationHyperparameters
        from ..infra.rpc.hosted import HOSTED_ENGINES
        from ..utils.dynamic_import import import_from_string

        if engine_name not in HOSTED_ENGINES:
            raise KeyError(f"no engine '{engine_name}' is hosted by this worker (have: {sorted(HOSTED_ENGINES)})")
        tok = import_from_string(tokenizer)(**(tokenizer_kwargs or {}))
        g = GenerationHyperparameters(**gconfig) if isinstance(gconfig, dict) else (gconfig or GenerationHyperparameters())
        self.server = OpenAIProxyServer(HOSTED_ENGINES[engine_name], tok, g, host=host, admin_key=admin_key,
                                        chat_template_type=chat_template_type)

    def initialize(self) -> str:
        self.server.start()
        return self.server.base_url

    def base_url(self) -> str:
        return self.server.base_url

    def n_sessions(self) -> int:
        return len(self.server._sessions)

    def destroy(self) -> None:
        self.server.stop()
