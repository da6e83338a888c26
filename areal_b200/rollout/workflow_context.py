"""Per-episode context (is_eval, task id, sample index) carried through asyncio via
``contextvars`` (reference: ``areal/infra/workflow_context.py:25-60``)."""
from __future__ import annotations

import contextvars
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class WorkflowContext:
    is_eval: bool = False
    task_id: Optional[int] = None
    sample_idx: Optional[int] = None


_CTX: contextvars.ContextVar[WorkflowContext] = contextvars.ContextVar("areal_workflow_ctx", default=WorkflowContext())


def get() -> WorkflowContext:
    return _CTX.get()


@contextmanager
def scoped(is_eval: bool = False, task_id: Optional[int] = None, sample_idx: Optional[int] = None):
    tok = _CTX.set(WorkflowContext(is_eval, task_id, sample_idx))
    try:
        yield
    finally:
        _CTX.reset(tok)


def stat_scope() -> str:
    return "eval-rollout" if get().is_eval else "rollout"


# --------------------------------------------------------------------------- shared HTTP clients
class HttpClientManager:
    """One ``aiohttp.ClientSession`` and one ``httpx.AsyncClient`` per running event loop, shared by every episode on
    that loop: workflows and agent SDKs that talk HTTP (tool servers, the per-episode proxy) reuse connections instead of
    opening a pool per episode. A client belongs to the loop it was made on; clients of loops that have closed are
    dropped on the next call, and :meth:`aclose` closes the current loop's clients. Reference:
    ``areal/infra/workflow_context.py:71-240`` (``HttpClientManager``)."""

    def __init__(self, timeout: float = 3600.0, max_connections: int = 0):
        self.timeout, self.max_connections = timeout, max_connections
        self._aio: dict[int, tuple] = {}
        self._httpx: dict[int, tuple] = {}

    @staticmethod
    def _loop():
        import asyncio

        return asyncio.get_running_loop()

    def _sweep(self, table: dict) -> None:
        for key, (loop, _client) in list(table.items()):
            if loop.is_closed():
                table.pop(key, None)          # its transports died with the loop

    def aiohttp_session(self):
        import aiohttp

        loop = self._loop()
        self._sweep(self._aio)
        ent = self._aio.get(id(loop))
        if ent is None or ent[1].closed:
            s = aiohttp.ClientSession(connector=aiohttp.TCPConnector(limit=self.max_connections), timeout=aiohttp.ClientTimeout(total=self.timeout))
            self._aio[id(loop)] = ent = (loop, s)
        return ent[1]

    def httpx_client(self):
        import httpx

        loop = self._loop()
        self._sweep(self._httpx)
        ent = self._httpx.get(id(loop))
        if ent is None or ent[1].is_closed:
            limits = httpx.Limits(max_connections=self.max_connections or None, max_keepalive_connections=self.max_connections or None)
            c = httpx.AsyncClient(timeout=httpx.Timeout(self.timeout), limits=limits)
            self._httpx[id(loop)] = ent = (loop, c)
        return ent[1]

    async def aclose(self) -> None:
        loop = self._loop()
        ent = self._aio.pop(id(loop), None)
        if ent is not None and not ent[1].closed:
            await ent[1].close()
        ent = self._httpx.pop(id(loop), None)
        if ent is not None and not ent[1].is_closed:
            await ent[1].aclose()


_HTTP = HttpClientManager()


def get_aiohttp_session():
    """The running loop's shared ``aiohttp.ClientSession``."""
    return _HTTP.aiohttp_session()


def get_httpx_client():
    """The running loop's shared ``httpx.AsyncClient`` (what the openai / anthropic SDKs accept as ``http_client``)."""
    return _HTTP.httpx_client()


async def close_http_clients() -> None:
    await _HTTP.aclose()
