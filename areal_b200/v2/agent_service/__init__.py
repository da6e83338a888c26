"""Agent service: runs user-written agents next to the inference gateway.

* a **worker** hosts one agent callable (an import string) and executes one turn per request:
  ``agent(message, session) -> text | dict``; the agent reaches the model through the inference
  gateway's OpenAI-compatible routes with the session's key, so every completion is recorded for
  training;
* the **gateway** is what clients talk to: ``POST /agent/run`` with a session id and a message.
  One run per session at a time; messages that arrive while a run is active are queued and either
  coalesced into one follow-up turn (``collect``, default) or replayed one by one (``followup``);
  ``GET /agent/runs/{id}`` polls a run, ``POST /agent/sessions/{id}/end`` closes a session
  (optionally forwarding a reward to the inference gateway);
* the **controller** starts workers and a gateway in-process or as child processes and tears them
  down.

Reference: ``areal/v2/agent_service/`` (gateway with ``req`` / ``res`` / ``event`` frames over a
WebSocket, queue modes ``collect`` / ``followup``, data proxy, router, workers, guard). The
transport here is plain JSON over HTTP with polling; payload fields follow ``protocol.py`` /
``types.py`` of the reference (``session_key``, ``message``, ``run_id``, ``status``, ``queue_mode``).
"""
from .service import AgentController, AgentGateway, AgentWorker, SessionInfo  # noqa: F401
