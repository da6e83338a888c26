"""Hosting an agent next to the inference gateway (opt-in v2 services).

``AgentController`` starts agent workers plus a gateway that keeps one queue per session: a message
for a session whose run is still active is queued and replayed afterwards (``collect`` folds the
queued messages into one follow-up turn, ``followup`` replays them one by one). The agent is an
ordinary callable ``agent(message, session) -> dict``; ``session.base_url`` / ``session.api_key``
point at the OpenAI-compatible inference gateway so that every model call of the session is recorded
for training (``/rl/start_session``, ``/rl/set_reward``, ``/rl/export_trajectories``).

    python examples/agent_service/chat_service.py                      # echo model, no GPU needed
    python examples/agent_service/chat_service.py http://host:port     # a running inference gateway

Reference behaviour: ``examples/agent_service/`` and ``areal/v2/agent_service`` of the reference project."""
import json
import os
import sys
import urllib.request

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.v2.agent_service import AgentController


def chat_agent(message, session):
    """One turn: the session's history plus the new message go to the model behind the gateway."""
    msgs = [{"role": h.get("role", "user"), "content": h.get("content", "")} for h in session.history if isinstance(h, dict)]
    msgs.append({"role": "user", "content": message})
    if not session.base_url:                                           # no model attached: answer locally
        return {"text": f"(no model) you said: {message}", "turns": len(msgs)}
    req = urllib.request.Request(session.base_url.rstrip("/") + "/chat/completions",
                                 data=json.dumps({"messages": msgs, "max_completion_tokens": 256}).encode(),
                                 headers={"Content-Type": "application/json", "Authorization": f"Bearer {session.api_key}"})
    with urllib.request.urlopen(req, timeout=120) as r:
        out = json.loads(r.read())
    return {"text": out["choices"][0]["message"]["content"], "turns": len(msgs)}


def main(argv):
    ctl = AgentController(chat_agent, n_workers=2, inference_gateway=argv[0] if argv else "")
    try:
        for msg in ("hello", "what did I just say?"):
            r = ctl.run("demo-session", msg)
            print(r["status"], "->", r["result"]["text"])
    finally:
        ctl.close()


if __name__ == "__main__":
    main(sys.argv[1:])
