"""Tiny JSON-over-HTTP helper shared by the session scripts (standard library only)."""
import json
import urllib.request


def post(url: str, body: dict, key: str, timeout: float = 600.0) -> dict:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json", "Authorization": f"Bearer {key}"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read() or b"{}")
