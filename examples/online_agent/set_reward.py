"""Scores a session (the last model call, or one interaction by id) and, unless ``--keep-open``, closes it: a closed
session is handed to the trainer as one episode."""
import argparse

from _http import post

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8090")
    ap.add_argument("--key", required=True, help="the session key printed by start_session.py")
    ap.add_argument("--reward", type=float, required=True)
    ap.add_argument("--interaction-id", default=None)
    ap.add_argument("--keep-open", action="store_true")
    a = ap.parse_args()
    body = {"reward": a.reward}
    if a.interaction_id:
        body["interaction_id"] = a.interaction_id
    post(f"{a.url}/rl/set_reward", body, a.key)
    if not a.keep_open:
        post(f"{a.url}/rl/end_session", {}, a.key)
    print("ok")
