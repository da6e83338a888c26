"""Opens a session on the trainer's proxy and prints its API key (use it as the OpenAI / Anthropic API key)."""
import argparse

from _http import post

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8090")
    ap.add_argument("--admin-key", required=True)
    a = ap.parse_args()
    r = post(f"{a.url}/rl/start_session", {}, a.admin_key)
    print(r["api_key"])
    print(f"# OPENAI_BASE_URL={r['base_url']} OPENAI_API_KEY={r['api_key']}")
