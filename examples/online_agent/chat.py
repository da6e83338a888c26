"""A chat loop against a session of the trainer's proxy (``You:`` prompt; an empty line ends it). Any other client works
the same way: point an OpenAI-compatible SDK at ``<url>/v1`` with the session key as the API key."""
import argparse

from _http import post

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8090")
    ap.add_argument("--key", required=True)
    ap.add_argument("--max-tokens", type=int, default=512)
    a = ap.parse_args()
    messages = []
    while True:
        try:
            text = input("You: ").strip()
        except EOFError:
            break
        if not text:
            break
        messages.append({"role": "user", "content": text})
        r = post(f"{a.url}/v1/chat/completions", {"messages": messages, "max_tokens": a.max_tokens}, a.key)
        reply = r["choices"][0]["message"]["content"]
        print("Model:", reply)
        messages.append({"role": "assistant", "content": reply})
