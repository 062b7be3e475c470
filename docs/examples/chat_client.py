"""A streaming chat request against a running server, standard library only.

    python -m hipengine_b200.server --model tiny-dense --backend cpu_reference --port 8000 &
    python docs/examples/chat_client.py --url http://127.0.0.1:8000
"""
import argparse
import json
import urllib.request


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--api-key", default=None)
    a = ap.parse_args()
    headers = {"Content-Type": "application/json"}
    if a.api_key:
        headers["Authorization"] = f"Bearer {a.api_key}"
    model = json.load(urllib.request.urlopen(urllib.request.Request(a.url + "/v1/models", headers=headers)))["data"][0]["id"]
    body = {"model": model, "stream": True, "max_tokens": 64,
            "messages": [{"role": "user", "content": "Say hello in three languages."}],
            "stream_options": {"include_usage": True, "include_hipengine": True}}
    req = urllib.request.Request(a.url + "/v1/chat/completions", data=json.dumps(body).encode(), headers=headers)
    for raw in urllib.request.urlopen(req):
        line = raw.decode().strip()
        if not line.startswith("data: ") or line == "data: [DONE]":
            continue
        ev = json.loads(line[6:])
        for ch in ev.get("choices", []):
            print(ch["delta"].get("content") or "", end="", flush=True)
        if ev.get("usage"):
            print("\n", ev["usage"])


if __name__ == "__main__":
    main()
