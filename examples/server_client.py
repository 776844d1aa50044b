"""Talk to a running server: list models, one blocking completion, one streamed chat (reference: examples/server_client.rs).

    python -m oxibonsai_b200.server --model-path model.gguf --port 8080 &
    python examples/server_client.py http://127.0.0.1:8080
"""
import json
import sys
import urllib.request

base = sys.argv[1] if len(sys.argv) > 1 else "http://127.0.0.1:8080"


def post(path, body):
    req = urllib.request.Request(base + path, json.dumps(body).encode(), {"content-type": "application/json"})
    return urllib.request.urlopen(req)


print(json.load(urllib.request.urlopen(base + "/v1/models")))
print(json.load(post("/v1/completions", {"prompt": "Hello", "max_tokens": 16}))["choices"][0]["text"])
with post("/v1/chat/completions", {"messages": [{"role": "user", "content": "Hi"}], "stream": True, "max_tokens": 32}) as r:
    for line in r:
        line = line.decode().strip()
        if line.startswith("data: ") and line != "data: [DONE]":
            sys.stdout.write(json.loads(line[6:])["choices"][0]["delta"].get("content", ""))
print()
