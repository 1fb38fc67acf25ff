"""Chat completion over the server's OpenAI-style route, streamed or blocking, with nothing but ``requests``.

    python examples/openai_client.py --port 8080 --stream "Tell me about the sea."

(The ``openai`` package works as well: ``OpenAI(base_url="http://host:port/v1", api_key="none")``.)
"""
import argparse
import json
import sys

import requests


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--stream", action="store_true")
    ap.add_argument("--max_tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("prompt", nargs="?", default="Hello, who are you?")
    args = ap.parse_args(argv)
    body = {"messages": [{"role": "user", "content": args.prompt}], "max_tokens": args.max_tokens,
            "temperature": args.temperature, "stream": args.stream}
    url = f"http://{args.host}:{args.port}/v1/chat/completions"
    if not args.stream:
        doc = requests.post(url, json=body, timeout=600).json()
        if "error" in doc:
            print("error:", doc["error"]["message"], file=sys.stderr)
            return 1
        print(doc["choices"][0]["message"]["content"])
        print(doc["usage"], file=sys.stderr)
        return 0
    with requests.post(url, json=body, stream=True, timeout=600) as resp:
        for line in resp.iter_lines():
            if not line.startswith(b"data: "):
                continue
            data = line[len(b"data: "):]
            if data == b"[DONE]":
                break
            for choice in json.loads(data).get("choices", []):
                sys.stdout.write((choice.get("delta") or {}).get("content") or "")
                sys.stdout.flush()
    print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
