"""Example streaming chat client: sends one instruction-style prompt to ``/generate`` with ``stream: true`` and prints
the growing answer as the NUL-separated JSON chunks arrive.

  python examples/streaming_client.py --port 8080 --prompt "Tell me about the moon."

Same command line as the reference's examples/streaming_client.py (which also wraps the prompt in [INST] tags).
"""
import argparse
import json
import sys

import requests


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--host", type=str, default="127.0.0.1")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("--prompt", type=str, default="You are an astronaut on the space station and you see something "
                                                  "approaching. What do you tell ground control?")
    p.add_argument("--stream", action="store_true", help="accepted for compatibility: this client always streams")
    a = p.parse_args(argv)
    body = {"prompt": f"[INST]{a.prompt}[/INST]", "stream": True,
            "sampling_config": {"temperature": 0.0, "topk": 1, "topp": 0.0}}
    resp = requests.post(f"http://{a.host}:{a.port}/generate", json=body, headers={"User-Agent": "ksana example client"},
                         stream=True)
    if resp.status_code != 200:
        print(f"HTTP {resp.status_code}: {resp.text[:400]}", file=sys.stderr)
        return 1
    for chunk in resp.iter_lines(chunk_size=8192, decode_unicode=False, delimiter=b"\0"):
        if chunk:
            print(json.loads(chunk.decode("utf-8"))["texts"], flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
