"""Example client of the ``/generate`` endpoint: one prompt, ``n`` answers, blocking or streamed.

  python examples/api_client.py --port 8080 --prompt "San Francisco is a" --n 2
  python examples/api_client.py --port 8080 --stream

Same command line as the reference's examples/api_client.py. The request body is the engine's JSON schema
(``prompt``, ``sampling_config``, ``stream``); a streamed reply is a sequence of JSON documents separated by NUL
bytes, each carrying every answer's text so far.
"""
import argparse
import json
import sys
from typing import Iterator, List

import requests


def post(url: str, prompt: str, n: int, stream: bool) -> requests.Response:
    body = {"prompt": prompt, "stream": stream,
            "sampling_config": {"temperature": 0.7, "topk": 1, "topp": 0.0, "num_return_sequences": n,
                                "max_new_tokens": 128}}
    return requests.post(url, json=body, headers={"User-Agent": "ksana example client"}, stream=stream)


def streamed_texts(resp: requests.Response) -> Iterator[List[str]]:
    for chunk in resp.iter_lines(chunk_size=8192, decode_unicode=False, delimiter=b"\0"):
        if chunk:
            yield json.loads(chunk.decode("utf-8"))["texts"]


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--host", type=str, default="localhost")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("--n", type=int, default=1)
    p.add_argument("--prompt", type=str, default="San Francisco is a")
    p.add_argument("--stream", action="store_true")
    a = p.parse_args(argv)
    url = f"http://{a.host}:{a.port}/generate"
    print(f"Prompt: {a.prompt!r}\n", flush=True)
    resp = post(url, a.prompt, a.n, a.stream)
    if resp.status_code != 200:
        print(f"HTTP {resp.status_code}: {resp.text[:400]}", file=sys.stderr)
        return 1
    if a.stream:
        shown = 0
        for texts in streamed_texts(resp):
            if shown and sys.stdout.isatty():
                sys.stdout.write("\033[1A\x1b[2K" * shown)          # redraw the answers in place
            for i, t in enumerate(texts):
                print(f"Answer {i}: {t!r}", flush=True)
            shown = len(texts)
    else:
        for i, t in enumerate(resp.json()["texts"]):
            print(f"Answer {i}: {t!r}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
