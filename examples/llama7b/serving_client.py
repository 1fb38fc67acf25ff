"""Several prompts sent to a running server at once, answers printed as they complete.

    python serving_server.py --config_file examples/llama7b/ksana_llm.yaml --port 8888
    python examples/llama7b/serving_client.py --port 8888 [--stream] [--max_new_tokens 128]

Every prompt is one `/generate` request on its own thread (the server batches them continuously); with `--stream` the
text so far is reprinted whenever a new piece arrives (the server sends one JSON object per step, ended by a zero
byte). Same request body as the reference's example client (examples/llama7b/serving_client.py there): a prompt and a
`sampling_config`.
"""
import argparse
import json
import threading
import time

import requests

PROMPTS = [
    "Write a short poem about the sea.",
    "Explain in two sentences why the sky is blue.",
    "List three uses of a paper clip.",
    "Translate 'good morning' into French, Spanish and German.",
]


def one_request(url, prompt, args, results, i):
    body = {"prompt": prompt, "stream": args.stream,
            "sampling_config": {"temperature": args.temperature, "topk": args.topk, "topp": args.topp,
                                "max_new_tokens": args.max_new_tokens, "repetition_penalty": args.repetition_penalty}}
    t0 = time.time()
    try:
        with requests.post(url, json=body, stream=args.stream, timeout=args.timeout) as resp:
            if resp.status_code != 200:
                results[i] = (f"HTTP {resp.status_code}: {resp.text[:200]}", time.time() - t0)
                return
            if not args.stream:
                results[i] = ((resp.json().get("texts") or [""])[0], time.time() - t0)
                return
            buf, text = b"", ""
            for chunk in resp.iter_content(chunk_size=None):
                buf += chunk
                while b"\0" in buf:
                    piece, buf = buf.split(b"\0", 1)
                    if piece:
                        text = (json.loads(piece).get("texts") or [text])[0]
                        print(f"[{i}] {text!r}", flush=True)
            results[i] = (text, time.time() - t0)
    except Exception as e:  # noqa: BLE001 - a failed request is reported, the others go on
        results[i] = (f"request failed: {e!r}", time.time() - t0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8888)
    ap.add_argument("--stream", action="store_true")
    ap.add_argument("--max_new_tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--topk", type=int, default=1)
    ap.add_argument("--topp", type=float, default=0.0)
    ap.add_argument("--repetition_penalty", type=float, default=1.0)
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("--prompt", action="append", help="a prompt of your own (repeatable) instead of the built-in ones")
    args = ap.parse_args()
    prompts = args.prompt or PROMPTS
    url = f"http://{args.host}:{args.port}/generate"
    results = [None] * len(prompts)
    threads = [threading.Thread(target=one_request, args=(url, p, args, results, i)) for i, p in enumerate(prompts)]
    t0 = time.time()
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for p, (text, secs) in zip(prompts, results):
        print(f"--- {p}\n{text}\n({secs:.2f} s)")
    print(f"{len(prompts)} requests in {time.time() - t0:.2f} s")


if __name__ == "__main__":
    main()
