"""Command-line client of ``/forward`` (counterpart of src/ksana_llm/python/serving_forward_client.py in the
reference): msgpack request with request targets, tensors decoded to numpy; prints shapes and, for a ``logits``
GATHER_TOKEN_ID target, the perplexity of the prompt.

  python serving_forward_client.py --port 8080 --prompt "Hello world" --target logits
  python serving_forward_client.py --port 8080 --input_tokens 1 5 9 --target layernorm --slice 0 2
"""
import argparse
import json

from ksanallm_b200.serving import clients


def args_config(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--host", type=str, default="localhost")
    p.add_argument("--port", type=int, default=8888)
    p.add_argument("--api", type=str, default="forward", help="path of the endpoint on the server")
    p.add_argument("--prompt", type=str, default="Hello, my name is")
    p.add_argument("--input_tokens", type=int, nargs="*", default=None)
    p.add_argument("--target", type=str, default="logits", choices=["logits", "layernorm", "transformer"])
    p.add_argument("--slice", type=int, nargs=2, action="append", default=None, help="[begin end] token range (inclusive)")
    p.add_argument("--token_id", type=int, nargs="*", default=None)
    p.add_argument("--reduce", type=str, default="GATHER_ALL", choices=["GATHER_ALL", "GATHER_TOKEN_ID"])
    return p.parse_args(argv)


def main(argv=None):
    a = args_config(argv)
    target = {"target_name": a.target, "token_reduce_mode": a.reduce}
    if a.slice:
        target["slice_pos"] = [list(s) for s in a.slice]
    if a.token_id:
        target["token_id"] = list(a.token_id)
    req = {"request_target": [target]}
    if a.input_tokens:
        req["input_tokens"] = list(a.input_tokens)
    else:
        req["prompt"] = a.prompt
    doc = clients.forward(f"http://{a.host}:{a.port}", [req], api=a.api)
    out = []
    for resp in doc.get("responses", []) or []:
        for t in resp["response"]:
            out.append({"target_name": t["target_name"], "shape": list(getattr(t["tensor"], "shape", []))})
    summary = {"responses": out}
    if a.target == "logits" and a.reduce == "GATHER_TOKEN_ID":
        summary["perplexity"] = clients.perplexity_from_forward(doc)
    print(json.dumps(summary, indent=1))
    return doc


if __name__ == "__main__":
    main()
