"""Clients of the two endpoints (counterparts of serving_generate_client.py / serving_forward_client.py /
examples/streaming_client.py of the reference): plain ``requests`` calls plus a streaming chunk reader."""
from __future__ import annotations

import json
from typing import Dict, Iterator, List, Optional

import msgpack
import numpy as np
import requests

from .request_packer import unpack_tensor


def generate(url: str, prompt: Optional[str] = None, input_tokens: Optional[List[int]] = None,
             sampling_config: Optional[dict] = None, stream: bool = False, **extra) -> dict:
    body = {"stream": stream, "sampling_config": sampling_config or {}}
    if prompt is not None:
        body["prompt"] = prompt
    if input_tokens is not None:
        body["input_tokens"] = input_tokens
    body.update(extra)
    r = requests.post(url.rstrip("/") + "/generate", json=body, stream=stream)
    if stream:
        return {"chunks": list(iter_stream(r))}
    return r.json()


def iter_stream(response) -> Iterator[dict]:
    """Chunks are JSON objects separated by a zero byte."""
    buf = b""
    for part in response.iter_content(chunk_size=8192):
        buf += part
        while b"\0" in buf:
            chunk, buf = buf.split(b"\0", 1)
            if chunk:
                yield json.loads(chunk.decode("utf-8"))


def forward(url: str, requests_list: List[dict], api: str = "forward") -> dict:
    """requests_list entries: {"input_tokens"|"prompt", "request_target": [{"target_name", "slice_pos"|"token_id",
    "token_reduce_mode"}]}. Tensors in the reply are decoded to numpy arrays."""
    r = requests.post(url.rstrip("/") + "/" + api.lstrip("/"), data=msgpack.packb({"requests": requests_list}, use_bin_type=True),
                      headers={"Content-Type": "application/x-msgpack"})
    doc = msgpack.unpackb(r.content, raw=False)
    for resp in doc.get("responses", []) or []:
        for t in resp["response"]:
            t["tensor"] = unpack_tensor(t["tensor"])
    return doc


def perplexity_from_forward(doc: dict) -> List[float]:
    """PPL per request from a ``logits`` GATHER_TOKEN_ID reply (probabilities of the next input token)."""
    out = []
    for resp in doc["responses"]:
        for t in resp["response"]:
            if t["target_name"] == "logits":
                p = np.clip(np.asarray(t["tensor"], dtype=np.float64), 1e-30, 1.0)
                out.append(float(np.exp(-np.log(p).mean())))
    return out
