"""msgpack wire format of the ``/forward`` endpoint.

Request:  {"requests": [{"prompt" | "input_tokens", "input_refit_embedding"?, "request_target": [
            {"target_name", "token_id"?, "slice_pos"?, "token_reduce_mode"?}]}]}
Response: {"responses": [{"input_token_ids": [...], "response": [{"target_name", "tensor":
            {"data": bytes, "shape": [...], "dtype": "float32"}}]}], "message": str, "code": int}
(src/ksana_llm/utils/request_serial.h:15-66, src/ksana_llm/utils/request_packer.cpp:1-124).
Decoding, validation and encoding run in the native runtime (csrc/engine/request_packer.cpp); this module maps the
decoded tree to engine requests and tensors to their wire form.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np
import torch

from ..utils import native_engine as ne

_DTYPES = {torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16", torch.int32: "int32"}


def unpack_requests(data: bytes, tokenizer=None) -> List[dict]:
    doc = ne.unpack_forward_body(bytes(data))          # native decode + validation (raises ValueError)
    out = []
    for r in doc.get("requests", []):
        tokens = r.get("input_tokens")
        if not tokens:
            prompt = r.get("prompt")
            if prompt is None or tokenizer is None:
                raise ValueError("request needs input_tokens (or a prompt and a tokenizer)")
            tokens = tokenizer.encode(prompt, add_special_tokens=True)
        targets: Dict[str, dict] = {}
        for t in r.get("request_target", []):
            targets[t["target_name"]] = {"token_id": list(t.get("token_id") or []),
                                         "slice_pos": [list(p) for p in (t.get("slice_pos") or [])],
                                         "token_reduce_mode": t.get("token_reduce_mode", "GATHER_ALL")}
        if not targets:
            raise ValueError("request_target is empty")
        out.append({"input_tokens": [int(x) for x in tokens], "request_target": targets,
                    "input_refit_embedding": r.get("input_refit_embedding")})
    if not out:
        raise ValueError("no requests")
    return out


def pack_tensor(t: torch.Tensor) -> dict:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        data = t.view(torch.int16).numpy().tobytes()
    else:
        data = t.numpy().tobytes()
    return {"data": data, "shape": list(t.shape), "dtype": _DTYPES.get(t.dtype, "float32")}


def pack_responses(items: List[Tuple[List[int], Dict[str, torch.Tensor]]], code: int = 0, message: str = "") -> bytes:
    responses = []
    for tokens, resp in items:
        responses.append({"input_token_ids": list(tokens),
                          "response": [{"target_name": k, "tensor": pack_tensor(v)} for k, v in resp.items()]})
    return ne.msgpack_pack({"responses": responses, "message": message, "code": code})


def unpack_tensor(d: dict) -> np.ndarray:
    dt = {"float32": np.float32, "float16": np.float16, "bfloat16": np.int16, "int32": np.int32}[d["dtype"]]
    arr = np.frombuffer(d["data"], dtype=dt).reshape(d["shape"])
    if d["dtype"] == "bfloat16":
        return torch.from_numpy(arr.copy()).view(torch.bfloat16).float().numpy()
    return arr
