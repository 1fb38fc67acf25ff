"""GGUF checkpoints (llama.cpp single-file format): parser, tensor source and a small writer for tests.

File layout: magic ``GGUF``, version (2 or 3), tensor count, metadata count; metadata key/value pairs; tensor
infos (name, dims with the innermost first, ggml type, offset); padding to ``general.alignment`` (default 32);
tensor data. Supported tensor types: F32, F16, BF16 and the block formats Q8_0 / Q4_0, which are dequantised
to fp32 on load (the engine re-quantises to its own FP8 format when asked to).

Llama-family GGUF files store q_proj / k_proj with the rotary halves of every head interleaved; the source
undoes that permutation so the rest of the loader sees Hugging Face layout. Same role as the reference's
loader and its name map (src/ksana_llm/utils/gguf_file_tensor_loader.cpp:60-393,
src/ksana_llm/python/weight_map/llama_gguf_weight_map.json, src/ksana_llm/models/llama/llama_weight.cpp:74-80).
"""
from __future__ import annotations

import json
import os
import re
import struct
from typing import Dict, List, Optional

import numpy as np
import torch

from ..config import ModelConfig

GGUF_MAGIC = 0x46554747
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0, GGML_BF16 = 0, 1, 2, 8, 30
_BLOCK = {GGML_Q4_0: (32, 18), GGML_Q8_0: (32, 34)}          # elements per block, bytes per block


class _Reader:
    def __init__(self, buf: memoryview):
        self.buf, self.pos = buf, 0

    def scalar(self, fmt: str):
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += struct.calcsize(fmt)
        return v

    def string(self) -> str:
        n = self.scalar("<Q")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vtype: int):
        if vtype in _SCALAR:
            return self.scalar(_SCALAR[vtype])
        if vtype == 8:
            return self.string()
        if vtype == 9:
            etype, n = self.scalar("<I"), self.scalar("<Q")
            return [self.value(etype) for _ in range(n)]
        raise ValueError(f"unknown GGUF metadata type {vtype}")


class GGUFFile:
    def __init__(self, path: str):
        self.path = path
        self.data = np.memmap(path, dtype=np.uint8, mode="r")
        r = _Reader(memoryview(self.data))
        if r.scalar("<I") != GGUF_MAGIC:
            raise ValueError(f"{path} is not a GGUF file")
        self.version = r.scalar("<I")
        if self.version not in (2, 3):
            raise ValueError(f"unsupported GGUF version {self.version}")
        n_tensors, n_kv = r.scalar("<Q"), r.scalar("<Q")
        self.meta: Dict[str, object] = {}
        for _ in range(n_kv):
            key = r.string()
            self.meta[key] = r.value(r.scalar("<I"))
        self.tensors: Dict[str, tuple] = {}
        for _ in range(n_tensors):
            name = r.string()
            nd = r.scalar("<I")
            dims = [r.scalar("<Q") for _ in range(nd)]
            gtype, off = r.scalar("<I"), r.scalar("<Q")
            self.tensors[name] = (tuple(reversed(dims)), gtype, off)       # dims stored innermost first
        align = int(self.meta.get("general.alignment", 32))
        self.data_start = (r.pos + align - 1) // align * align

    def names(self) -> List[str]:
        return list(self.tensors.keys())

    def get(self, name: str) -> torch.Tensor:
        shape, gtype, off = self.tensors[name]
        n = int(np.prod(shape)) if shape else 1
        start = self.data_start + off
        if gtype == GGML_F32:
            a = np.frombuffer(self.data, dtype="<f4", count=n, offset=start)
            return torch.from_numpy(a.copy()).reshape(shape)
        if gtype == GGML_F16:
            a = np.frombuffer(self.data, dtype="<f2", count=n, offset=start)
            return torch.from_numpy(a.copy()).reshape(shape).float()
        if gtype == GGML_BF16:
            a = np.frombuffer(self.data, dtype="<i2", count=n, offset=start)
            return torch.from_numpy(a.copy()).view(torch.bfloat16).reshape(shape).float()
        if gtype in _BLOCK:
            per, nbytes = _BLOCK[gtype]
            blocks = np.frombuffer(self.data, dtype=np.uint8, count=n // per * nbytes, offset=start).reshape(-1, nbytes)
            d = torch.from_numpy(blocks[:, :2].copy().view("<f2").astype(np.float32))          # [nb, 1]
            if gtype == GGML_Q8_0:
                q = torch.from_numpy(blocks[:, 2:].copy().view(np.int8).astype(np.float32))
            else:                                                                                 # Q4_0: low nibbles first
                b = torch.from_numpy(blocks[:, 2:].copy())
                q = torch.cat([(b & 0xF).float(), (b >> 4).float()], dim=1) - 8.0
            return (q * d).reshape(shape)
        raise ValueError(f"tensor {name}: ggml type {gtype} is not supported")


def _unpermute_rope(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """Inverse of llama.cpp's q/k permutation: [n_head, 2, d/2, ...] swapped to [n_head, d/2, 2, ...] at export."""
    rows = w.shape[0]
    return w.reshape(n_head, rows // n_head // 2, 2, *w.shape[1:]).swapaxes(1, 2).reshape(w.shape)


def _permute_rope(w: torch.Tensor, n_head: int) -> torch.Tensor:
    rows = w.shape[0]
    return w.reshape(n_head, 2, rows // n_head // 2, *w.shape[1:]).swapaxes(1, 2).reshape(w.shape)


def _load_gguf_rules() -> List[tuple]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "weight_map", "llama_gguf_weight_map.json")
    with open(path) as f:
        return [(re.compile("^" + k + "$"), v) for k, v in json.load(f).items()]


class GGUFSource:
    """Weight source over one ``.gguf`` file, with canonical (Hugging Face) tensor names."""

    def __init__(self, path: str):
        self.file = GGUFFile(path)
        arch = str(self.file.meta.get("general.architecture", "llama"))
        self.n_head = int(self.file.meta.get(f"{arch}.attention.head_count", 0))
        self.n_kv = int(self.file.meta.get(f"{arch}.attention.head_count_kv", self.n_head))
        self.unpermute = arch in ("llama", "mistral", "baichuan")
        rules = _load_gguf_rules()
        self.index: Dict[str, str] = {}
        for raw in self.file.names():
            name = raw
            for rx, repl in rules:
                if rx.match(raw):
                    name = rx.sub(re.sub(r"\$(\d+)", r"\\\1", repl), raw)
                    break
            self.index[name] = raw

    def has(self, name: str) -> bool:
        return name in self.index

    def names(self):
        return list(self.index.keys())

    def get(self, name: str, shape=None, device="cpu", kind: str = "normal") -> torch.Tensor:
        t = self.file.get(self.index[name])
        if self.unpermute and self.n_head:
            if name.endswith("self_attn.q_proj.weight"):
                t = _unpermute_rope(t, self.n_head)
            elif name.endswith("self_attn.k_proj.weight"):
                t = _unpermute_rope(t, self.n_kv)
        return t


def model_config_from_gguf(meta: Dict[str, object]) -> ModelConfig:
    arch = str(meta.get("general.architecture", "llama"))
    g = lambda k, d=None: meta.get(f"{arch}.{k}", d)                     # noqa: E731
    hidden, heads = int(g("embedding_length")), int(g("attention.head_count"))
    vocab = g("vocab_size") or len(meta.get("tokenizer.ggml.tokens", [])) or 32000
    return ModelConfig(model_type="llama" if arch in ("llama", "mistral") else arch, hidden_size=hidden,
                       num_layers=int(g("block_count")), num_heads=heads,
                       num_kv_heads=int(g("attention.head_count_kv", heads)),
                       head_dim=int(g("attention.key_length", hidden // heads)),
                       intermediate_size=int(g("feed_forward_length")), vocab_size=int(vocab),
                       max_position_embeddings=int(g("context_length", 4096)),
                       rms_norm_eps=float(g("attention.layer_norm_rms_epsilon", 1e-5)),
                       rope_theta=float(g("rope.freq_base", 10000.0)))


# ------------------------------------------------------------------------------------- writer (tests, export)
def _w_string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _w_value(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<I", 7) + struct.pack("<?", v)
    if isinstance(v, int):
        return struct.pack("<I", 4) + struct.pack("<I", v)
    if isinstance(v, float):
        return struct.pack("<I", 6) + struct.pack("<f", v)
    if isinstance(v, str):
        return struct.pack("<I", 8) + _w_string(v)
    if isinstance(v, (list, tuple)):
        body = b"".join(_w_string(x) for x in v)
        return struct.pack("<I", 9) + struct.pack("<I", 8) + struct.pack("<Q", len(v)) + body
    raise TypeError(type(v))


def _encode_tensor(t: torch.Tensor, gtype: int) -> bytes:
    t = t.detach().float().contiguous()
    if gtype == GGML_F32:
        return t.numpy().astype("<f4").tobytes()
    if gtype == GGML_F16:
        return t.numpy().astype("<f2").tobytes()
    if gtype == GGML_BF16:
        return t.to(torch.bfloat16).view(torch.int16).numpy().tobytes()
    if gtype == GGML_Q8_0:
        blocks = t.reshape(-1, 32)
        d = blocks.abs().amax(dim=1, keepdim=True) / 127.0
        q = torch.where(d > 0, blocks / d.clamp_min(1e-30), torch.zeros_like(blocks)).round().clamp(-127, 127).to(torch.int8)
        out = np.empty((blocks.shape[0], 34), dtype=np.uint8)
        out[:, :2] = d.numpy().astype("<f2").view(np.uint8).reshape(-1, 2)
        out[:, 2:] = q.numpy().view(np.uint8)
        return out.tobytes()
    raise ValueError(f"cannot write ggml type {gtype}")


def write_gguf(path: str, meta: Dict[str, object], tensors: Dict[str, torch.Tensor], gtypes: Optional[Dict[str, int]] = None,
               alignment: int = 32) -> None:
    gtypes = gtypes or {}
    head = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(meta) + 1)
    kv = _w_string("general.alignment") + _w_value(alignment)
    for k, v in meta.items():
        kv += _w_string(k) + _w_value(v)
    infos, blobs, off = b"", [], 0
    for name, t in tensors.items():
        gt = gtypes.get(name, GGML_F32)
        blob = _encode_tensor(t, gt)
        dims = list(reversed(t.shape))
        infos += _w_string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", gt, off)
        pad = (-len(blob)) % alignment
        blobs.append(blob + b"\0" * pad)
        off += len(blob) + pad
    pre = head + kv + infos
    pre += b"\0" * ((-len(pre)) % alignment)
    with open(path, "wb") as f:
        f.write(pre)
        for b in blobs:
            f.write(b)
