"""Vision plug-in for first-generation Qwen-VL: every ``<img>path</img>`` span of the prompt (the tokenizer spells
the path as UTF-8 bytes in the token ids between the image start and end ids, padded to 256 positions with the pad id)
is replaced by the 256 embeddings the vision tower produces for that picture (``input_refit_embedding`` at the
position right after the start token).

Role of the reference's ksana_plugin/qwen_vl/ksana_plugin.py:62-87 (find the spans, run the ViT through Torch or
TensorRT, hand back positions and embeddings). The tower here is plain PyTorch with the structure and parameter names
of the checkpoint's ``transformer.visual.*`` tensors: a 14-pixel patch convolution, learned absolute positions
(bicubically resized to the patch grid), pre-norm blocks whose fused QKV projection is laid out per head, and a
resampler - 256 learned queries with fixed 2-D sine/cosine positions cross-attending to the patch features - followed
by a final norm and projection. TensorRT engines are not used.
"""
from __future__ import annotations

import glob
import json
import math
import os
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def resize_positions(pos: torch.Tensor, target: int) -> torch.Tensor:
    """[s*s, C] position table resized to [t*t, C] (t*t = target) by bicubic interpolation over the grid."""
    src = int(math.sqrt(pos.shape[0]))
    tgt = int(math.sqrt(target))
    if src == tgt:
        return pos
    grid = pos.float().reshape(1, src, src, -1).permute(0, 3, 1, 2)
    out = F.interpolate(grid, size=(tgt, tgt), mode="bicubic", align_corners=False)
    return out.permute(0, 2, 3, 1).flatten(0, 2).to(pos.dtype)


def sincos_2d(dim: int, grid: int) -> torch.Tensor:
    """[grid*grid, dim]: half of the channels encode one grid axis, half the other, each as sin | cos of
    position / 10000^(2i/d)."""
    def axis(d, p):
        omega = 1.0 / (10000.0 ** (torch.arange(d // 2, dtype=torch.float64) / (d / 2.0)))
        out = p.reshape(-1, 1).double() * omega[None]
        return torch.cat([out.sin(), out.cos()], 1)
    ys, xs = torch.meshgrid(torch.arange(grid), torch.arange(grid), indexing="ij")
    return torch.cat([axis(dim // 2, xs), axis(dim // 2, ys)], 1).float()


class _VisualAttention(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.in_proj, self.out_proj = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
        self.heads = heads

    def forward(self, x):                                     # x [B, N, dim]
        B, N, C = x.shape
        hd = C // self.heads
        q, k, v = self.in_proj(x).view(B, N, self.heads, 3 * hd).split(hd, -1)      # per head: q | k | v
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return self.out_proj(a.transpose(1, 2).reshape(B, N, C))


class _Block(nn.Module):
    def __init__(self, dim: int, heads: int, mlp_dim: int):
        super().__init__()
        self.ln_1, self.ln_2 = nn.LayerNorm(dim, eps=1e-6), nn.LayerNorm(dim, eps=1e-6)
        self.attn = _VisualAttention(dim, heads)
        self.mlp = nn.Sequential()
        self.mlp.add_module("c_fc", nn.Linear(dim, mlp_dim))
        self.mlp.add_module("gelu", nn.GELU())
        self.mlp.add_module("c_proj", nn.Linear(mlp_dim, dim))

    def forward(self, x):
        x = x + self.attn(self.ln_1(x))
        return x + self.mlp(self.ln_2(x))


class _Blocks(nn.Module):
    def __init__(self, dim, depth, heads, mlp_dim):
        super().__init__()
        self.resblocks = nn.ModuleList([_Block(dim, heads, mlp_dim) for _ in range(depth)])

    def forward(self, x):
        for b in self.resblocks:
            x = b(x)
        return x


class Resampler(nn.Module):
    """``queries`` learned vectors (plus fixed 2-D positions) attend to the patch features (plus the same positions
    resized to the patch grid): a fixed number of embeddings per picture whatever its patch count."""

    def __init__(self, queries: int, dim: int, heads: int, kv_dim: int):
        super().__init__()
        self.pos_embed = nn.Parameter(sincos_2d(dim, int(math.sqrt(queries))), requires_grad=False)
        self.query = nn.Parameter(torch.zeros(queries, dim))
        self.kv_proj = nn.Linear(kv_dim, dim, bias=False) if kv_dim != dim else nn.Identity()
        self.attn = nn.MultiheadAttention(dim, heads)
        self.ln_q, self.ln_kv = nn.LayerNorm(dim, eps=1e-6), nn.LayerNorm(dim, eps=1e-6)

    def forward(self, x):                                     # x [B, N, kv_dim]
        pos = resize_positions(self.pos_embed, x.shape[1])
        x = self.ln_kv(self.kv_proj(x)).permute(1, 0, 2)      # [N, B, dim]
        q = self.ln_q(self.query)[:, None].expand(-1, x.shape[1], -1)
        out = self.attn(q + self.pos_embed[:, None], x + pos[:, None], x)[0]
        return out.permute(1, 0, 2)


class VisionTower(nn.Module):
    def __init__(self, image_size: int = 448, patch: int = 14, width: int = 1664, depth: int = 48, heads: int = 16,
                 mlp_ratio: float = 4.9231, queries: int = 256, out_dim: int = 4096, trained_grid: int = 16):
        super().__init__()
        self.image_size, self.patch, self.queries = image_size, patch, queries
        self.conv1 = nn.Conv2d(3, width, kernel_size=patch, stride=patch, bias=False)
        self.positional_embedding = nn.Parameter(width ** -0.5 * torch.randn(trained_grid * trained_grid, width))
        self.ln_pre = nn.LayerNorm(width, eps=1e-6)
        self.transformer = _Blocks(width, depth, heads, int(width * mlp_ratio))
        self.attn_pool = Resampler(queries, out_dim, max(1, out_dim // 128), width)
        self.ln_post = nn.LayerNorm(out_dim, eps=1e-6)
        self.proj = nn.Parameter(out_dim ** -0.5 * torch.randn(out_dim, out_dim))

    def preprocess(self, image: torch.Tensor) -> torch.Tensor:
        """[3, H, W] in 0..1 -> [3, S, S]: bicubic resize to the tower's square input, CLIP normalisation."""
        img = F.interpolate(image[None].float(), size=(self.image_size, self.image_size), mode="bicubic", align_corners=False)[0]
        mean = torch.tensor(CLIP_MEAN).view(3, 1, 1)
        std = torch.tensor(CLIP_STD).view(3, 1, 1)
        return (img.clamp(0, 1) - mean) / std

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [B, 3, S, S] (normalised) -> [B, queries, out_dim]"""
        w = self.conv1.weight
        x = self.conv1(pixels.to(w.device, w.dtype))
        x = x.flatten(2).permute(0, 2, 1)                                      # [B, patches, width]
        x = x + resize_positions(self.positional_embedding, x.shape[1])
        x = self.transformer(self.ln_pre(x))
        x = self.ln_post(self.attn_pool(x))
        return x @ self.proj


def image_spans(tokens: List[int], start_id: int):
    """[(position after the start token, path)] for every <img>...</img> span: the ids between start (start_id) and
    end (start_id + 1) are the bytes of the path, padded with start_id + 2."""
    spans, i = [], 0
    while i < len(tokens):
        if tokens[i] == start_id:
            try:
                end = tokens.index(start_id + 1, i + 1)
            except ValueError:
                break
            body = tokens[i + 1:end]
            if start_id + 2 in body:
                body = body[: body.index(start_id + 2)]
            try:
                spans.append((i + 1, end - (i + 1), bytes(body).decode("utf-8")))
            except (ValueError, UnicodeDecodeError):
                spans.append((i + 1, end - (i + 1), ""))
            i = end
        i += 1
    return spans


def load_image(path: str) -> torch.Tensor:
    """[3, H, W] floats in 0..1 from a local file (PIL when present, else a raw ``.pt`` tensor file)."""
    if path.endswith(".pt"):
        return torch.load(path).float()
    from PIL import Image                                  # noqa: WPS433 (optional dependency)
    import numpy as np
    with Image.open(path) as im:
        arr = np.asarray(im.convert("RGB"), dtype=np.float32) / 255.0
    return torch.from_numpy(arr).permute(2, 0, 1)


class KsanaPlugin:
    def init_plugin(self, **kwargs):
        model_path = kwargs.get("model_path") or ""
        cfg = {}
        p = os.path.join(model_path, "config.json")
        if os.path.isfile(p):
            with open(p, "r", encoding="utf-8") as f:
                cfg = json.load(f)
        vc = dict(cfg.get("visual") or {})
        vc.update(kwargs.get("visual") or {})
        self.start_id = int(vc.get("image_start_id", 151857))
        self.tower = VisionTower(image_size=int(vc.get("image_size", 448)), patch=int(vc.get("patch_size", 14)),
                                 width=int(vc.get("width", 1664)), depth=int(vc.get("layers", 48)),
                                 heads=int(vc.get("heads", 16)), mlp_ratio=float(vc.get("mlp_ratio", 4.9231)),
                                 queries=int(vc.get("n_queries", 256)), out_dim=int(vc.get("output_dim", cfg.get("hidden_size", 4096))))
        self._load_visual(model_path)
        self.tower.eval()
        if torch.cuda.is_available():
            self.tower.cuda().half()

    def _load_visual(self, model_path: str):
        files = sorted(glob.glob(os.path.join(model_path, "*.safetensors"))) if model_path else []
        if not files:
            return
        from safetensors import safe_open
        own = dict(self.tower.state_dict())
        for fpath in files:
            with safe_open(fpath, framework="pt") as sf:
                for k in sf.keys():
                    name = k.split("visual.", 1)[1] if "visual." in k else None
                    if name in own and tuple(sf.get_slice(k).get_shape()) == tuple(own[name].shape):
                        own[name].copy_(sf.get_tensor(k))

    def preprocess(self, **kwargs):
        inp = kwargs["ksana_python_input"]
        params = kwargs.get("additional_params") or {}
        tokens = list(inp["input_tokens"])
        spans = image_spans(tokens, self.start_id)
        if not spans:
            return
        given = params.get("images")                          # tensors supplied with the request take the paths' place
        pixels = []
        for i, (_, _, path) in enumerate(spans):
            img = torch.as_tensor(given[i]) if given is not None and i < len(given) else load_image(path)
            pixels.append(self.tower.preprocess(img))
        emb = self.tower(torch.stack(pixels)).float().cpu()
        for (pos, room, _), e in zip(spans, emb):
            if room < e.shape[0]:
                raise ValueError(f"image span of {room} positions cannot take {e.shape[0]} embeddings")
        inp["input_refit_embedding"] = {"pos": [s[0] for s in spans], "embeddings": [e for e in emb]}

    def postprocess(self, **kwargs):
        return None
