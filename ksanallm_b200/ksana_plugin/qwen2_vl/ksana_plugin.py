"""Vision plug-in in the style of Qwen2-VL: images in the request's ``additional_params["images"]`` (float tensors
[3, H, W] or [frames, 3, H, W]) go through a vision tower; its merged patch embeddings replace the image pad
tokens of the prompt (``input_refit_embedding``) and the 3-axis rotary positions (temporal, height, width) are
handed to the engine as ``additional_tensors["mrope_positions"]``.

Role of the reference's ksana_plugin/qwen2_vl/ksana_plugin.py (vision tower through Torch or TensorRT producing
``input_refit_embedding`` plus mrope positions consumed by src/ksana_llm/models/qwen2_vl/qwen2_vl_model.cpp:22-110).
The tower here is a plain PyTorch ViT with the structure and parameter names of the checkpoints (temporal-pair
patch embedding, pre-norm blocks with 2-D rotary attention and quick-GELU MLPs, a 2x2 patch merger); weights come
from the ``visual.*`` tensors of the checkpoint when present, otherwise they are random (tests).
TensorRT engines are not used.
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


class _Attn(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.qkv, self.proj = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)


class _Mlp(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(dim, hidden), nn.Linear(hidden, dim)


class VisionBlock(nn.Module):
    """Pre-norm block; parameter names follow the checkpoint (norm1, norm2, attn.qkv, attn.proj, mlp.fc1, mlp.fc2)."""

    def __init__(self, dim: int, heads: int, mlp_ratio: float = 4.0):
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(dim, eps=1e-6), nn.LayerNorm(dim, eps=1e-6)
        self.attn, self.mlp = _Attn(dim), _Mlp(dim, int(dim * mlp_ratio))
        self.heads = heads

    def forward(self, x, cos, sin, seg):
        """x [N, dim]; cos/sin [N, head_dim/2] (2-D rotary: row angles | column angles); seg [N] image/frame id
        (attention stays inside one temporal patch of one image)."""
        N, C = x.shape
        q, k, v = self.attn.qkv(self.norm1(x)).view(N, 3, self.heads, C // self.heads).unbind(1)

        def rot(t):
            d = t.shape[-1] // 2
            t0, t1 = t[..., :d], t[..., d:]
            return torch.cat([t0 * cos[:, None] - t1 * sin[:, None], t1 * cos[:, None] + t0 * sin[:, None]], -1)

        q, k = rot(q), rot(k)
        mask = seg[:, None] == seg[None, :]
        a = F.scaled_dot_product_attention(q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1), attn_mask=mask[None])
        x = x + self.attn.proj(a.transpose(0, 1).reshape(N, C))
        h = self.mlp.fc1(self.norm2(x))
        return x + self.mlp.fc2(h * torch.sigmoid(1.702 * h))            # quick GELU, as the checkpoints are trained


class _PatchEmbed(nn.Module):
    """The checkpoint stores a Conv3d kernel [dim, 3, temporal, patch, patch] whose stride equals its size: a matrix
    product over flattened patches."""

    def __init__(self, dim: int, patch: int, temporal: int):
        super().__init__()
        self.proj = nn.Conv3d(3, dim, kernel_size=(temporal, patch, patch), stride=(temporal, patch, patch), bias=False)

    def forward(self, flat):
        return flat.to(self.proj.weight.dtype) @ self.proj.weight.view(self.proj.weight.shape[0], -1).t()


class _Merger(nn.Module):
    def __init__(self, dim: int, merge: int, hidden_out: int):
        super().__init__()
        self.ln_q = nn.LayerNorm(dim, eps=1e-6)
        self.mlp = nn.Sequential(nn.Linear(dim * merge * merge, dim * merge * merge), nn.GELU(),
                                 nn.Linear(dim * merge * merge, hidden_out))
        self.group = dim * merge * merge

    def forward(self, x):
        return self.mlp(self.ln_q(x).view(-1, self.group))


class VisionTower(nn.Module):
    """Patches of ``temporal`` x ``patch`` x ``patch`` pixels -> ``depth`` blocks -> groups of ``merge`` x ``merge``
    patches merged into one embedding of the language model's hidden size. Module and parameter names, patch order
    and rotary layout are those of the Qwen2-VL checkpoints' ``visual.*`` tensors (checked against the Hugging Face
    implementation in tests/test_vision_plugin_cpu.py)."""

    def __init__(self, hidden_out: int, dim: int = 64, depth: int = 2, heads: int = 4, patch: int = 14, merge: int = 2,
                 temporal: int = 2, mlp_ratio: float = 4.0):
        super().__init__()
        self.patch, self.merge, self.dim, self.heads, self.temporal = patch, merge, dim, heads, temporal
        self.patch_embed = _PatchEmbed(dim, patch, temporal)
        self.blocks = nn.ModuleList([VisionBlock(dim, heads, mlp_ratio) for _ in range(depth)])
        self.merger = _Merger(dim, merge, hidden_out)

    def grid_of(self, image: torch.Tensor):
        f = image.shape[0] if image.dim() == 4 else 1
        H, W = image.shape[-2:]
        return (f + self.temporal - 1) // self.temporal, H // self.patch, W // self.patch

    def patchify(self, images: List[torch.Tensor]):
        """Flattened patches [N, 3 * temporal * patch * patch] in the checkpoint's order (temporal patch, merged row,
        merged column, then the merge window; inside a patch: channel, frame, row, column) and the grids
        [(temporal patches, rows, columns)]. A still image is its own second frame."""
        P, M, Tp = self.patch, self.merge, self.temporal
        flat, grids = [], []
        for img in images:
            img = img.float()
            if img.dim() == 3:
                img = img[None]
            if img.shape[0] % Tp:
                img = torch.cat([img, img[-1:].expand(Tp - img.shape[0] % Tp, -1, -1, -1)], 0)
            t, gh, gw = self.grid_of(img)
            if gh % M or gw % M or gh == 0 or gw == 0:
                raise ValueError(f"image size must be a multiple of {P * M} pixels in both directions")
            grids.append((t, gh, gw))
            x = img[:, :, : gh * P, : gw * P].reshape(t, Tp, 3, gh // M, M, P, gw // M, M, P)
            x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(t * gh * gw, 3 * Tp * P * P)
            flat.append(x)
        return torch.cat(flat), grids

    def forward_patches(self, flat: torch.Tensor, grids):
        """flat [N, 3 * temporal * patch * patch] as produced by ``patchify`` (or by the Hugging Face image
        processor), grids [(t, rows, cols)] -> merged embeddings [N / merge^2, hidden_out]."""
        M = self.merge
        dev = self.patch_embed.proj.weight.device
        rows, cols, seg = [], [], []
        sid = 0
        for t, gh, gw in grids:
            r = torch.arange(gh).view(gh // M, 1, M, 1).expand(gh // M, gw // M, M, M).reshape(-1)
            c = torch.arange(gw).view(1, gw // M, 1, M).expand(gh // M, gw // M, M, M).reshape(-1)
            rows.append(r.repeat(t))
            cols.append(c.repeat(t))
            for _ in range(t):
                seg.append(torch.full((gh * gw,), sid))
                sid += 1
        x = self.patch_embed(flat.to(dev))
        rows, cols, seg = torch.cat(rows).to(dev), torch.cat(cols).to(dev), torch.cat(seg).to(dev)
        hd = self.dim // self.heads
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, device=dev).float() / (hd // 2)))
        ang = torch.cat([rows[:, None].float() * inv, cols[:, None].float() * inv], -1)       # [N, hd/2]
        cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
        for blk in self.blocks:
            x = blk(x, cos, sin, seg)
        return self.merger(x)

    @torch.no_grad()
    def forward(self, images: List[torch.Tensor]):
        """Returns (embeddings [sum of merged patches, hidden_out], grids [(temporal patches, h, w) in patches])."""
        flat, grids = self.patchify(images)
        return self.forward_patches(flat, grids), grids


def mrope_positions(tokens: List[int], image_pad_id: int, grids, merge: int) -> torch.Tensor:
    """[3, T] (temporal, height, width) positions: text advances all three axes together; an image of (f, h, w)
    patches occupies f*(h/merge)*(w/merge) pad tokens whose positions are the grid coordinates offset by the running
    position; text after it continues from the largest position used."""
    T = len(tokens)
    pos = torch.zeros(3, T, dtype=torch.int32)
    nxt, i, g = 0, 0, 0
    while i < T:
        if tokens[i] == image_pad_id and g < len(grids):
            f, gh, gw = grids[g]
            h, w = gh // merge, gw // merge
            n = f * h * w
            t_idx = torch.arange(f).view(f, 1, 1).expand(f, h, w).reshape(-1)
            h_idx = torch.arange(h).view(1, h, 1).expand(f, h, w).reshape(-1)
            w_idx = torch.arange(w).view(1, 1, w).expand(f, h, w).reshape(-1)
            pos[:, i:i + n] = torch.stack([t_idx, h_idx, w_idx]).to(torch.int32) + nxt
            nxt += max(f, h, w)
            i += n
            g += 1
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    return pos


class KsanaPlugin:
    def init_plugin(self, **kwargs):
        model_path = kwargs.get("model_path") or ""
        cfg = {}
        p = os.path.join(model_path, "config.json")
        if os.path.isfile(p):
            with open(p, "r", encoding="utf-8") as f:
                cfg = json.load(f)
        vc = cfg.get("vision_config") or {}
        self.hidden = int(cfg.get("hidden_size", kwargs.get("hidden_size", 64)))
        self.image_pad_id = int(cfg.get("image_token_id", kwargs.get("image_token_id", 151655)))
        self.tower = VisionTower(self.hidden, dim=int(vc.get("embed_dim", 64)), depth=int(vc.get("depth", 2)),
                                 heads=int(vc.get("num_heads", 4)), patch=int(vc.get("patch_size", 14)),
                                 merge=int(vc.get("spatial_merge_size", 2)), temporal=int(vc.get("temporal_patch_size", 2)),
                                 mlp_ratio=float(vc.get("mlp_ratio", 4.0)))
        g = torch.Generator().manual_seed(0)
        with torch.no_grad():                                     # deterministic start; overwritten by visual.* weights
            for prm in self.tower.parameters():
                prm.copy_(torch.randn(prm.shape, generator=g) * 0.02 if prm.dim() > 1 else torch.zeros(prm.shape))
        for m in self.tower.modules():
            if isinstance(m, nn.LayerNorm):
                nn.init.ones_(m.weight)
        self._load_visual(model_path)
        self.tower.eval()
        if torch.cuda.is_available():
            self.tower.cuda()

    def _load_visual(self, model_path: str):
        files = sorted(glob.glob(os.path.join(model_path, "*.safetensors"))) if model_path else []
        if not files:
            return
        from safetensors import safe_open
        own = dict(self.tower.state_dict())
        for fpath in files:
            with safe_open(fpath, framework="pt") as sf:
                for k in sf.keys():
                    name = k.split("visual.", 1)[1] if "visual." in k else None     # "visual.x" or "model.visual.x"
                    if name in own and tuple(sf.get_slice(k).get_shape()) == tuple(own[name].shape):
                        own[name].copy_(sf.get_tensor(k))

    def preprocess(self, **kwargs):
        inp = kwargs["ksana_python_input"]
        params = kwargs.get("additional_params") or {}
        images = params.get("images")
        if params.get("pixel_values") is not None and params.get("image_grid_thw") is not None:
            # output of the Hugging Face image processor: flattened patches and their (t, h, w) grids
            grids = [tuple(int(v) for v in g) for g in torch.as_tensor(params["image_grid_thw"]).tolist()]
            with torch.no_grad():
                emb = self.tower.forward_patches(torch.as_tensor(params["pixel_values"]).float(), grids)
        elif images:
            emb, grids = self.tower([torch.as_tensor(im) for im in images])
        else:
            return
        tokens = list(inp["input_tokens"])
        per = [g[0] * (g[1] // self.tower.merge) * (g[2] // self.tower.merge) for g in grids]
        # a single pad token per image in the prompt stands for the whole image: expand it
        out_tokens, starts, gi = [], [], 0
        for t in tokens:
            if t == self.image_pad_id and gi < len(per):
                starts.append(len(out_tokens))
                out_tokens.extend([self.image_pad_id] * per[gi])
                gi += 1
            else:
                out_tokens.append(t)
        if gi != len(per):
            raise ValueError(f"{len(per)} images but {gi} image tokens in the prompt")
        inp["input_tokens"] = out_tokens
        pieces = torch.split(emb.float().cpu(), per)
        inp["input_refit_embedding"] = {"pos": starts, "embeddings": list(pieces)}
        inp.setdefault("additional_tensors", {})["mrope_positions"] = mrope_positions(out_tokens, self.image_pad_id, grids,
                                                                                       self.tower.merge)

    def postprocess(self, **kwargs):
        return None
