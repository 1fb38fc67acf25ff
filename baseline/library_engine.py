"""Measuring stick for bench.py (``--impl baseline``): the same Llama-architecture offline batch run as the
reference's op sequence built only from library calls - per-tensor FP8 cuBLASLt GEMMs (``torch._scaled_mm``),
PyTorch SDPA attention over a contiguous KV cache, unfused norm / rotary / activation / residual ops, NCCL
all-reduce after o_proj and down_proj and an NCCL all-gather of the vocabulary shards
(src/ksana_llm/models/common/common_model.cpp:446-980, src/ksana_llm/layers/nvidia/fp8_matmul_layer.cpp:36-70,
nccl_all_reduce_sum_layer.cpp:23-31). None of this package's kernels, scheduler or engine is used here; it is not
a product path.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn


class _Fp8Linear:
    """y = x W^T with W stored e4m3 [N, K] and one fp32 scale (the reference's per-tensor FP8 mode); the activation is
    quantised per call with a scale from its own maximum."""

    def __init__(self, n, k, device, std=0.02):
        w = torch.empty(n, k, dtype=torch.bfloat16, device=device).normal_(0.0, std)
        self.scale = (w.abs().amax().float() / 448.0).reshape(())
        self.w = (w.float() / self.scale).to(FP8)
        del w

    def __call__(self, x):
        s = (x.abs().amax().float() / 448.0).clamp_min(1e-12).reshape(())
        xq = (x.float() / s).to(FP8)
        return torch._scaled_mm(xq, self.w.t(), scale_a=s, scale_b=self.scale, out_dtype=torch.bfloat16)


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope(x, cos, sin):
    """x [B, S, H, D], cos/sin [B, S, 1, D/2] (rotate-half form)."""
    d = x.shape[-1] // 2
    x0, x1 = x[..., :d].float(), x[..., d:].float()
    return torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], -1).to(x.dtype)


class LibraryLlama:
    def __init__(self, cfg, rank, world, device, max_batch, max_len):
        self.cfg, self.rank, self.world, self.device = cfg, rank, world, device
        H, D = cfg.hidden_size, cfg.head_dim
        self.Hq, self.Hkv = cfg.num_heads // world, max(1, cfg.num_kv_heads // world)
        inter = cfg.intermediate_size // world
        self.layers = []
        for _ in range(cfg.num_layers):
            self.layers.append({
                "ln1": torch.ones(H, dtype=torch.bfloat16, device=device), "ln2": torch.ones(H, dtype=torch.bfloat16, device=device),
                "qkv": _Fp8Linear((self.Hq + 2 * self.Hkv) * D, H, device), "o": _Fp8Linear(H, self.Hq * D, device),
                "gate_up": _Fp8Linear(2 * inter, H, device), "down": _Fp8Linear(H, inter, device)})
        self.inter = inter
        self.embed = torch.empty(cfg.vocab_size, H, dtype=torch.bfloat16, device=device).normal_(0.0, 0.02)
        self.norm = torch.ones(H, dtype=torch.bfloat16, device=device)
        vs = (cfg.vocab_size + world - 1) // world
        self.lm_head = torch.empty(vs, H, dtype=torch.bfloat16, device=device).normal_(0.0, 0.02)
        self.vs = vs
        self.k_cache = torch.zeros(cfg.num_layers, max_batch, self.Hkv, max_len, D, dtype=torch.bfloat16, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32, device=device) / D))
        ang = torch.outer(torch.arange(max_len, dtype=torch.float32, device=device), inv)
        self.cos, self.sin = ang.cos(), ang.sin()

    def _reduce(self, x):
        if self.world > 1:
            dist.all_reduce(x)
        return x

    def forward(self, tokens, b0, start):
        """tokens [B, S] of sequences b0..b0+B whose cache holds ``start`` tokens; returns logits [B, vocab] (fp32)
        of the last position."""
        cfg, D = self.cfg, self.cfg.head_dim
        B, S = tokens.shape
        h = self.embed[tokens]                                            # [B, S, H]
        cos = self.cos[start:start + S].view(1, S, 1, D // 2)
        sin = self.sin[start:start + S].view(1, S, 1, D // 2)
        for li, L in enumerate(self.layers):
            x = _rms(h, L["ln1"], cfg.rms_norm_eps)
            qkv = L["qkv"](x.view(B * S, -1)).view(B, S, self.Hq + 2 * self.Hkv, D)
            q = _rope(qkv[:, :, : self.Hq], cos, sin)
            k = _rope(qkv[:, :, self.Hq: self.Hq + self.Hkv], cos, sin)
            v = qkv[:, :, self.Hq + self.Hkv:]
            self.k_cache[li, b0:b0 + B, :, start:start + S] = k.transpose(1, 2)
            self.v_cache[li, b0:b0 + B, :, start:start + S] = v.transpose(1, 2)
            kc = self.k_cache[li, b0:b0 + B, :, : start + S]
            vc = self.v_cache[li, b0:b0 + B, :, : start + S]
            a = F.scaled_dot_product_attention(q.transpose(1, 2), kc, vc, is_causal=(start == 0 and S > 1), enable_gqa=True)
            a = a.transpose(1, 2).reshape(B * S, self.Hq * D)
            h = h + self._reduce(L["o"](a)).view(B, S, -1)
            x = _rms(h, L["ln2"], cfg.rms_norm_eps)
            gu = L["gate_up"](x.view(B * S, -1))
            act = F.silu(gu[:, : self.inter]) * gu[:, self.inter:]
            h = h + self._reduce(L["down"](act)).view(B, S, -1)
        last = _rms(h[:, -1], self.norm, cfg.rms_norm_eps)
        logits = (last @ self.lm_head.t()).float()
        if self.world > 1:
            parts = [torch.empty_like(logits) for _ in range(self.world)]
            dist.all_gather(parts, logits)
            logits = torch.cat(parts, -1)
        return logits[:, : cfg.vocab_size]

    @torch.inference_mode()
    def generate(self, prompts: torch.Tensor, out_len: int, prefill_batch: int = 8) -> torch.Tensor:
        """prompts [B, S] (device, int64): greedy continuation of ``out_len`` tokens; prefill in groups of sequences
        (the reference's max_step_tokens budget), then one decode step per token for the whole batch."""
        B, S = prompts.shape
        nxt = torch.empty(B, dtype=torch.int64, device=self.device)
        for b0 in range(0, B, prefill_batch):
            lg = self.forward(prompts[b0:b0 + prefill_batch], b0, 0)
            nxt[b0:b0 + prefill_batch] = lg.argmax(-1)
        out = [nxt.clone()]
        for t in range(1, out_len):
            lg = self.forward(nxt.view(B, 1), 0, S + t - 1)
            nxt = lg.argmax(-1)
            out.append(nxt.clone())
        return torch.stack(out, 1)
