"""DeepSeek-V3 style model (MLA absorbed attention + sigmoid group-limited MoE + shared expert) through
the engine on CPU vs a plain, non-absorbed PyTorch restatement."""
import math

import torch

from ksanallm_b200.config import EngineConfig, ModelConfig
from ksanallm_b200.models.moe import route_reference
from ksanallm_b200.models.weights import RandomSource, build_model
from ksanallm_b200.runtime.engine import LLMEngine
from ksanallm_b200.utils import native_engine as ne


def ds_cfg():
    return ModelConfig(model_type="deepseek_v3", hidden_size=128, num_layers=3, num_heads=4, num_kv_heads=4, head_dim=48,
                       intermediate_size=256, vocab_size=500, rms_norm_eps=1e-6, rope_theta=10000.0, rope_neox=False,
                       max_position_embeddings=256, max_token_len=256, num_experts=8, num_experts_per_tok=2,
                       moe_intermediate_size=64, shared_expert_intermediate_size=64, num_shared_experts=1,
                       moe_scoring="sigmoid", routed_scaling_factor=2.5, n_group=4, topk_group=2, first_k_dense_replace=1,
                       q_lora_rank=32, kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32)


def rms(t, eps=1e-6):
    return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)


def rope_interleaved(t, pos, dim, theta=10000.0):
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2).float() / dim))
    ang = torch.outer(pos.float(), inv)
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = t[..., 0::2], t[..., 1::2]
    return torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2)


def plain_forward(cfg, src, tokens):
    g = lambda n, s: src.get(n, s).float()
    H, Hq = cfg.hidden_size, cfg.num_heads
    nope, rp, vd, lora = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
    T = len(tokens)
    pos = torch.arange(T)
    x = g("model.embed_tokens.weight", (cfg.vocab_size, H))[tokens]
    for l in range(cfg.num_layers):
        p = f"model.layers.{l}.self_attn."
        hn = rms(x)
        q = rms(hn @ g(p + "q_a_proj.weight", (cfg.q_lora_rank, H)).t()) @ g(p + "q_b_proj.weight", (Hq * (nope + rp), cfg.q_lora_rank)).t()
        q = q.view(T, Hq, nope + rp)
        kv = hn @ g(p + "kv_a_proj_with_mqa.weight", (lora + rp, H)).t()
        c_kv, k_pe = rms(kv[:, :lora]), kv[:, lora:].view(T, 1, rp)
        kvb = (c_kv @ g(p + "kv_b_proj.weight", (Hq * (nope + vd), lora)).t()).view(T, Hq, nope + vd)
        k = torch.cat([kvb[..., :nope], rope_interleaved(k_pe, pos, rp).expand(T, Hq, rp)], -1)
        qq = torch.cat([q[..., :nope], rope_interleaved(q[..., nope:], pos, rp)], -1)
        att = torch.einsum("qhd,khd->hqk", qq, k) / math.sqrt(nope + rp)
        att = att.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hqk,khd->qhd", att.softmax(-1), kvb[..., nope:]).reshape(T, Hq * vd)
        x = x + o @ g(p + "o_proj.weight", (H, Hq * vd)).t()
        hn = rms(x)
        lp = f"model.layers.{l}."
        if l < cfg.first_k_dense_replace:
            gate = hn @ g(lp + "mlp.gate_proj.weight", (cfg.intermediate_size, H)).t()
            up = hn @ g(lp + "mlp.up_proj.weight", (cfg.intermediate_size, H)).t()
            x = x + (torch.nn.functional.silu(gate) * up) @ g(lp + "mlp.down_proj.weight", (H, cfg.intermediate_size)).t()
        else:
            logits = hn @ g(lp + "mlp.gate.weight", (cfg.num_experts, H)).t()
            ids, w = route_reference(logits, cfg, torch.zeros(cfg.num_experts))
            out = torch.zeros_like(hn)
            I = cfg.moe_intermediate_size
            for t in range(T):
                for k in range(cfg.num_experts_per_tok):
                    e = int(ids[t, k])
                    ep = f"{lp}mlp.experts.{e}."
                    a = torch.nn.functional.silu(hn[t] @ g(ep + "gate_proj.weight", (I, H)).t()) * (hn[t] @ g(ep + "up_proj.weight", (I, H)).t())
                    out[t] += w[t, k] * (a @ g(ep + "down_proj.weight", (H, I)).t())
            sp = lp + "mlp.shared_expert."
            sI = cfg.shared_expert_intermediate_size
            sa = torch.nn.functional.silu(hn @ g(sp + "gate_proj.weight", (sI, H)).t()) * (hn @ g(sp + "up_proj.weight", (sI, H)).t())
            x = x + out + sa @ g(sp + "down_proj.weight", (H, sI)).t()
    return rms(x) @ g("lm_head.weight", (cfg.vocab_size, H)).t()


def test_deepseek_mla_moe_matches_plain():
    cfg, src = ds_cfg(), RandomSource(seed=2, std=0.08)
    model = build_model(cfg, src, device="cpu", dtype=torch.float32)
    assert model.layers[0].moe is None and model.layers[1].moe is not None
    assert model.kv_cache is None
    ec = EngineConfig()
    ec.batch_scheduler.max_token_len = 128
    ec.batch_scheduler.split_fuse_token_num = 16
    eng = LLMEngine(model, cfg, ec, num_blocks=64)
    assert model.kv_cache.shape[-1] == 64 + 16          # latent + rotary key per token
    s = ne.SamplingConfig()
    s.max_new_tokens, s.ignore_eos = 4, True
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (21, 7)]
    reqs = eng.generate(prompts, s)
    for r, p in zip(reqs, prompts):
        toks = list(p)
        for t in r.outputs[0].tokens:
            want = plain_forward(cfg, src, toks)[-1]
            assert int(want.argmax()) == t
            toks.append(t)
