"""DeepSeek-V3 style decoder: multi-head latent attention (MLA) with the "absorbed" formulation and
MoE feed-forward blocks (sigmoid group-limited routing + shared experts; first layers dense).

The reference has no MLA / DeepSeek support; the oracle is the plain PyTorch statement in
``tests/test_deepseek_cpu.py``. Cache layout: one latent row per token and layer,
``[blocks, layers, block_tokens, kv_lora_rank + qk_rope_head_dim]`` (the compressed KV c_kv followed by the
shared rotary key), i.e. 576 values per token instead of 2 * heads * head_dim.

Absorbed attention (per head h):   q_lat[h] = q_nope[h] @ W_uk[h]            (128 -> 512)
                                   s = (q_lat[h] . c_kv + q_pe[h] . k_pe) * scale
                                   o_lat[h] = softmax(s) @ c_kv                (512)
                                   o[h] = o_lat[h] @ W_uv[h]^T                 (512 -> 128)
so attention is multi-query over a single 576/512-wide latent "head" shared by all query heads.
The projections run on the tcgen05 GEMMs. On a GPU with the DeepSeek-V2/V3 dimensions (latent 512, rotary 64)
the attention core is the tcgen05 latent-attention kernel (csrc/kernels/mla_attention.cu); other dimensions
and the CPU use batched PyTorch matmuls over the gathered latent rows of each sequence.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from ..config import ModelConfig
from ..ops import dispatch as ops
from ..ops import reference as ref
from ..ops.dispatch import LinearWeight
from .common import CommonModel, LayerWeights, StepInput


@dataclass
class MLAWeights:
    q_a: Optional[LinearWeight]          # [q_lora_rank, H]
    q_a_norm: Optional[torch.Tensor]
    q_b: LinearWeight                    # [Hq*(nope+rope), q_lora_rank or H]
    kv_a: LinearWeight                   # [kv_lora_rank + rope, H]
    kv_a_norm: torch.Tensor
    w_uk: torch.Tensor                   # [Hq, nope, kv_lora_rank]
    w_uv: torch.Tensor                   # [Hq, v_dim, kv_lora_rank]
    w_uk_t: Optional[torch.Tensor] = None    # [Hq, kv_lora_rank, nope]: W_uk as the K-major operand of the batched GEMM (built on first use)


def yarn_mscale(scale: float, mscale: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


class DeepseekModel(CommonModel):
    def __init__(self, cfg: ModelConfig, *a, **kw):
        super().__init__(cfg, *a, **kw)
        self.nope, self.rope, self.vdim, self.lora = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        self.scale = 1.0 / math.sqrt(self.nope + self.rope)
        rs = cfg.rope_scaling or {}
        if rs.get("mscale_all_dim"):
            m = yarn_mscale(float(rs.get("factor", 1.0)), float(rs["mscale_all_dim"]))
            self.scale *= m * m
        self.rot_dim = self.rope
        self.cos_sin = ref.build_cos_sin_cache(self.rope, self.cos_sin.shape[0] if self.cos_sin is not None else cfg.max_token_len,
                                               cfg.rope_theta, cfg.rope_scaling, self.device)

    def allocate_kv_cache(self, num_blocks: int, block_tokens: int, dtype=None):
        self.block_tokens = block_tokens
        nl = self.layer_hi - self.layer_lo + 1
        self.kv_cache = torch.zeros(num_blocks, nl, block_tokens, self.lora + self.rope, dtype=dtype or self.dtype,
                                    device=self.device)
        return self.kv_cache

    def attention(self, li: int, lw: LayerWeights, x, step: StepInput) -> torch.Tensor:
        mw: MLAWeights = lw.attn_extra["mla"]
        cfg, Hq = self.cfg, self.Hq
        T = x.q.shape[0] if isinstance(x, ops.QTensor) else x.shape[0]
        if mw.q_a is not None:
            qa = ops.linear(x, mw.q_a)
            qa = ops.norm(qa, mw.q_a_norm, cfg.rms_norm_eps, quant_for=mw.q_b)
            q = ops.linear(qa, mw.q_b)
        else:
            q = ops.linear(x, mw.q_b)
        kv = ops.linear(x, mw.kv_a)                               # [T, lora + rope]
        if q.is_cuda and self._mla_native_ok(q):
            return self._attention_native(li, mw, q, kv, step)
        q = q.view(T, Hq, self.nope + self.rope)
        c_kv = ops.norm(kv[:, : self.lora].contiguous(), mw.kv_a_norm, cfg.rms_norm_eps)
        k_pe = kv[:, self.lora:].reshape(T, 1, self.rope)
        q_pe = q[..., self.nope:]
        q_pe = ref.apply_rope(q_pe, step.positions, self.cos_sin, self.rope, neox=False)
        k_pe = ref.apply_rope(k_pe, step.positions, self.cos_sin, self.rope, neox=False).reshape(T, self.rope)
        # append the latent rows to the paged cache
        cache = self.kv_cache[:, li - self.layer_lo]               # [blocks, bt, lora+rope]
        ok = step.slots >= 0
        sl = step.slots[ok].long()
        cache[sl // self.block_tokens, sl % self.block_tokens] = torch.cat([c_kv, k_pe], -1)[ok].to(cache.dtype)
        # absorbed scores
        q_lat = torch.einsum("thn,hnl->thl", q[..., : self.nope].float(), mw.w_uk.float())   # [T, Hq, lora]
        out_lat = torch.zeros(T, Hq, self.lora, dtype=torch.float32, device=q.device)
        cu = step.cu_q.tolist()
        kvl = step.kv_lens.tolist()
        bt = self.block_tokens
        for s in range(len(kvl)):
            q0, q1, kl = cu[s], cu[s + 1], kvl[s]
            if q1 == q0:
                continue
            nblk = (kl + bt - 1) // bt
            rows = cache[step.block_table[s, :nblk].long()].reshape(nblk * bt, -1)[:kl].float()
            ckv, kpe = rows[:, : self.lora], rows[:, self.lora:]
            sc = (torch.einsum("qhl,kl->hqk", q_lat[q0:q1], ckv) +
                  torch.einsum("qhr,kr->hqk", q_pe[q0:q1].float(), kpe)) * self.scale
            qpos = torch.arange(kl - (q1 - q0), kl, device=q.device).unsqueeze(1)
            kpos = torch.arange(kl, device=q.device).unsqueeze(0)
            sc = sc.masked_fill(kpos > qpos, float("-inf"))
            out_lat[q0:q1] = torch.einsum("hqk,kl->qhl", torch.softmax(sc, -1), ckv)
        out = torch.einsum("thl,hvl->thv", out_lat, mw.w_uv.float())                       # [T, Hq, v]
        return out.reshape(T, Hq * self.vdim).to(q.dtype)


    # ------------------------------------------------------------------ tcgen05 latent attention (GPU)
    def _mla_native_ok(self, q) -> bool:
        Hq = self.Hq
        return (self.lora == 512 and self.rope == 64 and q.dtype == torch.bfloat16 and Hq <= 128 and Hq & (Hq - 1) == 0
                and self.kv_cache is not None and self.kv_cache.dtype == torch.bfloat16)

    def _attention_native(self, li, mw, q, kv, step):
        """Fused latent norm + rotations + cache append, q_nope W_uk as a batched GEMM into the packed query rows,
        the tcgen05 latent-attention kernel (prefill rows and decode rows in one launch), then W_uv."""
        from ..ops import native
        T, Hq = q.shape[0], self.Hq
        cache = self.kv_cache[:, li - self.layer_lo]                # [blocks, bt, 576]
        qfull = torch.empty(T, Hq, self.lora + self.rope, dtype=q.dtype, device=q.device)
        native.mla_rope_append(q, self.nope, kv, mw.kv_a_norm, self.cfg.rms_norm_eps, step.positions, step.slots,
                               self.cos_sin, qfull, cache, cache.stride(0), self.block_tokens, Hq)
        # absorbed query: per head q_nope W_uk straight into the packed query rows (one batched tcgen05 GEMM whose
        # operand and result views are head-interleaved: no transposes, no copy)
        q_nope = q.view(T, Hq, self.nope + self.rope)[..., : self.nope].transpose(0, 1)          # [Hq, T, nope]
        if mw.w_uk_t is None:
            mw.w_uk_t = mw.w_uk.transpose(1, 2).contiguous()                                      # [Hq, lora, nope]
        native.gemm_bf16_batched(q_nope, mw.w_uk_t, qfull[..., : self.lora].transpose(0, 1))
        o_lat = torch.empty(T, Hq, self.lora, dtype=q.dtype, device=q.device)
        B = step.num_multi + step.num_single
        nsplit = native.mla_splits(B, step.max_q_len, step.max_kv_len) if step.num_multi == 0 else 1
        if not native.mla_attention(qfull, o_lat, cache, cache.stride(0), self.block_tokens, step.block_table, step.cu_q,
                                    step.kv_lens, B, max(step.max_q_len, 1), Hq, self.scale, nsplit):
            raise RuntimeError("latent-attention kernel rejected a configuration that _mla_native_ok accepted")
        o = torch.empty(T, Hq, self.vdim, dtype=q.dtype, device=q.device)
        native.gemm_bf16_batched(o_lat.transpose(0, 1), mw.w_uv, o.transpose(0, 1))              # per head o_lat W_uv^T
        return o.view(T, Hq * self.vdim)


def build_deepseek(cfg: ModelConfig, source, tp_rank, tp_size, comm, device, dtype, quant, layer_range, max_positions):
    """MLA attention weights + dense / MoE feed-forward, canonical names as in the HF checkpoint
    (q_a_proj, q_a_layernorm, q_b_proj, kv_a_proj_with_mqa, kv_a_layernorm, kv_b_proj, o_proj)."""
    from .moe import load_moe
    from .weights import RandomSource, _cat0, _cols, _dense, _make_linear, _rows
    m = DeepseekModel(cfg, tp_rank, tp_size, comm, device, dtype, layer_range, max_positions=max_positions)
    H, Hq_all = cfg.hidden_size, cfg.num_heads
    nope, rope, vdim, lora = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
    Hq = Hq_all // tp_size

    def get(name, shape, kind="normal"):
        return source.get(name, shape, device=device, kind=kind)

    m.embed = get("model.embed_tokens.weight", (cfg.vocab_size, H)).to(device=device, dtype=dtype)
    for li in range(m.layer_lo, m.layer_hi + 1):
        p = f"model.layers.{li}.self_attn."
        if cfg.q_lora_rank:
            q_a = _make_linear(get(p + "q_a_proj.weight", (cfg.q_lora_rank, H)), None, device, dtype, quant)
            q_a_norm = get(p + "q_a_layernorm.weight", (cfg.q_lora_rank,), "ones").to(device=device, dtype=dtype)
            q_b_full = get(p + "q_b_proj.weight", (Hq_all * (nope + rope), cfg.q_lora_rank))
        else:
            q_a, q_a_norm = None, None
            q_b_full = get(p + "q_proj.weight", (Hq_all * (nope + rope), H))
        q_b = _make_linear(_rows(q_b_full, tp_rank, tp_size), None, device, dtype, quant)
        kv_a = _make_linear(get(p + "kv_a_proj_with_mqa.weight", (lora + rope, H)), None, device, dtype, quant)
        kv_a_norm = get(p + "kv_a_layernorm.weight", (lora,), "ones").to(device=device, dtype=dtype)
        kv_b = _dense(_rows(get(p + "kv_b_proj.weight", (Hq_all * (nope + vdim), lora)), tp_rank, tp_size)).to(device)
        kv_b = kv_b.float().view(Hq, nope + vdim, lora)
        mla = MLAWeights(q_a, q_a_norm, q_b, kv_a, kv_a_norm, kv_b[:, :nope].contiguous().to(dtype),
                         kv_b[:, nope:].contiguous().to(dtype))
        o_w = _cols(get(p + "o_proj.weight", (H, Hq_all * vdim)), tp_rank, tp_size)
        lp = f"model.layers.{li}."
        lw = LayerWeights(
            input_norm=get(lp + "input_layernorm.weight", (H,), "ones").to(device=device, dtype=dtype), input_norm_bias=None,
            qkv=kv_a, o_proj=_make_linear(o_w, None, device, dtype, quant),
            post_norm=get(lp + "post_attention_layernorm.weight", (H,), "ones").to(device=device, dtype=dtype),
            post_norm_bias=None, attn_extra={"mla": mla})
        if cfg.is_moe and li >= cfg.first_k_dense_replace and li % max(cfg.moe_layer_freq, 1) == 0:
            from .moe import ep_layout
            ep_rank, ep = ep_layout(cfg, tp_rank, tp_size)
            lw.moe = load_moe(cfg, source, lp, tp_rank, tp_size, device, dtype, quant, ep_rank=ep_rank, ep_size=ep)
        else:
            inter = cfg.intermediate_size
            g = _rows(get(lp + "mlp.gate_proj.weight", (inter, H)), tp_rank, tp_size)
            u = _rows(get(lp + "mlp.up_proj.weight", (inter, H)), tp_rank, tp_size)
            d = _cols(get(lp + "mlp.down_proj.weight", (H, inter)), tp_rank, tp_size)
            lw.gate_up = _make_linear(_cat0([g, u]), None, device, dtype, quant)
            lw.down = _make_linear(d, None, device, dtype, quant)
        m.layers.append(lw)
    m.final_norm = get("model.norm.weight", (H,), "ones").to(device=device, dtype=dtype)
    head = get("lm_head.weight", (cfg.vocab_size, H))
    vs = (cfg.vocab_size + tp_size - 1) // tp_size
    vs_pad = (vs + 7) // 8 * 8
    shard = head[tp_rank * vs:(tp_rank + 1) * vs]
    if shard.shape[0] < vs_pad:
        shard = torch.cat([shard, torch.zeros(vs_pad - shard.shape[0], H, dtype=shard.dtype, device=shard.device)], 0)
    m.lm_head = LinearWeight(w=shard.to(device=device, dtype=dtype).contiguous())
    m.vocab_shard = vs
    return m
