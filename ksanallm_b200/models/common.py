"""The decoder implementation every dense / MoE architecture reuses, driven by ModelConfig flags
(pre/post norm, RMSNorm/LayerNorm, gated or plain MLP, RoPE variants / ALiBi / learned positions,
QKV bias, MoE blocks), mirroring the role of the reference's CommonModel
(src/ksana_llm/models/common/common_model.cpp:446-980) with a B200-first op sequence:

  norm(+residual, +FP8 quantise) -> fused QKV GEMM -> RoPE + paged KV append -> paged attention
  (prefill rows and decode rows in one buffer) -> o_proj GEMM with the residual add in its epilogue
  -> norm(+FP8 quantise) -> gate|up GEMM -> act*mul(+FP8 quantise) -> down GEMM (+residual epilogue)

Tensor parallelism: column-parallel QKV / gate-up / lm_head, row-parallel o_proj / down with the
reduction done by :mod:`ksanallm_b200.parallel.comm`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from ..config import ModelConfig
from ..ops import dispatch as ops
from ..ops import native
from ..ops import reference as ref
from ..ops.dispatch import LinearWeight
from ..utils import nvtx


@dataclass
class StepInput:
    """Device-side metadata of one engine step (built from a StepPlan)."""
    input_ids: torch.Tensor
    positions: torch.Tensor
    slots: torch.Tensor
    cu_q: torch.Tensor
    kv_lens: torch.Tensor
    block_table: torch.Tensor            # [num_seqs, max_blocks] int32
    num_multi: int = 0
    num_single: int = 0
    num_tokens: int = 0
    num_multi_tokens: int = 0
    max_q_len: int = 0
    max_kv_len: int = 0                  # host-side upper bound of kv_lens (split heuristics, no device sync)
    logits_rows: Optional[torch.Tensor] = None
    mrope_positions: Optional[torch.Tensor] = None      # [3, T]
    refit_positions: Optional[torch.Tensor] = None      # rows to overwrite with plugin embeddings
    refit_embeddings: Optional[torch.Tensor] = None     # [R, hidden] fp32
    decode_splits: int = 1
    decode_workspace: Optional[tuple] = None
    sample_k: int = 0                    # > 0: tensor-parallel ranks return merged per-shard top-k candidates, not logits
    want_hidden: bool = False            # keep final hidden states / post-norm states for /forward


@dataclass
class LogitCandidates:
    """What a tensor-parallel forward returns instead of whole logits rows when the step's sampling only needs the k
    largest logits of every row: each vocabulary shard's top k, gathered from all ranks. values [rows, tp * k] fp32,
    ids [rows, tp * k] int32 (token ids; padding columns carry -inf / 0x7fffffff)."""
    values: torch.Tensor
    ids: torch.Tensor


@dataclass
class LayerWeights:
    input_norm: torch.Tensor
    input_norm_bias: Optional[torch.Tensor]
    qkv: LinearWeight
    o_proj: LinearWeight
    post_norm: torch.Tensor
    post_norm_bias: Optional[torch.Tensor]
    gate_up: Optional[LinearWeight] = None       # dense MLP (gate rows then up rows) or plain fc1
    down: Optional[LinearWeight] = None
    moe: Optional[object] = None                 # models.moe.MoEWeights
    attn_extra: Optional[dict] = None            # MLA projections


def alibi_slopes(num_heads: int) -> torch.Tensor:
    """ALiBi head slopes (3rdparty/LLM_kernels/csrc/kernels/nvidia/alibi/alibi.cu:10-30)."""
    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]
    if math.log2(num_heads).is_integer():
        s = pow2(num_heads)
    else:
        c = 2 ** math.floor(math.log2(num_heads))
        s = pow2(c) + pow2(2 * c)[0::2][: num_heads - c]
    return torch.tensor(s, dtype=torch.float32)


class CommonModel:
    def __init__(self, cfg: ModelConfig, tp_rank: int = 0, tp_size: int = 1, comm=None, device="cpu",
                 dtype=torch.bfloat16, layer_range: Optional[tuple] = None, kv_cache_dtype=None,
                 max_positions: Optional[int] = None):
        self.cfg = cfg
        self.tp_rank, self.tp_size, self.comm = tp_rank, tp_size, comm
        self.device, self.dtype = torch.device(device), dtype
        self.layer_lo, self.layer_hi = layer_range if layer_range else (0, cfg.num_layers - 1)
        self.is_first_stage = self.layer_lo == 0
        self.is_last_stage = self.layer_hi == cfg.num_layers - 1
        self.Hq = cfg.num_heads // tp_size
        self.Hkv = max(1, cfg.num_kv_heads // tp_size)
        self.D = cfg.head_dim
        self.rot_dim = cfg.rotary_dim or cfg.head_dim
        self.scale = 1.0 / math.sqrt(self.D)
        self.layers: List[LayerWeights] = []
        self.embed: Optional[torch.Tensor] = None
        self.pos_embed: Optional[torch.Tensor] = None
        self.final_norm: Optional[torch.Tensor] = None
        self.final_norm_bias: Optional[torch.Tensor] = None
        self.lm_head: Optional[LinearWeight] = None
        self.kv_cache: Optional[torch.Tensor] = None
        self.block_tokens = 16
        self.kv_scales = cfg.kv_scales
        self.alibi = None
        if cfg.position_embedding == "alibi":
            self.alibi = alibi_slopes(cfg.num_heads)[tp_rank * self.Hq:(tp_rank + 1) * self.Hq].to(self.device)
        self.cos_sin = None
        if cfg.position_embedding in ("rope", "mrope"):
            n = max_positions or cfg.max_token_len
            self.cos_sin = ref.build_cos_sin_cache(self.rot_dim, n, cfg.rope_theta, cfg.rope_scaling, self.device)
        self.dp = None                       # parallel.data_parallel.AttentionDP when attention runs data parallel
        self.step_hidden: Optional[torch.Tensor] = None
        self.step_normed: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ KV cache
    def allocate_kv_cache(self, num_blocks: int, block_tokens: int, dtype=None):
        """[blocks, layers_on_rank, 2, kv_heads_on_rank, block_tokens, head_dim]: one block id names the
        K and V tiles of every layer, tiles are contiguous [tokens, head_dim] panels."""
        self.block_tokens = block_tokens
        nl = self.layer_hi - self.layer_lo + 1
        dt = dtype or self.dtype
        self.kv_cache = torch.zeros(num_blocks, nl, 2, self.Hkv, block_tokens, self.D, dtype=dt, device=self.device)
        return self.kv_cache

    def block_bytes(self) -> int:
        return self.kv_cache[0].numel() * self.kv_cache.element_size()

    def _kv_scale(self, layer: int):
        if self.kv_scales is None or self.kv_cache is None or self.kv_cache.dtype in (torch.bfloat16, torch.float16, torch.float32):
            return 1.0, 1.0
        return float(self.kv_scales[layer][0]), float(self.kv_scales[layer][1])

    # ------------------------------------------------------------------ blocks
    def embed_tokens(self, step: StepInput) -> torch.Tensor:
        cfg = self.cfg
        if self.embed.device.type != self.device.type:
            # embed_tokens_use_cpu: the table stays in (pinned) host memory, rows are looked up there and only the
            # step's rows travel to the device (src/ksana_llm/layers/cpu/emb_lookup_layer.cpp in the reference)
            ids = step.input_ids.to("cpu").long()
            h = (self.embed[ids].float() * cfg.emb_scale).to(self.dtype) if cfg.emb_scale != 1.0 else self.embed[ids]
            if self.pos_embed is not None:
                h = h + self.pos_embed.to("cpu")[step.positions.to("cpu").long()]
            h = h.to(self.device, non_blocking=True)
            if step.refit_positions is not None and step.refit_positions.numel() > 0:
                h[step.refit_positions.long()] = step.refit_embeddings.to(h.dtype)
            return h
        V = self.embed.shape[0]
        lo = self.tp_rank * V if self.embed_sharded else 0
        h = ops.embedding(step.input_ids, self.embed, vocab_lo=lo, vocab_hi=lo + V,
                          positions=step.positions if self.pos_embed is not None else None,
                          pos_table=self.pos_embed, scale=cfg.emb_scale)
        if self.embed_sharded and self.tp_size > 1:
            h = self.comm.all_reduce(h)
        if step.refit_positions is not None and step.refit_positions.numel() > 0:
            if h.is_cuda:
                ops.native.refit_rows(h, step.refit_positions, step.refit_embeddings)
            else:
                h[step.refit_positions.long()] = step.refit_embeddings.to(h.dtype)
        return h

    def attention(self, li: int, lw: LayerWeights, x, step: StepInput) -> torch.Tensor:
        cfg = self.cfg
        qkv = ops.linear(x, lw.qkv)
        cache_layer = self.kv_cache[:, li - self.layer_lo]
        ks, vs = self._kv_scale(li)
        use_rope = cfg.position_embedding in ("rope", "mrope")
        pos = step.mrope_positions if (cfg.position_embedding == "mrope" and step.mrope_positions is not None) else step.positions
        sections = cfg.mrope_section if (cfg.position_embedding == "mrope" and step.mrope_positions is not None) else None
        ops.rope_kv_append(qkv, pos, step.slots, self.cos_sin if use_rope else _dummy_cs(qkv), cache_layer,
                           self.block_tokens, self.Hq, self.Hkv, self.D, self.rot_dim, cfg.rope_neox, sections, ks, vs,
                           apply_rope=use_rope)
        # pure decode steps hand the o_proj GEMM its FP8 operand straight from the attention kernels
        return ops.paged_attention(qkv, None, cache_layer, self.block_tokens, step.block_table, step.cu_q, step.kv_lens,
                                   step.num_multi, step.num_single, step.num_multi_tokens, step.max_q_len, self.Hq,
                                   self.Hkv, self.D, self.scale, self.alibi, ks, vs, step.decode_splits,
                                   step.decode_workspace, quant_for=lw.o_proj)

    def row_parallel(self, x, W: LinearWeight, h: torch.Tensor) -> torch.Tensor:
        """h += x W^T, reduced over the tensor-parallel group. Single rank: the add is the GEMM's epilogue."""
        if self.tp_size == 1:
            return ops.linear(x, W, residual=h, out=h)
        return self.comm.row_parallel_linear(x, W, h)

    def mlp(self, lw: LayerWeights, x, h: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        gu = ops.linear(x, lw.gate_up)
        a = ops.act_mul(gu, cfg.activation, cfg.gated_mlp, quant_for=lw.down)
        return self.row_parallel(a, lw.down, h)

    def layer_forward(self, li: int, lw: LayerWeights, h: torch.Tensor, step: StepInput) -> torch.Tensor:
        cfg = self.cfg
        ln = cfg.norm_type == "layernorm"
        if cfg.post_norm:
            # h = norm(h + attn(h)); h = norm(h + mlp(h))   (GPT-1 / fairseq without pre-normalisation)
            a = self.attention(li, lw, h, step)
            h = self.row_parallel(a, lw.o_proj, h)
            h = ops.norm(h, lw.input_norm, cfg.rms_norm_eps, beta=lw.input_norm_bias, layernorm=ln)
            h = self.mlp(lw, h, h)
            return ops.norm(h, lw.post_norm, cfg.rms_norm_eps, beta=lw.post_norm_bias, layernorm=ln)
        x = ops.norm(h, lw.input_norm, cfg.rms_norm_eps, beta=lw.input_norm_bias, layernorm=ln, quant_for=lw.qkv)
        with nvtx.annotate("attention"):
            a = self.attention(li, lw, x, step)
        with nvtx.annotate("o_proj"):
            h = self.row_parallel(a, lw.o_proj, h)
        if lw.moe is not None:
            from .moe import moe_forward
            x = ops.norm(h, lw.post_norm, cfg.rms_norm_eps, beta=lw.post_norm_bias, layernorm=ln)
            return moe_forward(self, lw.moe, x, h)
        x = ops.norm(h, lw.post_norm, cfg.rms_norm_eps, beta=lw.post_norm_bias, layernorm=ln, quant_for=lw.gate_up)
        with nvtx.annotate("mlp"):
            return self.mlp(lw, x, h)

    def _final_norm(self, h: torch.Tensor) -> torch.Tensor:
        if self.final_norm is None:
            return h
        return ops.norm(h, self.final_norm, self.cfg.rms_norm_eps, beta=self.final_norm_bias,
                        layernorm=self.cfg.norm_type == "layernorm")

    def compute_logits(self, normed: torch.Tensor) -> torch.Tensor:
        """Vocab-sharded lm_head GEMM with fp32 output, shards gathered across the TP group."""
        logits = ops.linear(normed, self.lm_head, out_f32=True)
        if self.tp_size > 1:
            logits = self.comm.all_gather_last_dim(logits, valid=self.vocab_shard)
        return logits[:, : self.cfg.vocab_size] if logits.shape[1] != self.cfg.vocab_size else logits

    def compute_candidates(self, normed: torch.Tensor, k: int):
        """Vocabulary-sharded sampling: the lm_head shard's logits stay on this rank; only each row's k largest
        (value, token id) pairs cross NVLink, k x 8 bytes per row and rank instead of the row's whole fp32 shard
        (the reference gathers the shards in full: src/ksana_llm/models/common/common_model.cpp:905-980). Every
        sampling choice the engine offers - greedy, top-k, top-p within the top k, top-N log-probs - depends on the
        k largest logits only, and the global top k is contained in the union of the shards' top k, so the merged
        lists give exactly the tokens the full rows would. Returns None when the lists do not fit the exchange area."""
        symm = getattr(self.comm, "symm", None) if self.comm is not None else None
        B = normed.shape[0]
        stage = symm.candidate_stage(B, k) if (symm is not None and normed.is_cuda) else None
        if stage is None:
            return None
        logits = ops.linear(normed, self.lm_head, out_f32=True)
        lo = self.tp_rank * self.vocab_shard
        valid = max(0, min(self.vocab_shard, self.cfg.vocab_size - lo))
        ops.native.shard_topk(logits, valid, k, lo, stage[0], stage[1])
        vals, ids = symm.gather_candidates(B, k)
        return LogitCandidates(vals, ids)

    def logits_or_candidates(self, hn: torch.Tensor, step: StepInput):
        if step.sample_k > 0 and self.tp_size > 1:
            cand = self.compute_candidates(hn, step.sample_k)
            if cand is not None:
                return cand
        return self.compute_logits(hn)

    def lm_head_forward(self, h: torch.Tensor, step: StepInput) -> torch.Tensor:
        """final norm -> rows that need logits -> lm_head. With ``want_hidden`` the hidden states of every
        row (before and after the final norm) are kept for /forward request targets."""
        rows = step.logits_rows
        if step.want_hidden:
            self.step_hidden = h
            self.step_normed = self._final_norm(h)
            hn = ops.gather_rows(self.step_normed, rows) if rows is not None else self.step_normed
        else:
            if rows is not None:
                h = ops.gather_rows(h, rows)
            hn = self._final_norm(h)
        return self.logits_or_candidates(hn, step)

    def rerotate_blocks(self, triples) -> None:
        """Flexible-cache copies land at another position: rotate the copied K by the position delta
        (RoPE rotations add), every layer and KV head of the destination blocks. One kernel on the GPU
        (``ksana_rerotate_blocks``); plain tensor ops elsewhere."""
        if self.cos_sin is None:
            return
        kv = self.kv_cache
        if (kv.is_cuda and native.available() and kv.dim() == 6 and self.cos_sin.dtype == torch.float32 and
                kv.dtype in (torch.bfloat16, torch.float8_e4m3fn)):
            t3 = torch.as_tensor(np.ascontiguousarray(triples, dtype=np.int32)).to(kv.device, non_blocking=False)
            native.rerotate_blocks(kv, t3, self.cos_sin, self.rot_dim, self.cfg.rope_neox)
            return
        half = self.rot_dim // 2
        for src, dst, delta in triples:
            delta = int(delta)
            if delta == 0:
                continue
            cs = self.cos_sin[abs(delta)]
            cos, sin = cs[:half], cs[half:] * (1.0 if delta > 0 else -1.0)
            k = self.kv_cache[int(dst), :, 0].float()                  # [layers, Hkv, bt, D]
            rot = k[..., : self.rot_dim]
            if self.cfg.rope_neox:
                x0, x1 = rot[..., :half], rot[..., half:]
                r = torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1)
            else:
                x0, x1 = rot[..., 0::2], rot[..., 1::2]
                r = torch.stack([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1).flatten(-2)
            k[..., : self.rot_dim] = r
            self.kv_cache[int(dst), :, 0] = k.to(self.kv_cache.dtype)

    def forward_empty_dp(self) -> None:
        """Attention data parallelism, a step in which this rank owns no rows: it still takes part in the dispatch /
        combine collectives of every MoE block (its experts may be needed by the other ranks' rows)."""
        x = torch.zeros(0, self.cfg.hidden_size, dtype=self.dtype, device=self.device)
        for lw in self.layers:
            if lw.moe is not None:
                self.dp.moe(self, lw.moe, x, x)

    def forward_layers(self, step: StepInput, hidden_in: Optional[torch.Tensor] = None) -> torch.Tensor:
        """This stage's layers only (embedding on the first stage): the hidden states to hand to the next
        pipeline stage, or to ``lm_head_forward`` on the last one."""
        h = self.embed_tokens(step) if self.is_first_stage else hidden_in
        for i, lw in enumerate(self.layers):
            h = self.layer_forward(self.layer_lo + i, lw, h, step)
        return h

    def forward(self, step: StepInput, hidden_in: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs this pipeline stage. The last stage returns fp32 logits [rows, vocab]; earlier stages return
        the hidden states to ship to the next stage."""
        h = self.embed_tokens(step) if self.is_first_stage else hidden_in
        if self._tp_fused_ok(h):
            return self._forward_tp_fused(h, step)
        for i, lw in enumerate(self.layers):
            h = self.layer_forward(self.layer_lo + i, lw, h, step)
        if not self.is_last_stage:
            return h
        return self.lm_head_forward(h, step)

    # ------------------------------------------------------------------ fused tensor-parallel path
    def _tp_fused_ok(self, h) -> bool:
        symm = getattr(self.comm, "symm", None) if self.comm is not None else None
        return (symm is not None and h.is_cuda and not self.cfg.post_norm and self.is_last_stage
                and self.is_first_stage and h.shape[0] <= symm.max_tokens and h.shape[1] == symm.hidden)

    def _forward_tp_fused(self, h0: torch.Tensor, step: StepInput) -> torch.Tensor:
        """Row-parallel GEMMs push their partial tiles into peer memory from the epilogue; one kernel then
        reduces, adds the residual and applies the following norm (and FP8 quantisation), so a layer has
        no stand-alone all-reduce, add or norm launches."""
        cfg, symm = self.cfg, self.comm.symm
        ln = cfg.norm_type == "layernorm"
        symm.begin_forward()
        T = h0.shape[0]
        if not symm.one_shot(T):
            h = symm.h[:T]
            h.copy_(h0)
        else:
            h = h0
        first = self.layers[0]
        x = ops.norm(h, first.input_norm, cfg.rms_norm_eps, beta=first.input_norm_bias, layernorm=ln, quant_for=first.qkv)
        n = len(self.layers)
        for i, lw in enumerate(self.layers):
            with nvtx.annotate("attention"):
                a = self.attention(self.layer_lo + i, lw, x, step)
            with nvtx.annotate("o_proj+reduce+norm"):
                h, x = symm.row_parallel_norm(a, lw.o_proj, h, lw.post_norm, lw.post_norm_bias, cfg.rms_norm_eps, ln,
                                              quant_for=lw.gate_up if lw.moe is None else None)
            if i + 1 < n:
                nw, nb, nq = self.layers[i + 1].input_norm, self.layers[i + 1].input_norm_bias, self.layers[i + 1].qkv
            else:
                nw, nb, nq = self.final_norm, self.final_norm_bias, None
            last_h = step.want_hidden and i + 1 == n
            if lw.moe is not None:
                # expert (or expert-slice) outputs of this rank are combined into the peer-visible slot; the
                # cross-rank sum, the residual add and the next norm are the same reduce kernel as for a GEMM
                from .moe import moe_partial
                h, x = symm.partial_norm(lambda part, _m=lw.moe, _x=x: moe_partial(self, _m, _x, into=part), T, h, nw, nb,
                                         cfg.rms_norm_eps, ln, quant_for=nq, gather_h=last_h)
                continue
            with nvtx.annotate("gate_up+act"):
                gu = ops.linear(x, lw.gate_up)
                act = ops.act_mul(gu, cfg.activation, cfg.gated_mlp, quant_for=lw.down)
            with nvtx.annotate("down+reduce+norm"):
                h, x = symm.row_parallel_norm(act, lw.down, h, nw, nb, cfg.rms_norm_eps, ln, quant_for=nq,
                                              gather_h=last_h)
        if step.want_hidden:
            self.step_hidden, self.step_normed = h, x
        hn = ops.gather_rows(x, step.logits_rows) if step.logits_rows is not None else x
        return self.logits_or_candidates(hn, step)

    # ------------------------------------------------------------------ misc
    embed_sharded = False
    vocab_shard = 0

    def weight_bytes(self) -> int:
        n = 0
        for lw in self.layers:
            for w in (lw.qkv, lw.o_proj, lw.gate_up, lw.down):
                if w is not None:
                    n += w.nbytes()
            if lw.moe is not None:
                n += lw.moe.nbytes()
        for t in (self.embed, self.final_norm):
            if t is not None:
                n += t.numel() * t.element_size()
        if self.lm_head is not None:
            n += self.lm_head.nbytes()
        return n


_DUMMY = {}


def _dummy_cs(x):
    key = str(x.device)
    if key not in _DUMMY:
        _DUMMY[key] = torch.zeros(2, dtype=torch.float32, device=x.device)
    return _DUMMY[key]
