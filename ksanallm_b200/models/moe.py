"""Mixture-of-experts block: router -> top-k -> expert-major permutation -> grouped GEMM (gate|up) ->
act*mul -> grouped GEMM (down) -> top-k weighted combine (+ shared expert), then the tensor-parallel
reduction and the residual add.

Covers Mixtral (softmax top-2, renormalised), Qwen2-MoE (softmax top-k, optional renorm, shared expert
with a sigmoid gate) and DeepSeek-V3 (sigmoid scores, correction bias, group-limited top-8, scaling,
shared experts). Reference semantics: src/ksana_llm/models/common_moe/common_moe_model.cpp:35-63,
src/ksana_llm/models/qwen2_moe/qwen2_moe_model.cpp:57-130 and the routing kernels in
3rdparty/LLM_kernels/csrc/kernels/nvidia/mixture_of_experts/moe_kernels.cu:209-433,779 (renorm modes).
Experts are stacked [E, 2*inter/tp, hidden] and [E, hidden, inter/tp]
(src/ksana_llm/models/common_moe/common_moe_weight.cpp:31-104); ``expert_range`` restricts a rank to
its own experts for expert parallelism.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..config import ModelConfig
from ..ops import dispatch as ops
from ..ops import native, reference as ref
from ..ops.dispatch import LinearWeight


@dataclass
class MoEWeights:
    router: torch.Tensor                    # [E, H]
    router_bias: Optional[torch.Tensor]     # selection-only correction bias [E]
    w13: torch.Tensor                       # [E * 2I, H]  (gate rows then up rows per expert), bf16 or e4m3
    w13_scale: Optional[torch.Tensor]
    w2: torch.Tensor                        # [E * H, I]
    w2_scale: Optional[torch.Tensor]
    num_experts: int
    inter: int
    hidden: int
    shared_gate_up: Optional[LinearWeight] = None
    shared_down: Optional[LinearWeight] = None
    shared_gate: Optional[torch.Tensor] = None       # [1, H] sigmoid gate of the shared expert (Qwen2-MoE)
    expert_lo: int = 0
    expert_hi: int = 0
    # NVFP4 experts: w13 / w2 hold packed e2m1 pairs ([rows, K/2] bytes), *_bs the e4m3 scales per 16 elements
    # ([rows, K/16]) and *_ts one fp32 tensor scale per local expert
    w13_bs: Optional[torch.Tensor] = None
    w13_ts: Optional[torch.Tensor] = None
    w2_bs: Optional[torch.Tensor] = None
    w2_ts: Optional[torch.Tensor] = None

    @property
    def nvfp4(self) -> bool:
        return self.w13_bs is not None

    def nbytes(self) -> int:
        n = 0
        for t in (self.router, self.w13, self.w13_scale, self.w2, self.w2_scale, self.shared_gate, self.w13_bs,
                  self.w13_ts, self.w2_bs, self.w2_ts):
            if t is not None:
                n += t.numel() * t.element_size()
        for w in (self.shared_gate_up, self.shared_down):
            if w is not None:
                n += w.nbytes()
        return n


def _rows(t, rank, size):
    from .weights import _rows as rows          # FP8 checkpoint pairs are sliced with their block scales
    return rows(t, rank, size)


def _cols(t, rank, size):
    from .weights import _cols as cols
    return cols(t, rank, size)


def load_moe(cfg: ModelConfig, source, prefix: str, tp_rank, tp_size, device, dtype, quant, ep_rank=0, ep_size=1):
    """Expert parallelism (``ep_size`` > 1, over the tensor-parallel group whose ranks all hold every token):
    each rank keeps whole experts ``[lo, hi)`` (no intermediate-dimension slicing) and computes only their
    contributions; the block's all-reduce is the combine. The shared expert stays tensor-parallel."""
    from .weights import Fp8Pair, RandomSource, _cat0, _dense, _make_linear
    sh_rank, sh_size = tp_rank, tp_size
    if ep_size > 1:
        tp_rank, tp_size = 0, 1
    H, E, I_full = cfg.hidden_size, cfg.num_experts, cfg.moe_intermediate_size
    I = (I_full + tp_size - 1) // tp_size
    per = (E + ep_size - 1) // ep_size
    lo, hi = ep_rank * per, min(E, (ep_rank + 1) * per)
    rnd = isinstance(source, RandomSource)
    router = source.get(prefix + "mlp.gate.weight", (E, H), device=device).to(device=device, dtype=torch.float32)
    rbias = None
    if cfg.moe_scoring == "sigmoid":
        name = prefix + "mlp.gate.e_score_correction_bias"
        if rnd or source.has(name):
            rbias = source.get(name, (E,), device=device, kind="zeros").to(device=device, dtype=torch.float32)
    w13_parts, w2_parts = [], []
    fused_gu, fused_d = prefix + "mlp.experts.gate_up_proj", prefix + "mlp.experts.down_proj"
    fused = (not rnd) and source.has(fused_gu) and source.has(fused_d)
    if fused:
        # checkpoints that stack the experts: gate_up_proj [E, 2*I, H] (gate rows, then up rows), down_proj [E, H, I]
        gu_all, d_all = source.get(fused_gu, None, device=device), source.get(fused_d, None, device=device)
    for e in range(E):
        if not (lo <= e < hi):
            # experts owned by other expert-parallel ranks keep a zero-size placeholder row range
            continue
        ep = f"{prefix}mlp.experts.{e}."
        if fused:
            g, u = gu_all[e, :I_full], gu_all[e, I_full:]
            g_u = _cat0([_rows(g, tp_rank, tp_size), _rows(u, tp_rank, tp_size)])
            d = _cols(d_all[e], tp_rank, tp_size)
        elif rnd and source.on_device:
            g_u = source.get(ep + f"gate_up_proj.weight.tp{tp_rank}", (2 * I, H), device=device)
            d = source.get(ep + f"down_proj.weight.tp{tp_rank}", (H, I), device=device)
        else:
            g = _rows(source.get(ep + "gate_proj.weight", (I_full, H), device=device), tp_rank, tp_size)
            u = _rows(source.get(ep + "up_proj.weight", (I_full, H), device=device), tp_rank, tp_size)
            g_u = _cat0([g, u])
            d = _cols(source.get(ep + "down_proj.weight", (H, I_full), device=device), tp_rank, tp_size)
        w13_parts.append(g_u.to(device))
        w2_parts.append(d.to(device))
    n_local = hi - lo
    w13 = _cat0(w13_parts)
    w2 = _cat0(w2_parts)
    w13_s = w2_s = None
    nv = {}
    if isinstance(w13, Fp8Pair) and isinstance(w2, Fp8Pair) and quant in (None, "fp8_block") and H % 128 == 0 and I % 128 == 0:
        # an FP8 checkpoint's expert stacks: its own values and block scales, bit for bit
        w13, w13_s = w13.q.contiguous(), w13.s.float().contiguous()
        w2, w2_s = w2.q.contiguous(), w2.s.float().contiguous()
    elif quant == "nvfp4" and H % 256 == 0 and I % 256 == 0 and n_local > 0:
        # NVFP4 experts: every expert's two matrices quantised on their own (e2m1 values, e4m3 scales per 16
        # elements, one fp32 tensor scale per expert and matrix), stacked for the grouped block-scaled GEMM
        w13, w2 = _dense(w13), _dense(w2)
        q13 = [ref.quant_nvfp4(w13[e * 2 * I:(e + 1) * 2 * I]) for e in range(n_local)]
        q2 = [ref.quant_nvfp4(w2[e * H:(e + 1) * H]) for e in range(n_local)]
        nv = dict(w13_bs=torch.cat([q[1] for q in q13]).contiguous(), w13_ts=torch.stack([q[2] for q in q13]).float().contiguous(),
                  w2_bs=torch.cat([q[1] for q in q2]).contiguous(), w2_ts=torch.stack([q[2] for q in q2]).float().contiguous())
        w13, w2 = torch.cat([q[0] for q in q13]).contiguous(), torch.cat([q[0] for q in q2]).contiguous()
    elif quant in ("fp8_block", "nvfp4") and H % 128 == 0 and I % 128 == 0:     # grouped experts: FP8 blocks
        w13, w2 = _dense(w13), _dense(w2)
        w13, w13_s = ref.quant_weight_fp8_block(w13)
        w2, w2_s = ref.quant_weight_fp8_block(w2)
    else:
        w13, w2 = _dense(w13).to(dtype).contiguous(), _dense(w2).to(dtype).contiguous()
    mw = MoEWeights(router, rbias, w13, w13_s, w2, w2_s, E, I, H, expert_lo=lo, expert_hi=hi, **nv)
    sI_full = cfg.shared_expert_intermediate_size
    if sI_full:
        sp = prefix + "mlp.shared_expert."
        g = _rows(source.get(sp + "gate_proj.weight", (sI_full, H), device=device), sh_rank, sh_size)
        u = _rows(source.get(sp + "up_proj.weight", (sI_full, H), device=device), sh_rank, sh_size)
        d = _cols(source.get(sp + "down_proj.weight", (H, sI_full), device=device), sh_rank, sh_size)
        mw.shared_gate_up = _make_linear(_cat0([g, u]), None, device, dtype, quant)
        mw.shared_down = _make_linear(d, None, device, dtype, quant)
        if cfg.shared_expert_gate:
            mw.shared_gate = source.get(prefix + "mlp.shared_expert_gate.weight", (1, H), device=device).to(device=device, dtype=dtype)
    return mw


def route_reference(logits, cfg: ModelConfig, bias=None):
    """Plain statement of the routing rules; returns (ids [T,K] int64, weights [T,K] fp32)."""
    K = cfg.num_experts_per_tok
    if cfg.moe_scoring == "sigmoid":
        score = torch.sigmoid(logits.float())
    else:
        score = torch.softmax(logits.float(), dim=-1)
    sel = score + (bias.float() if bias is not None else 0.0)
    if cfg.n_group > 1 and cfg.topk_group < cfg.n_group:
        T, E = sel.shape
        grp = sel.view(T, cfg.n_group, E // cfg.n_group)
        gscore = grp.topk(2, dim=-1).values.sum(-1)
        keep = gscore.topk(cfg.topk_group, dim=-1).indices
        mask = torch.zeros(T, cfg.n_group, dtype=torch.bool, device=sel.device).scatter_(1, keep, True)
        sel = sel.masked_fill(~mask.unsqueeze(-1).expand_as(grp).reshape(T, E), float("-inf"))
    ids = sel.topk(K, dim=-1).indices
    w = score.gather(1, ids)
    if cfg.norm_topk_prob:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return ids, w * cfg.routed_scaling_factor


def moe_forward(model, mw: MoEWeights, x: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
    """h += MoE(x) (reduced over the TP group). ``x`` is the normalised hidden state [T, H] (bf16)."""
    if getattr(model, "dp", None) is not None:
        return model.dp.moe(model, mw, x, h)           # attention data parallelism: dispatch / experts / combine
    out = moe_partial(model, mw, x)
    if model.tp_size > 1:
        out = model.comm.all_reduce(out)
    return ops.add(h, out)


def ep_layout(cfg: ModelConfig, tp_rank: int, tp_size: int):
    """(expert-parallel rank, size) of this rank: an explicit layout set by the engine (attention data parallelism:
    experts spread over the data-parallel ranks) or the tensor-parallel group when ``expert_para_size`` > 1."""
    forced = getattr(cfg, "ep_layout_override", None)
    if forced is not None:
        return forced
    return (tp_rank, tp_size) if cfg.expert_para_size > 1 else (0, 1)


def shared_expert(model, mw: MoEWeights, x: torch.Tensor) -> torch.Tensor:
    """Shared expert(s) of an MoE block applied to ``x`` (this rank's slice under tensor parallelism)."""
    cfg = model.cfg
    sg = ops.linear(x, mw.shared_gate_up)
    sa = ops.act_mul(sg, cfg.activation, True, quant_for=mw.shared_down)
    so = ops.linear(sa, mw.shared_down)
    if mw.shared_gate is not None:
        so = (so.float() * torch.sigmoid(x.float() @ mw.shared_gate.float().t())).to(x.dtype)
    return so


def route(model, mw: MoEWeights, x: torch.Tensor):
    """Expert choice of every row of ``x``: (ids [T, K] int32, weights [T, K] fp32), by the router of this block."""
    cfg = model.cfg
    T = x.shape[0]
    K, E = cfg.num_experts_per_tok, mw.num_experts
    if x.is_cuda:
        logits = torch.empty(T, E, dtype=torch.float32, device=x.device)
        native.gemm_bf16(x, mw.router.to(torch.bfloat16) if mw.router.dtype != torch.bfloat16 else mw.router, out_f32=logits)
        return native.moe_route(logits, K, cfg.moe_scoring, cfg.norm_topk_prob, cfg.routed_scaling_factor,
                                mw.router_bias, cfg.n_group, cfg.topk_group)
    ids, w = route_reference(x.float() @ mw.router.float().t(), cfg, mw.router_bias)
    return ids.to(torch.int32), w.float()


def moe_partial(model, mw: MoEWeights, x: torch.Tensor, into: Optional[torch.Tensor] = None,
                shared: bool = True, routing=None) -> torch.Tensor:
    """This rank's share of MoE(x): the weighted outputs of the experts (or expert slices) it holds plus its slice
    of the shared expert, before any reduction over ranks. ``into`` ([T, H], e.g. a peer-visible buffer that a
    reduce kernel pulls from) receives the result when given. ``routing`` = (ids [T, K] int32, weights [T, K] fp32)
    decided elsewhere (the row's home rank under expert-parallel all-to-all dispatch; choices of experts this rank
    does not hold carry id -1) replaces this block's own router."""
    cfg = model.cfg
    T, H = x.shape
    K, E = cfg.num_experts_per_tok, mw.num_experts
    n_local = mw.expert_hi - mw.expert_lo
    if x.is_cuda:
        ids, w = routing if routing is not None else route(model, mw, x)
        dst_row, tile_expert, _, _, cap = native.moe_align(ids, E, mw.expert_lo, mw.expert_hi)
        if mw.expert_lo:
            tile_expert = torch.where(tile_expert >= 0, tile_expert - mw.expert_lo, tile_expert)
        perm = native.moe_permute(x, dst_row, K, cap, zero=mw.nvfp4)
        if mw.nvfp4:
            # activations go to NVFP4 too: one tensor scale per GEMM input from its own maximum (no host sync);
            # padding rows are zero so that they do not enter the maximum
            a_ts = native.absmax_scale(x, 448.0 * 6.0)
            pq, pbs, _ = native.quant_nvfp4(perm, a_ts)
            g = native.gemm_grouped_nvfp4(pq, pbs, a_ts, mw.w13, mw.w13_bs, mw.w13_ts, tile_expert, n_local, 2 * mw.inter)
            a = native.act_mul(g, cfg.activation, True)
            a_ts2 = native.absmax_scale(a, 448.0 * 6.0)
            aq, abs_, _ = native.quant_nvfp4(a, a_ts2)
            y = native.gemm_grouped_nvfp4(aq, abs_, a_ts2, mw.w2, mw.w2_bs, mw.w2_ts, tile_expert, n_local, H)
        elif mw.w13_scale is not None:
            pq, ps = native.quant_fp8(perm)
            g = native.gemm_grouped(pq, mw.w13, tile_expert, n_local, 2 * mw.inter, a_scale=ps, w_scale=mw.w13_scale)
            _, aq, as_ = native.act_mul(g, cfg.activation, True, quant=True, want_out=False)
            y = native.gemm_grouped(aq, mw.w2, tile_expert, n_local, H, a_scale=as_, w_scale=mw.w2_scale)
        else:
            g = native.gemm_grouped(perm, mw.w13, tile_expert, n_local, 2 * mw.inter)
            a = native.act_mul(g, cfg.activation, True)
            y = native.gemm_grouped(a, mw.w2, tile_expert, n_local, H)
        out = into if into is not None else torch.empty(T, H, dtype=x.dtype, device=x.device)
        have_shared = shared and mw.shared_gate_up is not None
        if have_shared:
            sg = ops.linear(x, mw.shared_gate_up)
            sa = ops.act_mul(sg, cfg.activation, True, quant_for=mw.shared_down)
            ops.linear(sa, mw.shared_down, out=out)
            if mw.shared_gate is not None:
                gate = torch.sigmoid(x.float() @ mw.shared_gate.float().t())
                out.copy_(out.float() * gate)
        native.moe_combine(y, dst_row, w, out, K, accumulate=have_shared)
        return out
    else:
        if routing is not None:
            ids, w = routing[0].long(), routing[1].float()
        else:
            ids, w = route_reference(x.float() @ mw.router.float().t(), cfg, mw.router_bias)
        out = torch.zeros(T, H, dtype=torch.float32)
        if mw.nvfp4:
            I2 = 2 * mw.inter
            w13 = torch.cat([ref.dequant_nvfp4(mw.w13[e * I2:(e + 1) * I2], mw.w13_bs[e * I2:(e + 1) * I2], mw.w13_ts[e])
                             for e in range(n_local)])
            w2 = torch.cat([ref.dequant_nvfp4(mw.w2[e * H:(e + 1) * H], mw.w2_bs[e * H:(e + 1) * H], mw.w2_ts[e])
                            for e in range(n_local)])
        else:
            w13 = ref.dequant_weight_fp8_block(mw.w13, mw.w13_scale) if mw.w13_scale is not None else mw.w13.float()
            w2 = ref.dequant_weight_fp8_block(mw.w2, mw.w2_scale) if mw.w2_scale is not None else mw.w2.float()
        fq = (lambda t, ts: ref.dequant_nvfp4(*ref.quant_nvfp4(t, ts))) if mw.nvfp4 else (lambda t, ts: t)
        a_ts = (x.float().abs().amax() / (448.0 * 6.0)).clamp_min(1e-12) if mw.nvfp4 else None
        acts = []
        for e in range(mw.expert_lo, mw.expert_hi):
            tok, slot = (ids == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            le = e - mw.expert_lo
            xe = fq(x[tok].float(), a_ts)
            gu = (xe @ w13[le * 2 * mw.inter:(le + 1) * 2 * mw.inter].t()).to(x.dtype).float()
            a = (ref.act(gu[:, :mw.inter], cfg.activation) * gu[:, mw.inter:]).to(x.dtype).float()
            acts.append((le, tok, slot, a))
        a_ts2 = None
        if mw.nvfp4 and acts:
            a_ts2 = (torch.stack([a.abs().amax() for _, _, _, a in acts]).amax() / (448.0 * 6.0)).clamp_min(1e-12)
        for le, tok, slot, a in acts:
            ye = (fq(a, a_ts2) @ w2[le * H:(le + 1) * H].t()).to(x.dtype).float()
            out.index_add_(0, tok, ye * w[tok, slot].unsqueeze(-1))
        if shared and mw.shared_gate_up is not None:
            sg = ops.linear(x, mw.shared_gate_up)
            sa = ops.act_mul(sg, cfg.activation, True, quant_for=mw.shared_down)
            so = ops.linear(sa, mw.shared_down).float()
            if mw.shared_gate is not None:
                so = so * torch.sigmoid(x.float() @ mw.shared_gate.float().t())
            out = out + so
        out = out.to(x.dtype)
    if into is not None:
        into.copy_(out)
        return into
    return out
