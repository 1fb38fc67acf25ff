"""Device dispatch for the operator layer: CUDA tensors go to the hand-written sm_100a kernels
(:mod:`.native`), CPU tensors to the PyTorch statements (:mod:`.reference`). Model code calls
only this module, so the same model definition runs the CPU test slice and the B200 path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from . import native, reference as ref


@dataclass
class QTensor:
    """FP8 GEMM operand: e4m3 values [M,K] and fp32 scales [K/128, ld] (one per row and 128 columns)."""
    q: torch.Tensor
    s: torch.Tensor

    @property
    def shape(self):
        return self.q.shape


class LinearWeight:
    """[N,K] weight of y = x W^T (+bias): dense bf16/fp32, or e4m3 with one fp32 scale per 128x128 block."""

    def __init__(self, w: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                 wq: Optional[torch.Tensor] = None, ws: Optional[torch.Tensor] = None):
        self.w, self.bias, self.wq, self.ws = w, bias, wq, ws
        # NVFP4 form: packed e2m1 [N, K/2], e4m3 scales per 16 elements [N, K/16], fp32 tensor scale
        self.w4 = self.w4_bs = self.w4_ts = None
        # weight-only 4-bit groups (GPTQ / AWQ family): packed levels [N, K/2], fp16 scale and zero*scale [N, K/g]
        self.q4 = self.q4_scale = self.q4_zs = None
        # power-of-two block scales: the tensor cores can apply them (hardware block-scaled MMA)
        self.ue8m0 = ws is not None and ref.is_pow2(ws)

    @property
    def fp8(self) -> bool:
        return self.wq is not None

    @property
    def nvfp4(self) -> bool:
        return self.w4 is not None

    @property
    def w4a16(self) -> bool:
        return self.q4 is not None

    def _any(self) -> torch.Tensor:
        if self.w4a16:
            return self.q4
        return self.w4 if self.nvfp4 else (self.wq if self.fp8 else self.w)

    @property
    def out_features(self) -> int:
        return self._any().shape[0]

    @property
    def in_features(self) -> int:
        return self._any().shape[1] * 2 if (self.nvfp4 or self.w4a16) else self._any().shape[1]

    @property
    def device(self):
        return self._any().device

    def without_bias(self) -> "LinearWeight":
        """Shallow copy that shares the weight tensors and has no bias (row-parallel ranks other than the first)."""
        if self.bias is None:
            return self
        if getattr(self, "_nb", None) is None:
            import copy
            self._nb = copy.copy(self)
            self._nb.bias = None
        return self._nb

    def quantize_nvfp4(self) -> "LinearWeight":
        """e2m1 weights with e4m3 scales per 16 input features (in_features must be a multiple of 256)."""
        if not self.nvfp4 and not self.fp8:
            self.w4, self.w4_bs, self.w4_ts = ref.quant_nvfp4(self.w)
            self.w = None
        return self

    def quantize_w4(self, group: int = 128) -> "LinearWeight":
        """4-bit weight-only groups along the input features (in_features must be a multiple of 32)."""
        if not (self.w4a16 or self.nvfp4 or self.fp8):
            self.q4, self.q4_scale, self.q4_zs = ref.quant_w4(self.w, group)
            self.w = None
        return self

    def quantize_fp8_block(self) -> "LinearWeight":
        if not self.fp8:
            self.wq, self.ws = ref.quant_weight_fp8_block(self.w)
            self.w = None
            self.ue8m0 = True
        return self

    def dense(self) -> torch.Tensor:
        if self.w4a16:
            return ref.dequant_w4(self.q4, self.q4_scale, self.q4_zs)
        if self.nvfp4:
            return ref.dequant_nvfp4(self.w4, self.w4_bs, self.w4_ts)
        return ref.dequant_weight_fp8_block(self.wq, self.ws) if self.fp8 else self.w

    def nbytes(self) -> int:
        t = [x for x in (self.w, self.wq, self.ws, self.bias, self.w4, self.w4_bs, self.q4, self.q4_scale, self.q4_zs)
             if x is not None]
        return sum(x.numel() * x.element_size() for x in t)


def _is_cuda(x) -> bool:
    return (x.q if isinstance(x, QTensor) else x).is_cuda


def quantize(x: torch.Tensor) -> QTensor:
    if x.is_cuda:
        return QTensor(*native.quant_fp8(x))
    return QTensor(*ref.quant_fp8(x))


def linear(x, W: LinearWeight, residual=None, out=None, out_f32: bool = False):
    """y = x W^T (+bias) (+residual). ``x`` may be a QTensor when W is FP8. ``out`` may alias ``residual``."""
    if W.w4a16:
        if isinstance(x, QTensor):
            raise TypeError("4-bit weight-only layers take bf16 activations")
        if x.is_cuda:
            if out_f32:
                return native.linear_w4(x, W.q4, W.q4_scale, W.q4_zs, bias=W.bias, residual=residual).float()
            return native.linear_w4(x, W.q4, W.q4_scale, W.q4_zs, out=out, bias=W.bias, residual=residual)
        y = ref.gemm(x, W.dense().to(x.dtype), W.bias, residual, torch.float32 if out_f32 else None)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if W.nvfp4:
        # activations are quantised to NVFP4 too (per-tensor scale from the tensor's own maximum, no host sync)
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0:
            a_ts = native.absmax_scale(x, 448.0 * 6.0)          # one pass over x, scale stays on the device
        else:
            a_ts = (x.float().abs().amax() / (448.0 * 6.0)).clamp_min(1e-12).reshape(())
        if x.is_cuda:
            aq, a_bs, _ = native.quant_nvfp4(x, a_ts)
            if out_f32:
                o = torch.empty(x.shape[0], W.out_features, dtype=torch.float32, device=x.device)
                return native.gemm_nvfp4(aq, a_bs, a_ts, W.w4, W.w4_bs, W.w4_ts, bias=W.bias, residual=residual, out_f32=o)
            return native.gemm_nvfp4(aq, a_bs, a_ts, W.w4, W.w4_bs, W.w4_ts, out=out, bias=W.bias, residual=residual)
        aq, a_bs, _ = ref.quant_nvfp4(x, a_ts)
        y = ref.gemm_nvfp4(aq, a_bs, a_ts, W.w4, W.w4_bs, W.w4_ts, W.bias, residual, torch.float32 if out_f32 else x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if _is_cuda(x):
        if W.fp8:
            if not isinstance(x, QTensor):
                x = quantize(x)
            if out_f32:
                o = torch.empty(x.q.shape[0], W.out_features, dtype=torch.float32, device=x.q.device)
                return native.gemm_fp8(x.q, x.s, W.wq, W.ws, bias=W.bias, residual=residual, out_f32=o, hw_scale=W.ue8m0)
            return native.gemm_fp8(x.q, x.s, W.wq, W.ws, out=out, bias=W.bias, residual=residual, hw_scale=W.ue8m0)
        if out_f32:
            o = torch.empty(x.shape[0], W.out_features, dtype=torch.float32, device=x.device)
            return native.gemm_bf16(x, W.w, bias=W.bias, residual=residual, out_f32=o)
        return native.gemm_bf16(x, W.w, out=out, bias=W.bias, residual=residual)
    # CPU statement
    if W.fp8:
        xq = x if isinstance(x, QTensor) else QTensor(*ref.quant_fp8(x))
        y = ref.gemm_fp8(xq.q, xq.s, W.wq, W.ws, W.bias, residual, torch.float32 if out_f32 else torch.bfloat16)
    else:
        y = ref.gemm(x, W.w, W.bias, residual, torch.float32 if out_f32 else x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def norm(x, w, eps, residual=None, beta=None, layernorm=False, quant_for: Optional[LinearWeight] = None):
    """Returns the normalised activations in the form the consuming linear wants (QTensor for FP8
    weights on CUDA). ``residual`` (if given) is updated in place with residual + x."""
    want_q = quant_for is not None and quant_for.fp8 and x.shape[-1] % 128 == 0
    if x.is_cuda:
        if want_q:
            _, q, s = native.norm(x, w, eps, residual=residual, beta=beta, layernorm=layernorm, quant=True,
                                  want_out=False)
            return QTensor(q, s)
        return native.norm(x, w, eps, residual=residual, beta=beta, layernorm=layernorm)
    y, new_res = ref.norm(x, w, eps, residual, beta, layernorm)
    if residual is not None:
        residual.copy_(new_res)
    return QTensor(*ref.quant_fp8(y)) if want_q else y


def act_mul(x, kind="silu", gated=True, quant_for: Optional[LinearWeight] = None):
    inter = x.shape[-1] // 2 if gated else x.shape[-1]
    want_q = quant_for is not None and quant_for.fp8 and inter % 128 == 0
    if x.is_cuda:
        if want_q:
            _, q, s = native.act_mul(x, kind, gated, quant=True, want_out=False)
            return QTensor(q, s)
        return native.act_mul(x, kind, gated)
    y = ref.act_mul(x, kind, gated)
    return QTensor(*ref.quant_fp8(y)) if want_q else y


def embedding(ids, table, vocab_lo=0, vocab_hi=None, positions=None, pos_table=None, scale=1.0):
    if table.is_cuda:
        return native.embedding(ids, table, vocab_lo=vocab_lo, vocab_hi=vocab_hi, positions=positions,
                                pos_table=pos_table, scale=scale)
    return ref.embedding(ids, table, vocab_lo, vocab_hi, positions, pos_table, scale)


def gather_rows(x, idx):
    if x.is_cuda:
        return native.gather_rows(x, idx)
    return x[idx.long()]


def add(a, b=None, bias=None):
    if a.is_cuda:
        return native.add(a, b, bias)
    y = a.float()
    if b is not None:
        y = y + b.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(a.dtype)


def rope_kv_append(qkv, positions, slots, cos_sin, cache_layer, block_tokens, Hq, Hkv, D, rot_dim, neox=True,
                   mrope_sections=None, k_scale=1.0, v_scale=1.0, apply_rope=True):
    if qkv.is_cuda:
        native.rope_kv_append(qkv, positions, slots, cos_sin, cache_layer,
                              cache_layer.stride(0) if cache_layer is not None else 0, block_tokens, Hq, Hkv, D,
                              rot_dim, neox, mrope_sections, k_scale, v_scale, apply_rope)
    else:
        ref.rope_kv_append(qkv, positions, slots, cos_sin, cache_layer, block_tokens, Hq, Hkv, D, rot_dim, neox,
                           mrope_sections, k_scale, v_scale, apply_rope)


def decode_splits(batch: int, hkv: int, max_kv_len: int, sms: int = 148, ctas_per_sm: int = 2) -> int:
    """Split-KV factor of the decode attention kernel. One CTA serves one (sequence, kv head, split) and two CTAs
    fit an SM (shared memory), so the time is about waves x (64-token tiles per split + a fixed set-up cost of about
    two tiles); the factor minimising that is chosen, with at least two tiles per split."""
    import os
    forced = int(os.environ.get("KSANA_DECODE_SPLITS", "0"))
    tiles = max(1, (max_kv_len + 63) // 64)
    most = max(1, min(32, tiles // 2))
    if forced > 0:
        return min(forced, most)
    slots = sms * ctas_per_sm
    best, best_cost = 1, None
    for n in range(1, most + 1):
        waves = (batch * hkv * n + slots - 1) // slots
        cost = waves * ((tiles + n - 1) // n + 2)
        if best_cost is None or cost < best_cost:
            best, best_cost = n, cost
    return best


def paged_attention(qkv, out, cache_layer, block_tokens, block_table, cu_q, kv_lens, num_multi, num_single,
                    num_multi_tokens, max_q_len, Hq, Hkv, D, scale, alibi=None, k_scale=1.0, v_scale=1.0,
                    num_splits=1, workspace=None, quant_for: Optional[LinearWeight] = None):
    """Attention of this step's new tokens (rows of ``qkv``: multi-token sequences first, then one row per
    single-token sequence) against the paged cache, which already holds their K/V. ``out`` None allocates the
    result; with ``quant_for`` (the FP8 linear that consumes it) a pure decode step returns the QTensor that linear
    wants, quantised inside the attention kernels."""
    T = qkv.shape[0]
    if qkv.is_cuda and quant_for is not None and quant_for.fp8 and num_multi == 0 and num_single and D == 128 and out is None:
        po, pml = workspace if workspace is not None else (None, None)
        if num_splits > 1 and po is None:
            po = torch.empty(num_single * Hq * num_splits * D, dtype=torch.float32, device=qkv.device)
            pml = torch.empty(num_single * Hq * num_splits * 2, dtype=torch.float32, device=qkv.device)
        oq = torch.empty(T, Hq * D, dtype=torch.float8_e4m3fn, device=qkv.device)
        osc = torch.empty(Hq, max(4, (T + 3) // 4 * 4), dtype=torch.float32, device=qkv.device)
        native.paged_decode(qkv, qkv.stride(0), None, cache_layer, cache_layer.stride(0), block_tokens, block_table,
                            kv_lens, num_single, Hq, Hkv, D, scale, alibi, k_scale, v_scale, num_splits, po, pml,
                            out_q=oq, out_scale=osc)
        return QTensor(oq, osc)
    if out is None:
        out = torch.empty(T, Hq * D, dtype=qkv.dtype, device=qkv.device)
    if qkv.is_cuda:
        if num_multi:
            native.paged_prefill(qkv, qkv.stride(0), out, cache_layer, cache_layer.stride(0), block_tokens, block_table,
                                 cu_q, kv_lens, num_multi, max_q_len, Hq, Hkv, D, scale, alibi, k_scale, v_scale)
        if num_single:
            po, pml = workspace if workspace is not None else (None, None)
            if num_splits > 1 and po is None:
                po = torch.empty(num_single * Hq * num_splits * D, dtype=torch.float32, device=qkv.device)
                pml = torch.empty(num_single * Hq * num_splits * 2, dtype=torch.float32, device=qkv.device)
            native.paged_decode(qkv[num_multi_tokens:], qkv.stride(0), out[num_multi_tokens:], cache_layer,
                                cache_layer.stride(0), block_tokens, block_table[num_multi:], kv_lens[num_multi:],
                                num_single, Hq, Hkv, D, scale, alibi, k_scale, v_scale, num_splits, po, pml)
        return out
    q = qkv[:, : Hq * D]
    o = ref.paged_attention(q, cache_layer, block_table, cu_q, kv_lens, Hq, Hkv, D, scale, alibi, k_scale, v_scale)
    out.copy_(o)
    return out
