"""GPTQ / AWQ 4-bit checkpoints: unpacking of the packed int32 tensors into dense weights.

The reference converts these layouts for its CUTLASS fpA_intB / Marlin kernels
(src/ksana_llm/models/quant/quant_weight.cpp:239-662: unpack, act-order reordering, zero-point handling).
Here a packed linear layer is expanded to its exact dense values when the loader asks for ``<layer>.weight``; the
loader then slices / packs QKV as for any other checkpoint and re-encodes the result in the one 4-bit group
format the W4A16 kernels read (``reference.quant_w4``), or in bf16 / block FP8 / NVFP4 when another
``weight_quant_method`` is configured.

Layouts (K = in_features, N = out_features, g = group size, 8 nibbles per int32):
  GPTQ (AutoGPTQ v1): qweight [K/8, N] packed along K; qzeros [K/g, N/8] packed along N, stored minus one;
                      scales [K/g, N]; optional g_idx [K] = group of every input feature (act-order).
  AWQ  (AutoAWQ GEMM): qweight [K, N/8] packed along N with nibble order 0,2,4,6,1,3,5,7; qzeros [K/g, N/8]
                      in the same order, stored as is; scales [K/g, N].
"""
from __future__ import annotations

from typing import Optional

import torch

AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def _unpack_rows(packed: torch.Tensor) -> torch.Tensor:
    """int32 [R, C] with 8 nibbles per word along the row axis -> [R*8, C] (values 0..15)."""
    shifts = torch.arange(0, 32, 4, dtype=torch.int32).view(1, 8, 1)
    return ((packed.to(torch.int32).unsqueeze(1) >> shifts) & 15).reshape(packed.shape[0] * 8, packed.shape[1])


def _unpack_cols(packed: torch.Tensor, order=None) -> torch.Tensor:
    """int32 [R, C] with 8 nibbles per word along the column axis -> [R, C*8]; ``order[i]`` is the column
    (inside its group of 8) that nibble i holds."""
    shifts = torch.arange(0, 32, 4, dtype=torch.int32).view(1, 1, 8)
    nib = (packed.to(torch.int32).unsqueeze(-1) >> shifts) & 15               # [R, C, 8] by nibble index
    if order is not None:
        out = torch.empty_like(nib)
        out[..., list(order)] = nib
        nib = out
    return nib.reshape(packed.shape[0], packed.shape[1] * 8)


def unpack_gptq(qweight, qzeros, scales, g_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dense fp32 weight [N, K] of a GPTQ layer."""
    q = _unpack_rows(qweight).float()                       # [K, N]
    z = (_unpack_cols(qzeros) + 1).float()                  # [K/g, N]
    K = q.shape[0]
    groups = scales.shape[0]
    if g_idx is None:
        g_idx = torch.arange(K) // (K // groups)
    gi = g_idx.long()
    w = (q - z[gi]) * scales.float()[gi]
    return w.t().contiguous()


def unpack_awq(qweight, qzeros, scales) -> torch.Tensor:
    """Dense fp32 weight [N, K] of an AWQ (GEMM layout) layer."""
    q = _unpack_cols(qweight, AWQ_ORDER).float()            # [K, N]
    z = _unpack_cols(qzeros, AWQ_ORDER).float()             # [K/g, N]
    K = q.shape[0]
    g = K // scales.shape[0]
    gi = torch.arange(K) // g
    w = (q - z[gi]) * scales.float()[gi]
    return w.t().contiguous()


def unpack_auto(qweight, qzeros, scales, g_idx=None) -> torch.Tensor:
    """GPTQ packs along K (qweight has N columns), AWQ along N (qweight has N/8 columns)."""
    if qweight.shape[1] == scales.shape[1]:
        return unpack_gptq(qweight, qzeros, scales, g_idx)
    return unpack_awq(qweight, qzeros, scales)


# --------------------------------------------------------------------------- packers (tests, checkpoint writers)
def _pack_rows(q: torch.Tensor) -> torch.Tensor:
    R, C = q.shape
    v = q.to(torch.int64).reshape(R // 8, 8, C)
    out = torch.zeros(R // 8, C, dtype=torch.int64)
    for i in range(8):
        out |= v[:, i] << (4 * i)
    return ((out + (1 << 31)) % (1 << 32) - (1 << 31)).to(torch.int32)


def _pack_cols(q: torch.Tensor, order=None) -> torch.Tensor:
    R, C = q.shape
    v = q.to(torch.int64).reshape(R, C // 8, 8)
    out = torch.zeros(R, C // 8, dtype=torch.int64)
    for i in range(8):
        out |= v[..., order[i] if order is not None else i] << (4 * i)
    return ((out + (1 << 31)) % (1 << 32) - (1 << 31)).to(torch.int32)


def quantize_levels(w: torch.Tensor, group: int):
    """Asymmetric 4-bit levels of w [N, K]: (q [K, N] ints, zero [K/g, N] ints, scale [K/g, N] fp16)."""
    N, K = w.shape
    wf = w.float().reshape(N, K // group, group)
    lo, hi = wf.amin(-1), wf.amax(-1)
    scale = ((hi - lo) / 15).clamp_min(1e-8).to(torch.float16)
    zero = torch.round(-lo / scale.float()).clamp(0, 15)
    q = torch.round(wf / scale.float().unsqueeze(-1) + zero.unsqueeze(-1)).clamp(0, 15)
    return q.reshape(N, K).t().contiguous().to(torch.int32), zero.t().contiguous().to(torch.int32), scale.t().contiguous()


def pack_gptq(w: torch.Tensor, group: int = 128, act_order: bool = False):
    """Tensors of a GPTQ layer for the dense weight w [N, K] (quantised here): dict with qweight, qzeros, scales, g_idx."""
    N, K = w.shape
    perm = torch.randperm(K, generator=torch.Generator().manual_seed(K)) if act_order else torch.arange(K)
    q, zero, scale = quantize_levels(w[:, perm], group)          # groups are formed in the permuted order
    inv = torch.argsort(perm)
    g_idx = (torch.arange(K) // group)[inv].to(torch.int32)      # group of every original input feature
    q = q[inv]                                                   # rows back in original feature order
    return {"qweight": _pack_rows(q), "qzeros": _pack_cols(zero - 1), "scales": scale, "g_idx": g_idx}


def pack_awq(w: torch.Tensor, group: int = 128):
    q, zero, scale = quantize_levels(w, group)
    return {"qweight": _pack_cols(q, AWQ_ORDER), "qzeros": _pack_cols(zero, AWQ_ORDER), "scales": scale}
