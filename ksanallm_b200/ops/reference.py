"""Plain PyTorch statements of every op (fp32 math). They are the oracles the CUDA kernels are
tested against and the execution path for CPU tensors (unit tests, the CPU end-to-end slice).
Signatures mirror :mod:`ksanallm_b200.ops.native`.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

E4M3_MAX = 448.0


def gemm(x, w, bias=None, residual=None, out_dtype=None):
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def pow2_scale(amax):
    """Smallest power of two >= amax / 448 (UE8M0 scale), computed on the fp32 bit pattern like the kernels do."""
    s = amax.float().clamp_min(1e-10) * (1.0 / E4M3_MAX)
    bits = s.contiguous().view(torch.int32)
    e = (bits >> 23) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return (e << 23).view(torch.float32)


def is_pow2(scale) -> bool:
    """True when every (positive, normal) fp32 scale is an exact power of two."""
    bits = scale.float().contiguous().view(torch.int32)
    return bool(((bits & 0x7FFFFF) == 0).all() and (bits > 0).all())


def quant_fp8(x):
    """Per (row, 128 columns) e4m3 quantisation with power-of-two scales; scales returned as [K/128, M]
    (k-group major)."""
    M, K = x.shape
    g = x.float().reshape(M, K // 128, 128)
    scale = pow2_scale(g.abs().amax(dim=-1))
    q = (g / scale.unsqueeze(-1)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).reshape(M, K)
    return q, scale.t().contiguous()


WEIGHT_SCALE_POW2 = True   # default scale rule of quant_weight_fp8_block (engine option quantization.fp8_scale_mode)


def quant_weight_fp8_block(w, block=128, pow2=None):
    """[N,K] weight -> e4m3 + one fp32 scale per (128 x 128) block, scales [ceil(N/128), ceil(K/128)].
    pow2: power-of-two scales (what the tensor cores can apply themselves); False: amax / 448 exactly;
    None: the module default ``WEIGHT_SCALE_POW2``."""
    if pow2 is None:
        pow2 = WEIGHT_SCALE_POW2
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.reshape(nb, block, kb, block)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = pow2_scale(amax) if pow2 else amax / E4M3_MAX
    q = (blocks / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).reshape(nb * block, kb * block)[:N, :K]
    return q.to(torch.float8_e4m3fn).contiguous(), scale.contiguous()


def dequant_weight_fp8_block(wq, ws, block=128):
    N, K = wq.shape
    s = ws.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return wq.float() * s


def gemm_fp8(xq, xs, wq, ws, bias=None, residual=None, out_dtype=torch.bfloat16):
    M, K = xq.shape
    x = xq.float().reshape(M, K // 128, 128) * xs[:, :M].t().unsqueeze(-1)
    y = x.reshape(M, K) @ dequant_weight_fp8_block(wq, ws).t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype)


def norm(x, w, eps, residual=None, beta=None, layernorm=False):
    """Returns (y, new_residual). With a residual the sum is rounded to the activation dtype first."""
    h = x.float()
    if residual is not None:
        h = (h + residual.float()).to(x.dtype).float()
    if layernorm:
        mu = h.mean(-1, keepdim=True)
        var = (h - mu).pow(2).mean(-1, keepdim=True)
        y = (h - mu) * torch.rsqrt(var + eps) * w.float()
    else:
        y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    if beta is not None:
        y = y + beta.float()
    return y.to(x.dtype), h.to(x.dtype)


def act(x, kind="silu"):
    if kind in ("silu", "swiglu"):
        return F.silu(x)
    if kind in ("gelu", "gelu_new", "gelu_pytorch_tanh"):
        return F.gelu(x, approximate="tanh")
    if kind == "relu":
        return F.relu(x)
    raise ValueError(kind)


def act_mul(x, kind="silu", gated=True):
    xf = x.float()
    if gated:
        inter = x.shape[-1] // 2
        return (act(xf[..., :inter], kind) * xf[..., inter:]).to(x.dtype)
    return act(xf, kind).to(x.dtype)


def embedding(ids, table, vocab_lo=0, vocab_hi=None, positions=None, pos_table=None, scale=1.0):
    hi = vocab_lo + table.shape[0] if vocab_hi is None else vocab_hi
    mine = (ids >= vocab_lo) & (ids < hi)
    local = torch.where(mine, ids - vocab_lo, torch.zeros_like(ids)).long()
    out = table[local].float() * scale
    if pos_table is not None:
        out = out + pos_table[positions.long()].float()
    out = out * mine.unsqueeze(-1)
    return out.to(table.dtype)


def build_cos_sin_cache(rot_dim, max_pos, base=10000.0, scaling=None, device="cpu"):
    """[max_pos, rot_dim] = cos | sin. ``scaling`` follows HF ``rope_scaling`` dicts
    (linear, dynamic, llama3, yarn) as handled by the reference
    (3rdparty/LLM_kernels/csrc/kernels/nvidia/rotary_embedding/rotary_embedding.cu:202-340)."""
    half = rot_dim // 2
    inv_freq = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float64) * 2 / rot_dim))
    t = torch.arange(max_pos, dtype=torch.float64)
    mscale = 1.0
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type", "default"))
        factor = float(scaling.get("factor", 1.0))
        if kind == "linear":
            t = t / factor
        elif kind == "dynamic":
            orig = scaling.get("original_max_position_embeddings", max_pos)
            alpha = scaling.get("alpha")
            if alpha is not None:   # NTK-alpha variant
                nb = base * float(alpha) ** (rot_dim / (rot_dim - 2))
            else:
                nb = base * ((factor * max_pos / orig) - (factor - 1)) ** (rot_dim / (rot_dim - 2)) if max_pos > orig else base
            inv_freq = 1.0 / (nb ** (torch.arange(0, half, dtype=torch.float64) * 2 / rot_dim))
        elif kind == "llama3":
            low, high = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv_freq
            smooth = ((orig / wavelen) - low) / (high - low)
            scaled = torch.where(wavelen > orig / low, inv_freq / factor, inv_freq)
            mid = (wavelen <= orig / low) & (wavelen >= orig / high)
            inv_freq = torch.where(mid, (1 - smooth) * inv_freq / factor + smooth * inv_freq, scaled)
        elif kind == "yarn":
            orig = float(scaling.get("original_max_position_embeddings", 4096))
            beta_fast, beta_slow = float(scaling.get("beta_fast", 32)), float(scaling.get("beta_slow", 1))

            def corr_dim(rot):
                return rot_dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(base))

            lo = max(math.floor(corr_dim(beta_fast)), 0)
            hi = min(math.ceil(corr_dim(beta_slow)), rot_dim - 1)
            ramp = ((torch.arange(half, dtype=torch.float64) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
            mask = 1 - ramp
            inv_freq = inv_freq / factor * (1 - mask) + inv_freq * mask
            ms = float(scaling.get("mscale", 1.0))
            ms_all = float(scaling.get("mscale_all_dim", 0.0))

            def get_mscale(s, m):
                return 1.0 if s <= 1 else 0.1 * m * math.log(s) + 1.0

            mscale = get_mscale(factor, ms) / get_mscale(factor, ms_all) if ms_all else get_mscale(factor, 1.0)
    freqs = torch.outer(t, inv_freq)
    return torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1).float().to(device)


def apply_rope(x, positions, cos_sin, rot_dim, neox=True, mrope_sections=None):
    """x [T, H, D]; positions [T] or [3, T] with mrope_sections."""
    T, H, D = x.shape
    half = rot_dim // 2
    if mrope_sections is not None:
        s0, s1 = mrope_sections[0], mrope_sections[0] + mrope_sections[1]
        j = torch.arange(half, device=x.device)
        sec = torch.where(j < s0, 0, torch.where(j < s1, 1, 2))
        pos = positions.long()[sec, :].t()                     # [T, half]
        cs_cos = cos_sin[:, :half][pos, j]                     # [T, half]
        cs_sin = cos_sin[:, half:][pos, j]
    else:
        cs = cos_sin[positions.long()]
        cs_cos, cs_sin = cs[:, :half], cs[:, half:]
    cos, sin = cs_cos.unsqueeze(1).float(), cs_sin.unsqueeze(1).float()
    xf = x.float()
    rot = xf[..., :rot_dim]
    if neox:
        x0, x1 = rot[..., :half], rot[..., half:]
        r = torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1)
    else:
        x0, x1 = rot[..., 0::2], rot[..., 1::2]
        r = torch.stack([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1).flatten(-2)
    return torch.cat([r, xf[..., rot_dim:]], dim=-1).to(x.dtype)


def rope_kv_append(qkv, positions, slots, cos_sin, cache_layer, block_tokens, Hq, Hkv, D, rot_dim, neox=True,
                   mrope_sections=None, k_scale=1.0, v_scale=1.0, apply=True):
    """In place on qkv [T,(Hq+2Hkv)*D]; cache_layer viewed as [blocks, 2, Hkv, block_tokens, D]."""
    T = qkv.shape[0]
    q = qkv[:, : Hq * D].reshape(T, Hq, D)
    k = qkv[:, Hq * D: (Hq + Hkv) * D].reshape(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    if apply:
        q.copy_(apply_rope(q, positions, cos_sin, rot_dim, neox, mrope_sections))
        k.copy_(apply_rope(k, positions, cos_sin, rot_dim, neox, mrope_sections))
    if cache_layer is None:
        return
    ok = slots >= 0
    sl = slots[ok].long()
    blk, off = sl // block_tokens, sl % block_tokens
    if cache_layer.dtype == torch.float8_e4m3fn:
        cache_layer[blk, 0, :, off] = (k[ok].float() / k_scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
        cache_layer[blk, 1, :, off] = (v[ok].float() / v_scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    else:
        cache_layer[blk, 0, :, off] = k[ok].to(cache_layer.dtype)
        cache_layer[blk, 1, :, off] = v[ok].to(cache_layer.dtype)


def paged_attention(q, cache_layer, block_table, cu_q, kv_lens, Hq, Hkv, D, scale, alibi=None, k_scale=1.0,
                    v_scale=1.0):
    """q [T, Hq*D] (new tokens only); returns [T, Hq*D]. Query i of sequence s sits at absolute position
    kv_len - q_len + i and sees cache positions <= its own."""
    T = q.shape[0]
    out = torch.zeros(T, Hq * D, dtype=q.dtype, device=q.device)
    B = kv_lens.numel()
    G = Hq // Hkv
    bt = cache_layer.shape[3]
    for s in range(B):
        q0, q1 = int(cu_q[s]), int(cu_q[s + 1])
        ql, kl = q1 - q0, int(kv_lens[s])
        if ql == 0:
            continue
        nblk = (kl + bt - 1) // bt
        blocks = block_table[s, :nblk].long()
        kv = cache_layer[blocks].float()                                  # [nblk, 2, Hkv, bt, D]
        k = kv[:, 0].permute(1, 0, 2, 3).reshape(Hkv, nblk * bt, D)[:, :kl] * k_scale
        v = kv[:, 1].permute(1, 0, 2, 3).reshape(Hkv, nblk * bt, D)[:, :kl] * v_scale
        qs = q[q0:q1].float().reshape(ql, Hkv, G, D).permute(1, 2, 0, 3)  # [Hkv, G, ql, D]
        att = torch.einsum("hgqd,hkd->hgqk", qs, k) * scale
        qpos = torch.arange(kl - ql, kl, device=q.device).unsqueeze(1)
        kpos = torch.arange(kl, device=q.device).unsqueeze(0)
        if alibi is not None:
            att = att + alibi.float().reshape(Hkv, G, 1, 1) * (kpos - qpos).float()
        att = att.masked_fill(kpos > qpos, float("-inf"))
        p = torch.softmax(att, dim=-1)
        o = torch.einsum("hgqk,hkd->hgqd", p, v).permute(2, 0, 1, 3).reshape(ql, Hq * D)
        out[q0:q1] = o.to(q.dtype)
    return out


def sample(logits, temperature, top_k, top_p, uniforms, num_logprobs=0):
    """Row-wise reference of the fused sampler; ``uniforms`` [B] in [0,1) replaces the device RNG."""
    B, V = logits.shape
    tokens = torch.zeros(B, dtype=torch.int64)
    lp_ids = torch.full((B, num_logprobs), -1, dtype=torch.int64)
    lp_vals = torch.full((B, num_logprobs), float("-inf"))
    for b in range(B):
        row = logits[b].float()
        t = float(temperature[b]) if float(temperature[b]) > 0 else 1.0
        k = max(1, min(int(top_k[b]), 1024, V))
        vals, idx = torch.sort(row, descending=True, stable=True)
        if num_logprobs:
            n = min(num_logprobs, V)
            lp = torch.log_softmax(vals[:n] / t, dim=-1)
            lp_ids[b, :n], lp_vals[b, :n] = idx[:n], lp
        if k == 1:
            tokens[b] = idx[0]
            continue
        w = torch.exp(vals[:k] / t - vals[0] / t)
        p = float(top_p[b]) if 0 < float(top_p[b]) < 1 else 1.0
        cum = torch.cumsum(w, 0)
        keep = k if p >= 1 else int((cum >= p * cum[-1]).nonzero()[0]) + 1
        mass = cum[keep - 1] if p < 1 else cum[-1]
        u = float(uniforms[b]) * float(mass)
        pick = int((cum[:keep] > u).nonzero()[0]) if bool((cum[:keep] > u).any()) else keep - 1
        tokens[b] = idx[pick]
    return tokens, lp_ids, lp_vals


# ------------------------------------------------------------------------------------- NVFP4
# e2m1 values in blocks of 16 along K, one e4m3 scale per block and one fp32 scale per tensor:
#   x ~= e2m1 * e4m3_block_scale * tensor_scale.  Two values per byte, the even element in the low nibble.
_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def quant_nvfp4(x, tensor_scale=None):
    """[M, K] -> (packed uint8 [M, K/2], block scales float8_e4m3fn [M, K/16], tensor scale fp32 scalar tensor).
    K must be a multiple of 16. ``tensor_scale`` None: amax / (448 * 6), so that block scales use the e4m3 range."""
    M, K = x.shape
    xf = x.float()
    if tensor_scale is None:
        tensor_scale = (xf.abs().amax().clamp_min(1e-12) / (448.0 * 6.0)).reshape(())
    tensor_scale = torch.as_tensor(tensor_scale, dtype=torch.float32, device=x.device).reshape(())
    g = xf.reshape(M, K // 16, 16) / tensor_scale
    bs = (g.abs().amax(dim=-1) / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)       # e4m3 rounding of amax / 6
    bsf = bs.float().clamp_min(2.0 ** -9)
    v = (g / bsf.unsqueeze(-1)).clamp(-6.0, 6.0)
    grid = torch.tensor(_E2M1_VALUES, device=x.device)
    # round to nearest e2m1 magnitude, ties to the even code (codes 0..7)
    mag = v.abs()
    mids = (grid[1:] + grid[:-1]) / 2
    code = torch.bucketize(mag, mids, right=False)            # mag == midpoint -> lower code
    tie = mag == mids[(code).clamp(max=6)]
    up = tie & (code % 2 == 1) & (code < 7)
    code = torch.where(up, code + 1, code)
    code = (code | ((v < 0).to(code.dtype) << 3)).to(torch.uint8).reshape(M, K)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), bs.contiguous(), tensor_scale


def dequant_nvfp4(packed, block_scale, tensor_scale):
    M, K2 = packed.shape
    grid = torch.tensor(_E2M1_VALUES, device=packed.device)
    lo, hi = packed & 0xF, packed >> 4
    codes = torch.stack([lo, hi], dim=-1).reshape(M, K2 * 2).long()
    val = grid[codes & 7] * torch.where((codes & 8) != 0, -1.0, 1.0)
    return (val.reshape(M, -1, 16) * block_scale.float().unsqueeze(-1)).reshape(M, K2 * 2) * tensor_scale


def gemm_nvfp4(aq, a_bs, a_ts, wq, w_bs, w_ts, bias=None, residual=None, out_dtype=torch.bfloat16):
    y = dequant_nvfp4(aq, a_bs, a_ts) @ dequant_nvfp4(wq, w_bs, w_ts).t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype)


def mla_attention(qfull, cache_layer, block_table, cu_q, kv_lens, scale, lora=512):
    """Absorbed multi-head latent attention, plain fp32 statement. qfull [T, G, lora+rope] (q_lat | q_pe),
    cache_layer [blocks, block_tokens, lora+rope] (c_kv | k_pe). Returns [T, G, lora] fp32."""
    T, G, _ = qfull.shape
    bt = cache_layer.shape[1]
    out = torch.zeros(T, G, lora, dtype=torch.float32, device=qfull.device)
    cu, kvl = cu_q.tolist(), kv_lens.tolist()
    for s in range(len(kvl)):
        q0, q1, kl = cu[s], cu[s + 1], kvl[s]
        if q1 == q0:
            continue
        nblk = (kl + bt - 1) // bt
        rows = cache_layer[block_table[s, :nblk].long()].reshape(nblk * bt, -1)[:kl].float()
        sc = torch.einsum("qhd,kd->hqk", qfull[q0:q1].float(), rows) * scale
        qpos = torch.arange(kl - (q1 - q0), kl, device=qfull.device).unsqueeze(1)
        kpos = torch.arange(kl, device=qfull.device).unsqueeze(0)
        sc = sc.masked_fill(kpos > qpos, float("-inf"))
        out[q0:q1] = torch.einsum("hqk,kl->qhl", torch.softmax(sc, -1), rows[:, :lora])
    return out


# ----------------------------------------------------------------------------- 4-bit weight-only groups (W4A16)
def quant_w4(w, group=128):
    """Asymmetric 4-bit group quantisation along K of w [N, K]: returns (packed uint8 [N, K/2] with the even k in
    the low nibble, scale fp16 [N, K/g], zs = zero_point * scale fp16 [N, K/g]); w ~= q * scale - zs.
    Per group the step is (max - min) / n for the n in 15..12 with the smallest error, so a group whose values
    already sit on a 16-level lattice (a dequantised GPTQ / AWQ group, which need not use all 16 levels) is
    reproduced up to the fp16 rounding of zs."""
    N, K = w.shape
    g = min(group, K)
    wf = w.float().reshape(N, K // g, g)
    lo, hi = wf.amin(-1, keepdim=True), wf.amax(-1, keepdim=True)
    best = None
    for n in (15.0, 14.0, 13.0, 12.0):
        scale = ((hi - lo) / n).clamp_min(1e-8).to(torch.float16).float()
        zp = torch.round(-lo / scale)
        q = torch.round(wf / scale + zp).clamp(0, 15)
        zs = (zp * scale).to(torch.float16).float()
        err = (q * scale - zs - wf).abs().amax(-1, keepdim=True)
        if best is None:
            best = [err, q, scale, zs]
        else:
            take = err < best[0] * 0.5          # a coarser step must be clearly better (an exact lattice hit)
            best = [torch.where(take, err, best[0]), torch.where(take, q, best[1]), torch.where(take, scale, best[2]),
                    torch.where(take, zs, best[3])]
    _, q, scale, zs = best
    q = q.to(torch.uint8).reshape(N, K)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()
    return packed, scale.to(torch.float16).reshape(N, K // g).contiguous(), zs.to(torch.float16).reshape(N, K // g).contiguous()


def pack_w4(q, scale, zero):
    """From integer levels q [N, K] (0..15), scales and integer zero points [N, K/g] to the packed form."""
    q = q.to(torch.uint8)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()
    sb = scale.to(torch.float16)
    return packed, sb.contiguous(), (zero.float() * sb.float()).to(torch.float16).contiguous()


def dequant_w4(packed, scale, zs):
    N, K2 = packed.shape
    K = K2 * 2
    q = torch.empty(N, K, dtype=torch.float32, device=packed.device)
    q[:, 0::2] = (packed & 15).float()
    q[:, 1::2] = (packed >> 4).float()
    g = K // scale.shape[1]
    s = scale.float().repeat_interleave(g, dim=1)
    z = zs.float().repeat_interleave(g, dim=1)
    return q * s - z
