"""Numerics of every sm_100a kernel against the plain PyTorch fp32 statement of the same op."""
import math

import pytest
import torch

from ksanallm_b200.ops import native, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


@pytest.mark.parametrize("M,N,K,bn", [
    (128, 256, 512, 0), (256, 512, 1024, 128), (200, 328, 576, 64), (1, 4096, 4096, 0), (17, 1024, 2048, 32),
    (1024, 4096, 4096, 256), (4096, 10240, 8192, 0), (3000, 2048, 8192, 0),
])
def test_gemm_bf16(M, N, K, bn):
    torch.manual_seed(0)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    y = native.gemm_bf16(x, w, bn=bn)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    want = ref.gemm(x, w, out_dtype=torch.float32)
    assert rel_err(y, want) < 1e-2, (M, N, K, bn, rel_err(y, want))


@pytest.mark.parametrize("B,M,N,K", [(16, 64, 512, 128), (128, 300, 128, 512), (3, 1000, 264, 72), (1, 130, 512, 128)])
def test_gemm_bf16_batched_head_interleaved(B, M, N, K):
    """Batched tcgen05 GEMM on head-interleaved views (the absorbed-query and value projections of latent attention):
    operand [M, B, Kpad] read per head through a three-dimensional tensor map, result written into a slice of a
    wider [M, B, Npad] tensor; against the fp32 batched product. Columns outside the slice stay untouched."""
    torch.manual_seed(B + M)
    kpad, npad = K + 64, N + 64
    x = torch.randn(M, B, kpad, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(B, N, K, device=DEV, dtype=torch.bfloat16) * 0.1
    out = torch.full((M, B, npad), 3.0, device=DEV, dtype=torch.bfloat16)
    a = x[..., :K].transpose(0, 1)
    native.gemm_bf16_batched(a, w, out[..., :N].transpose(0, 1))
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    want = torch.bmm(a.float(), w.float().transpose(1, 2)).transpose(0, 1)
    assert rel_err(out[..., :N], want) < 1e-2
    assert bool((out[..., N:] == 3.0).all())


def test_gemm_bf16_epilogue():
    torch.manual_seed(1)
    M, N, K = 300, 1024, 768
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    y = native.gemm_bf16(x, w, bias=bias, residual=res)
    want = ref.gemm(x, w, bias, res, out_dtype=torch.float32)
    assert rel_err(y, want) < 1e-2
    yf = torch.empty(M, N, device=DEV, dtype=torch.float32)
    native.gemm_bf16(x, w, out_f32=yf)
    assert rel_err(yf, ref.gemm(x, w, out_dtype=torch.float32)) < 2e-3
    # in-place residual accumulate (out aliases residual), as the decoder layers use it
    res2 = res.clone()
    native.gemm_bf16(x, w, out=res2, residual=res2)
    assert rel_err(res2, ref.gemm(x, w, None, res, out_dtype=torch.float32)) < 1e-2


@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 512, 128), (300, 1280, 1024, 64), (5, 4096, 8192, 32),
                                       (2048, 8192, 8192, 128), (1000, 7168, 3584, 0), (4096, 10240, 8192, 256),
                                       (300, 1000, 1024, 256), (2500, 57344, 1024, 0)])
def test_gemm_fp8_block(M, N, K, bn):
    torch.manual_seed(2)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.float32) * 0.05
    wq, ws = ref.quant_weight_fp8_block(w)
    xq, xs = native.quant_fp8(x)
    xq_r, xs_r = ref.quant_fp8(x)
    # identical up to e4m3 rounding ties (the kernel multiplies by the reciprocal scale)
    assert (xq.float() != xq_r.float()).float().mean() < 1e-3
    assert torch.allclose(xs[:, :M], xs_r, rtol=1e-6)
    y = native.gemm_fp8(xq, xs, wq, ws, bn=bn)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    want = ref.gemm_fp8(xq, xs, wq, ws, out_dtype=torch.float32)
    assert rel_err(y, want) < 1e-2, rel_err(y, want)
    # and the quantised product stays close to the unquantised one
    assert rel_err(y, x.float() @ w.t()) < 6e-2


@pytest.mark.parametrize("kind", ["bf16", "fp8"])
@pytest.mark.parametrize("M,N,K,splits", [(1, 512, 1024, 0), (8, 8192, 8192, 0), (16, 1280, 8192, 37), (17, 4096, 4096, 7),
                                            (64, 57344, 8192, -1), (64, 8192, 28672, -1), (128, 1000, 2048, 3),
                                            (100, 128256, 1024, -1), (8, 10240, 8192, 0), (32, 57344, 8192, 0),
                                            (3, 8192, 28672, 0), (8, 7168, 8192, 1)])
def test_gemm_smallm(kind, M, N, K, splits):
    torch.manual_seed(5)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    if kind == "bf16":
        w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
        for _ in range(2):   # twice: the tile counters must come back to zero
            y = native.gemm_bf16(x, w, bias=bias, residual=res, splits=splits)
        want = ref.gemm(x, w, bias, res, out_dtype=torch.float32)
        yf = torch.empty(M, N, device=DEV, dtype=torch.float32)
        native.gemm_bf16(x, w, out_f32=yf, splits=splits)
        assert rel_err(yf, ref.gemm(x, w, out_dtype=torch.float32)) < 3e-3
    else:
        w = torch.randn(N, K, device=DEV, dtype=torch.float32) * 0.05
        wq, ws = ref.quant_weight_fp8_block(w)
        xq, xs = native.quant_fp8(x)
        for _ in range(2):
            y = native.gemm_fp8(xq, xs, wq, ws, bias=bias, residual=res, splits=splits)
        want = ref.gemm_fp8(xq, xs, wq, ws, bias, res, out_dtype=torch.float32)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    assert rel_err(y, want) < 1e-2, rel_err(y, want)
    # in-place residual accumulate
    r2 = res.clone()
    if kind == "bf16":
        native.gemm_bf16(x, w, out=r2, residual=r2, splits=splits)
        assert rel_err(r2, ref.gemm(x, w, None, res, out_dtype=torch.float32)) < 1e-2


@pytest.mark.parametrize("H", [256, 4096, 8192, 5120])
@pytest.mark.parametrize("layernorm", [False, True])
def test_norm(H, layernorm):
    torch.manual_seed(3)
    M = 37
    x = torch.randn(M, H, device=DEV, dtype=torch.bfloat16)
    r = torch.randn(M, H, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(H, device=DEV, dtype=torch.bfloat16)
    beta = torch.randn(H, device=DEV, dtype=torch.bfloat16) if layernorm else None
    want, want_res = ref.norm(x, w, 1e-5, r, beta, layernorm)
    r2 = r.clone()
    y = native.norm(x, w, 1e-5, residual=r2, beta=beta, layernorm=layernorm)
    assert rel_err(y, want) < 1e-2
    assert torch.equal(r2, want_res)
    y2 = native.norm(x, w, 1e-5, beta=beta, layernorm=layernorm)
    assert rel_err(y2, ref.norm(x, w, 1e-5, None, beta, layernorm)[0]) < 1e-2
    if H % 128 == 0:
        y3, q, s = native.norm(x, w, 1e-5, beta=beta, layernorm=layernorm, quant=True)
        q_r, s_r = ref.quant_fp8(y3)
        assert torch.allclose(s[:, :M], s_r, rtol=1e-6)
        assert (q.float() != q_r.float()).float().mean() < 1e-3


@pytest.mark.parametrize("kind,gated", [("silu", True), ("gelu", True), ("relu", False), ("gelu", False)])
def test_act_mul(kind, gated):
    torch.manual_seed(4)
    M, inter = 33, 1024
    x = torch.randn(M, inter * (2 if gated else 1), device=DEV, dtype=torch.bfloat16)
    y = native.act_mul(x, kind, gated)
    assert rel_err(y, ref.act_mul(x, kind, gated)) < 1e-2
    y2, q, s = native.act_mul(x, kind, gated, quant=True)
    q_r, s_r = ref.quant_fp8(y2)
    assert torch.allclose(s[:, :M], s_r, rtol=1e-6)
    assert (q.float() != q_r.float()).float().mean() < 1e-3


def test_embedding_and_gather():
    torch.manual_seed(5)
    V, H, T = 1000, 512, 77
    table = torch.randn(V, H, device=DEV, dtype=torch.bfloat16)
    ids = torch.randint(0, 2 * V, (T,), device=DEV, dtype=torch.int32)
    y = native.embedding(ids, table, vocab_lo=V // 2)
    assert torch.equal(y, ref.embedding(ids, table, vocab_lo=V // 2))
    pos_table = torch.randn(128, H, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 128, (T,), device=DEV, dtype=torch.int32)
    ids2 = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    y2 = native.embedding(ids2, table, positions=pos, pos_table=pos_table, scale=2.0)
    assert rel_err(y2, ref.embedding(ids2, table, positions=pos, pos_table=pos_table, scale=2.0)) < 1e-2
    idx = torch.randint(0, T, (9,), device=DEV, dtype=torch.int32)
    assert torch.equal(native.gather_rows(y, idx), y[idx.long()])


def _make_paged(B, q_lens, kv_lens, Hq, Hkv, D, bt, fp8=False, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    nblk_seq = [(k + bt - 1) // bt for k in kv_lens]
    total = sum(nblk_seq) + 3
    perm = torch.randperm(total, generator=g)
    table = torch.zeros(B, max(nblk_seq), dtype=torch.int32)
    c = 0
    for s in range(B):
        table[s, : nblk_seq[s]] = perm[c: c + nblk_seq[s]]
        c += nblk_seq[s]
    cache = (torch.randn(total, 2, Hkv, bt, D, generator=g) * 0.5)
    cache = cache.to(torch.float8_e4m3fn) if fp8 else cache.to(torch.bfloat16)
    T = sum(q_lens)
    q = torch.randn(T, Hq * D, generator=g).to(torch.bfloat16)
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    return q.to(DEV), cache.to(DEV), table.to(DEV), cu_q.to(DEV), torch.tensor(kv_lens, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 1, 128), (4, 2, 64), (32, 8, 128), (8, 8, 128)])
@pytest.mark.parametrize("fp8", [False, True])
def test_paged_prefill(Hq, Hkv, D, fp8):
    q_lens, kv_lens = [70, 1, 33, 128], [70, 50, 100, 300]
    B, bt = 4, 16
    q, cache, table, cu_q, kvl = _make_paged(B, q_lens, kv_lens, Hq, Hkv, D, bt, fp8)
    out = torch.zeros(q.shape[0], Hq * D, device=DEV, dtype=torch.bfloat16)
    ks, vs = (0.5, 0.25) if fp8 else (1.0, 1.0)
    native.paged_prefill(q, q.stride(0), out, cache, cache.stride(0), bt, table, cu_q, kvl, B, max(q_lens), Hq, Hkv, D,
                         1 / math.sqrt(D), k_scale=ks, v_scale=vs)
    want = ref.paged_attention(q, cache, table, cu_q, kvl, Hq, Hkv, D, 1 / math.sqrt(D), k_scale=ks, v_scale=vs)
    assert rel_err(out, want) < 2e-2, rel_err(out, want)


@pytest.mark.parametrize("tc", [True, False])
@pytest.mark.parametrize("Hq,Hkv,bt,alibi", [(16, 2, 16, False), (8, 8, 32, True), (4, 1, 64, False)])
def test_paged_prefill_long(Hq, Hkv, bt, alibi, tc):
    """Chunked prefill with a cached prefix, several KV tiles per query tile; tcgen05 kernel and general kernel."""
    D = 128
    q_lens, kv_lens = [1000, 77, 513], [1500, 77, 2048]
    B = len(q_lens)
    q, cache, table, cu_q, kvl = _make_paged(B, q_lens, kv_lens, Hq, Hkv, D, bt, False, seed=7)
    # rows past a sequence's end inside its last block hold NaN: they must not leak into the output
    last_blk, last = table[1, (kv_lens[1] - 1) // bt].long(), kv_lens[1] % bt
    cache[last_blk, :, :, last:] = float("nan")
    # the layer's blocks sit inside a per-block record that holds several layers, as in the engine's cache
    record = torch.zeros(cache.shape[0], 3, *cache.shape[1:], device=DEV, dtype=cache.dtype)
    record[:, 1] = cache
    cache = record[:, 1]
    slopes = torch.tensor([2.0 ** (-(i + 1) / 2) for i in range(Hq)], device=DEV, dtype=torch.float32) if alibi else None
    out = torch.zeros(q.shape[0], Hq * D, device=DEV, dtype=torch.bfloat16)
    old = native.PREFILL_TC
    native.PREFILL_TC = tc
    try:
        native.paged_prefill(q, q.stride(0), out, cache, cache.stride(0), bt, table, cu_q, kvl, B, max(q_lens), Hq, Hkv, D,
                             1 / math.sqrt(D), alibi=slopes)
        torch.cuda.synchronize()
        native.check_err_flag(DEV)
    finally:
        native.PREFILL_TC = old
    want = ref.paged_attention(q, torch.nan_to_num(cache), table, cu_q, kvl, Hq, Hkv, D, 1 / math.sqrt(D), alibi=slopes)
    assert rel_err(out, want) < 2e-2, rel_err(out, want)


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 1, 128), (4, 2, 64), (64, 8, 128), (16, 16, 128)])
@pytest.mark.parametrize("splits", [1, 4])
@pytest.mark.parametrize("fp8", [False, True])
def test_paged_decode(Hq, Hkv, D, splits, fp8):
    kv_lens = [1, 17, 64, 65, 700, 2304]
    B, bt = len(kv_lens), 16
    q, cache, table, cu_q, kvl = _make_paged(B, [1] * B, kv_lens, Hq, Hkv, D, bt, fp8, seed=1)
    out = torch.zeros(B, Hq * D, device=DEV, dtype=torch.bfloat16)
    po = torch.empty(B * Hq * splits * D, device=DEV, dtype=torch.float32)
    pml = torch.empty(B * Hq * splits * 2, device=DEV, dtype=torch.float32)
    alibi = None
    if Hq == 16:
        alibi = torch.tensor([2.0 ** (-(i + 1) / 2) for i in range(Hq)], device=DEV, dtype=torch.float32)
    native.paged_decode(q, q.stride(0), out, cache, cache.stride(0), bt, table, kvl, B, Hq, Hkv, D, 1 / math.sqrt(D),
                        alibi=alibi, num_splits=splits, part_o=po, part_ml=pml)
    want = ref.paged_attention(q, cache, table, cu_q, kvl, Hq, Hkv, D, 1 / math.sqrt(D), alibi=alibi)
    assert rel_err(out, want) < 2e-2, rel_err(out, want)
    if D == 128:
        # the same launch can emit the FP8 operand of the next GEMM: bit-identical to quantising its bf16 output
        oq = torch.zeros(B, Hq * D, device=DEV, dtype=torch.float8_e4m3fn)
        osc = torch.zeros(Hq, 8, device=DEV, dtype=torch.float32)
        native.paged_decode(q, q.stride(0), None, cache, cache.stride(0), bt, table, kvl, B, Hq, Hkv, D, 1 / math.sqrt(D),
                            alibi=alibi, num_splits=splits, part_o=po, part_ml=pml, out_q=oq, out_scale=osc)
        wq, ws = native.quant_fp8(out)
        assert torch.equal(oq.view(torch.uint8), wq.view(torch.uint8))
        assert torch.equal(osc[:, :B], ws[:, :B])


@pytest.mark.parametrize("neox", [True, False])
@pytest.mark.parametrize("fp8", [False, True])
def test_rope_kv_append(neox, fp8):
    torch.manual_seed(7)
    T, Hq, Hkv, D, bt, nblk, rot = 50, 8, 2, 128, 16, 12, 64
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(nblk * bt, device=DEV)[:T].to(torch.int32)
    slots[3] = -1
    cs = ref.build_cos_sin_cache(rot, 512, 10000.0, device=DEV)
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    cache = torch.zeros(nblk, 2, Hkv, bt, D, device=DEV, dtype=dt)
    cache_r = cache.clone()
    qkv_r = qkv.clone()
    ks, vs = (0.5, 2.0) if fp8 else (1.0, 1.0)
    native.rope_kv_append(qkv, pos, slots, cs, cache, cache.stride(0), bt, Hq, Hkv, D, rot, neox, k_scale=ks, v_scale=vs)
    ref.rope_kv_append(qkv_r, pos, slots, cs, cache_r, bt, Hq, Hkv, D, rot, neox, k_scale=ks, v_scale=vs)
    assert rel_err(qkv, qkv_r) < 1e-2
    assert rel_err(cache.float(), cache_r.float()) < (7e-2 if fp8 else 1e-2)


def test_sampler_greedy_and_topk():
    torch.manual_seed(8)
    B, V = 6, 128256
    logits = torch.randn(B, V, device=DEV, dtype=torch.float32) * 3
    temp = torch.tensor([1.0, 0.7, 1.3, 1.0, 0.5, 1.0], device=DEV)
    topk = torch.tensor([1, 50, 1024, 1, 5, 200], device=DEV, dtype=torch.int32)
    topp = torch.tensor([1.0, 0.9, 1.0, 0.5, 0.3, 0.95], device=DEV)
    seeds = torch.arange(B, device=DEV, dtype=torch.int64) + 1234
    steps = torch.zeros(B, device=DEV, dtype=torch.int32)
    out = torch.zeros(B, device=DEV, dtype=torch.int32)
    native.sample(logits, temp, topk, topp, seeds, steps, out)
    am = logits.argmax(-1)
    assert int(out[0]) == int(am[0]) and int(out[3]) == int(am[3])
    for b in (1, 2, 4, 5):
        k = int(topk[b])
        allowed = set(torch.topk(logits[b], k).indices.tolist())
        assert int(out[b]) in allowed
    # log-probs: top-N of temperature-scaled logits, log-softmax over those N only
    N = 5
    lp_ids = torch.zeros(B, N, device=DEV, dtype=torch.int32)
    lp_vals = torch.zeros(B, N, device=DEV, dtype=torch.float32)
    native.sample(logits, temp, topk, topp, seeds, steps, out, num_logprobs=N, lp_ids=lp_ids, lp_vals=lp_vals)
    _, want_ids, want_vals = ref.sample(logits.cpu(), temp.cpu(), topk.cpu(), topp.cpu(), torch.zeros(B), N)
    assert torch.equal(lp_ids.cpu().long(), want_ids)
    assert torch.allclose(lp_vals.cpu(), want_vals, atol=1e-3)
    assert int(out[0]) == int(am[0])


def test_sampler_distribution():
    # empirical frequencies of a 4-way top-k draw follow the softmax of the 4 largest logits
    V, n = 1000, 4000
    logits = torch.full((n, V), -10.0, device=DEV)
    logits[:, 10], logits[:, 20], logits[:, 30], logits[:, 40] = 2.0, 1.0, 0.0, -1.0
    out = torch.zeros(n, device=DEV, dtype=torch.int32)
    native.sample(logits, torch.ones(n, device=DEV), torch.full((n,), 4, device=DEV, dtype=torch.int32),
                  torch.ones(n, device=DEV), torch.full((n,), 7, device=DEV, dtype=torch.int64),
                  torch.arange(n, device=DEV, dtype=torch.int32), out)
    p = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0]), 0)
    freq = torch.tensor([(out == t).float().mean().item() for t in (10, 20, 30, 40)])
    assert freq.sum() > 0.999 and (freq - p).abs().max() < 0.03


def test_penalties_and_blocks():
    B, V = 2, 100
    logits = torch.ones(B, V, device=DEV)
    offsets = torch.tensor([0, 2, 3], device=DEV, dtype=torch.int32)
    ids = torch.tensor([5, 7, 9], device=DEV, dtype=torch.int32)
    native.repetition_penalty(logits, offsets, ids, torch.tensor([2.0, 4.0], device=DEV))
    assert logits[0, 5] == 0.5 and logits[0, 7] == 0.5 and logits[1, 9] == 0.25 and logits[1, 5] == 1.0
    native.ban_tokens(logits, offsets, ids)
    assert logits[0, 5] == float("-inf") and logits[1, 9] == float("-inf")
    cache = torch.randn(8, 4096, device=DEV).to(torch.bfloat16)
    want = cache.clone()
    want[6], want[7] = want[1], want[2]
    native.copy_blocks(cache, torch.tensor([1, 6, 2, 7], device=DEV, dtype=torch.int32), 4096 * 2)
    assert torch.equal(cache, want)
    # swaps: (device block, host block) pairs against a pinned host pool, moved by the kernel itself
    pool = torch.zeros(4, 4096 * 2, dtype=torch.uint8).pin_memory()
    native.swap_blocks(cache, pool, torch.tensor([3, 2, 5, 0], device=DEV, dtype=torch.int32), 4096 * 2, True)
    torch.cuda.synchronize()
    assert torch.equal(pool[2].view(torch.bfloat16), cache[3].cpu()) and torch.equal(pool[0].view(torch.bfloat16), cache[5].cpu())
    before = cache.clone()
    native.swap_blocks(cache, pool, torch.tensor([1, 2, 4, 0], device=DEV, dtype=torch.int32), 4096 * 2, False)
    torch.cuda.synchronize()
    assert torch.equal(cache[1], before[3]) and torch.equal(cache[4], before[5]) and torch.equal(cache[0], before[0])
    # block ids outside the cache or the pool are skipped and reported through the error word
    native.check_err_flag(DEV)
    native.copy_blocks(cache, torch.tensor([1, 99], device=DEV, dtype=torch.int32), 4096 * 2)
    with pytest.raises(RuntimeError, match="block-table entry"):
        native.check_err_flag(DEV)
    native.swap_blocks(cache, pool, torch.tensor([2, 7], device=DEV, dtype=torch.int32), 4096 * 2, True)
    with pytest.raises(RuntimeError, match="block-table entry"):
        native.check_err_flag(DEV)
    assert torch.equal(cache[1], before[3])


def test_peer_wait_runs_out_and_reports_through_the_error_word():
    """Failure detection on the device without a fault: a barrier over two "ranks" whose buffers are both plain local
    allocations; the second rank never signals, the wait's budget is about a millisecond, the kernel returns, the error
    word reads 3 (peer wait ran out), and the next launch on the same context works."""
    import ctypes as C
    lib = native.lib()
    lib.ksana_comm_set_spin_limit.argtypes = [C.c_int]
    lib.ksana_comm_set_spin_limit.restype = None
    native.check_err_flag(DEV)
    pads = [torch.zeros(4096, dtype=torch.uint8, device=DEV) for _ in range(2)]     # flag pad of rank 0 and of the absent rank 1
    ptrs = (C.c_ulonglong * 8)(*([p.data_ptr() for p in pads] + [0] * 6))
    ctrs = torch.zeros(16, dtype=torch.int32, device=DEV)
    err = native.err_flag(DEV)
    st = torch.cuda.current_stream().cuda_stream
    lib.ksana_comm_set_spin_limit(5000)
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        rc = lib.ksana_comm_barrier(ptrs, ptrs, 0, 2, ctrs.data_ptr(), err.data_ptr(), st)
        t1.record()
        assert rc == 0
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 200.0                       # gave up within its budget (milliseconds, not a second)
        assert int(err.item()) == 3
        with pytest.raises(RuntimeError, match="peer"):
            native.check_err_flag(DEV)                            # the host side turns the word into an error and clears it
        assert int(ctrs[2].item()) == 0                           # the barrier's epoch did not advance
        # the context is intact: a one-rank barrier and an ordinary kernel run afterwards
        rc = lib.ksana_comm_barrier(ptrs, ptrs, 0, 1, ctrs.data_ptr(), err.data_ptr(), st)
        assert rc == 0
        x = torch.randn(4, 256, device=DEV, dtype=torch.bfloat16)
        y = native.add(x, x)
        torch.cuda.synchronize()
        assert int(err.item()) == 0 and int(ctrs[2].item()) == 1
        assert torch.equal(y, (x.float() * 2).to(torch.bfloat16))
    finally:
        lib.ksana_comm_set_spin_limit(0)


@pytest.mark.parametrize("kv_dtype", [torch.bfloat16, torch.float8_e4m3fn])
@pytest.mark.parametrize("neox", [True, False])
def test_rerotate_blocks_matches_tensor_ops(kv_dtype, neox):
    """Flexible-cache copies: K rows of the destination blocks rotated by the position delta, kernel against the
    fp32 tensor statement (rotation by |delta| with the sign on the sine); V and other blocks untouched; a block id
    outside the pool is recorded and skipped."""
    from ksanallm_b200.ops import reference as ref
    nb, layers, hkv, bt, D, rot = 12, 3, 2, 16, 128, 64
    cache = (torch.randn(nb, layers, 2, hkv, bt, D, device=DEV) * 2).to(kv_dtype)
    before = cache.clone()
    cs = ref.build_cos_sin_cache(rot, 512, 10000.0, None, DEV)
    triples = torch.tensor([[0, 3, 37], [1, 5, -120], [2, 7, 0], [4, 9, 511]], dtype=torch.int32, device=DEV)
    native.rerotate_blocks(cache, triples, cs, rot, neox)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    half = rot // 2
    for _, dst, delta in triples.tolist():
        k = before[dst, :, 0].float()
        if delta != 0:
            c, s = cs[abs(delta)][:half], cs[abs(delta)][half:] * (1.0 if delta > 0 else -1.0)
            r = k[..., :rot]
            if neox:
                x0, x1 = r[..., :half], r[..., half:]
                out = torch.cat([x0 * c - x1 * s, x1 * c + x0 * s], -1)
            else:
                x0, x1 = r[..., 0::2], r[..., 1::2]
                out = torch.stack([x0 * c - x1 * s, x1 * c + x0 * s], -1).flatten(-2)
            k = k.clone()
            k[..., :rot] = out
        got, want = cache[dst, :, 0].float(), k.to(kv_dtype).float()
        # one rounding step apart at most (the kernel may contract the multiply-adds)
        step = 0.008 if kv_dtype == torch.bfloat16 else 0.13
        assert bool(((got - want).abs() <= step * want.abs() + 2e-3).all())
        assert float((got - want).norm() / want.norm()) < (1e-3 if kv_dtype == torch.bfloat16 else 2e-2)
        if delta == 0:
            assert torch.equal(got, want)
        assert torch.equal(cache[dst, :, 1].view(torch.uint8), before[dst, :, 1].view(torch.uint8))
    untouched = [b for b in range(nb) if b not in (3, 5, 7, 9)]
    assert torch.equal(cache[untouched].view(torch.uint8), before[untouched].view(torch.uint8))
    bad = torch.tensor([[0, nb + 4, 5]], dtype=torch.int32, device=DEV)
    native.rerotate_blocks(cache, bad, cs, rot, neox)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError):
        native.check_err_flag(DEV)
    native.clear_err_flag(DEV)


def test_absmax_scale_on_device():
    """Tensor scale of an NVFP4 activation computed on the device: max |x| / divisor with a floor, strided rows, and the
    scratch word left at zero so that back-to-back calls are independent."""
    torch.manual_seed(3)
    big = torch.randn(300, 1024 + 64, device=DEV, dtype=torch.bfloat16) * 3
    x = big[:, :1024]                                    # rows 1088 elements apart
    x[17, 400] = -77.5
    s = native.absmax_scale(x, 448.0 * 6.0)
    torch.cuda.synchronize()
    assert s.shape == () and abs(float(s) - 77.5 / (448.0 * 6.0)) < 1e-7
    y = torch.randn(8, 64, device=DEV, dtype=torch.bfloat16) * 0.01
    s2 = native.absmax_scale(y, 448.0 * 6.0)
    assert abs(float(s2) - float(y.float().abs().amax()) / (448.0 * 6.0)) < 1e-9      # not the larger value of the first call
    z = torch.zeros(4, 16, device=DEV, dtype=torch.bfloat16)
    assert float(native.absmax_scale(z, 6.0, floor=1e-12)) == pytest.approx(1e-12)
