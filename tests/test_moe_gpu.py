"""MoE kernels (routing, alignment, permutation, grouped tcgen05 GEMM, combine) against PyTorch."""
import pytest
import torch

from ksanallm_b200.config import ModelConfig
from ksanallm_b200.models.moe import route_reference
from ksanallm_b200.ops import native, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


@pytest.mark.parametrize("E,K,scoring,groups", [(8, 2, "softmax", (1, 1)), (60, 4, "softmax", (1, 1)),
                                                 (256, 8, "sigmoid", (8, 4)), (64, 6, "sigmoid", (1, 1))])
def test_route(E, K, scoring, groups):
    torch.manual_seed(0)
    T = 37
    logits = torch.randn(T, E, device=DEV)
    bias = torch.randn(E, device=DEV) * 0.1 if scoring == "sigmoid" else None
    cfg = ModelConfig(num_experts=E, num_experts_per_tok=K, moe_scoring=scoring, n_group=groups[0], topk_group=groups[1],
                      routed_scaling_factor=2.5 if scoring == "sigmoid" else 1.0, norm_topk_prob=True)
    ids, w = native.moe_route(logits, K, scoring, True, cfg.routed_scaling_factor, bias, groups[0], groups[1])
    want_ids, want_w = route_reference(logits, cfg, bias)
    assert torch.equal(ids.long().sort(-1).values, want_ids.sort(-1).values)
    order = ids.long().argsort(-1)
    worder = want_ids.argsort(-1)
    assert torch.allclose(w.gather(1, order), want_w.gather(1, worder), rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("quant", [False, True])
def test_grouped_moe_pipeline(quant):
    torch.manual_seed(1)
    T, H, I, E, K = 300, 512, 256, 8, 2
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    w13 = torch.randn(E * 2 * I, H, device=DEV) * 0.05
    w2 = torch.randn(E * H, I, device=DEV) * 0.05
    logits = torch.randn(T, E, device=DEV)
    ids, w = native.moe_route(logits, K, "softmax", True, 1.0)
    dst_row, tile_expert, offsets, total, cap = native.moe_align(ids, E)
    # every (token,k) row is unique, lands in its expert's segment
    rows = dst_row.long()
    assert rows.unique().numel() == T * K
    off = offsets.long()
    e_of_row = torch.bucketize(rows, off[1:], right=True)
    assert torch.equal(e_of_row, ids.long().reshape(-1))
    perm = native.moe_permute(x, dst_row, K, cap)
    assert torch.equal(perm[rows], x.repeat_interleave(K, 0))
    if quant:
        w13q, w13s = ref.quant_weight_fp8_block(w13)
        w2q, w2s = ref.quant_weight_fp8_block(w2)
        perm[:] = torch.where(torch.isfinite(perm.float()), perm.float(), torch.zeros(1, device=DEV)).to(torch.bfloat16)
        pq, ps = native.quant_fp8(perm)
        g = native.gemm_grouped(pq, w13q, tile_expert, E, 2 * I, a_scale=ps, w_scale=w13s)
        _, aq, as_ = native.act_mul(g, "silu", True, quant=True, want_out=False)
        y = native.gemm_grouped(aq, w2q, tile_expert, E, H, a_scale=as_, w_scale=w2s)
        w13d, w2d = ref.dequant_weight_fp8_block(w13q, w13s), ref.dequant_weight_fp8_block(w2q, w2s)
        tol = 6e-2
    else:
        g = native.gemm_grouped(perm, w13.to(torch.bfloat16), tile_expert, E, 2 * I)
        a = native.act_mul(g, "silu", True)
        y = native.gemm_grouped(a, w2.to(torch.bfloat16), tile_expert, E, H)
        w13d, w2d = w13.to(torch.bfloat16).float(), w2.to(torch.bfloat16).float()
        tol = 2e-2
    out = torch.zeros(T, H, device=DEV, dtype=torch.bfloat16)
    native.moe_combine(y, dst_row, w, out, K, accumulate=False)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    want = torch.zeros(T, H, device=DEV)
    for e in range(E):
        tok, slot = (ids.long() == e).nonzero(as_tuple=True)
        gu = x[tok].float() @ w13d[e * 2 * I:(e + 1) * 2 * I].t()
        a = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        want.index_add_(0, tok, (a @ w2d[e * H:(e + 1) * H].t()) * w[tok, slot].unsqueeze(-1))
    assert rel_err(out, want) < tol, rel_err(out, want)


def test_grouped_nvfp4_gemm_against_fp32_statement():
    """Grouped NVFP4 GEMM: every 128-row tile of expert-major rows times its expert's e2m1 matrix (e4m3 block scales,
    one tensor scale per expert) against the dequantised fp32 product; rows of unused tiles are not touched."""
    torch.manual_seed(2)
    E, N, K, cap = 5, 384, 512, 128 * 7
    tile_expert = torch.tensor([0, 0, 2, -1, 4, 4, 3], dtype=torch.int32, device=DEV)
    a = torch.randn(cap, K, device=DEV, dtype=torch.bfloat16)
    a_ts = (a.float().abs().amax() / (448.0 * 6.0)).reshape(())
    aq, abs_, _ = native.quant_nvfp4(a, a_ts)
    ws = [torch.randn(N, K, device=DEV) * (0.02 * (e + 1)) for e in range(E)]
    qs = [ref.quant_nvfp4(w) for w in ws]
    wq, wbs = torch.cat([q[0] for q in qs]).contiguous(), torch.cat([q[1] for q in qs]).contiguous()
    wts = torch.stack([q[2] for q in qs]).float().contiguous()
    out = torch.full((cap, N), 7.0, device=DEV, dtype=torch.bfloat16)
    for bn in (0, 128):
        native.gemm_grouped_nvfp4(aq, abs_, a_ts, wq, wbs, wts, tile_expert, E, N, out=out, bn=bn)
        torch.cuda.synchronize()
        native.check_err_flag(DEV)
        ad = ref.dequant_nvfp4(aq, abs_, a_ts)
        for t, e in enumerate(tile_expert.tolist()):
            rows = slice(128 * t, 128 * (t + 1))
            if e < 0:
                assert bool((out[rows] == 7.0).all())
                continue
            want = ad[rows] @ ref.dequant_nvfp4(qs[e][0], qs[e][1], qs[e][2]).t()
            assert rel_err(out[rows], want) < 1e-2, (t, e, rel_err(out[rows], want))


def test_moe_block_with_nvfp4_experts_matches_cpu_statement():
    """An MoE block whose routed experts are NVFP4 (weights and activations) on the GPU against the same block
    restated with dequantised operands on the CPU."""
    from ksanallm_b200.models.weights import RandomSource, build_model
    cfg = ModelConfig(model_type="mixtral", hidden_size=512, num_layers=1, num_heads=4, num_kv_heads=2, head_dim=128,
                      intermediate_size=512, moe_intermediate_size=512, vocab_size=1000, num_experts=8,
                      num_experts_per_tok=2, max_position_embeddings=256, max_token_len=256)
    from ksanallm_b200.models.moe import moe_partial
    gpu = build_model(cfg, RandomSource(seed=4, std=0.05), device=DEV, dtype=torch.bfloat16, quant="nvfp4")
    cpu = build_model(cfg, RandomSource(seed=4, std=0.05), device="cpu", dtype=torch.bfloat16, quant="nvfp4")
    mw_g, mw_c = gpu.layers[0].moe, cpu.layers[0].moe
    assert mw_g.nvfp4 and mw_c.nvfp4
    assert torch.equal(mw_g.w13.cpu(), mw_c.w13) and torch.equal(mw_g.w2_bs.cpu().view(torch.uint8), mw_c.w2_bs.view(torch.uint8))
    x = torch.randn(200, 512, dtype=torch.bfloat16) * 0.5
    got = moe_partial(gpu, mw_g, x.to(DEV)).float().cpu()
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    want = moe_partial(cpu, mw_c, x).float()
    assert rel_err(got, want) < 0.12, rel_err(got, want)      # e2m1 bucket flips of the second GEMM's input


def test_moe_block_with_restricted_choices_matches_cpu_statement():
    """Routing decided elsewhere with some choices struck out (id -1, weight 0: held by another rank under all-to-all
    dispatch): the GPU block computes only the remaining ones, raises no guard, and agrees with the CPU statement."""
    from ksanallm_b200.models.moe import moe_partial, route
    from ksanallm_b200.models.weights import RandomSource, build_model
    cfg = ModelConfig(model_type="mixtral", hidden_size=512, num_layers=1, num_heads=4, num_kv_heads=2, head_dim=128,
                      intermediate_size=512, moe_intermediate_size=256, vocab_size=1000, num_experts=8,
                      num_experts_per_tok=2, max_position_embeddings=256, max_token_len=256)
    gpu = build_model(cfg, RandomSource(seed=5, std=0.05), device=DEV, dtype=torch.bfloat16)
    cpu = build_model(cfg, RandomSource(seed=5, std=0.05), device="cpu", dtype=torch.bfloat16)
    mw_g, mw_c = gpu.layers[0].moe, cpu.layers[0].moe
    x = torch.randn(150, 512, dtype=torch.bfloat16) * 0.5
    ids, w = route(gpu, mw_g, x.to(DEV))
    keep = ids < 4                                   # as if experts 4..7 lived on another rank
    ids_r = torch.where(keep, ids, torch.full_like(ids, -1)).contiguous()
    w_r = torch.where(keep, w, torch.zeros_like(w)).contiguous()
    assert bool((ids_r == -1).any()) and bool(keep.any())
    got = moe_partial(gpu, mw_g, x.to(DEV), shared=False, routing=(ids_r, w_r)).float().cpu()
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    want = moe_partial(cpu, mw_c, x, shared=False, routing=(ids_r.cpu(), w_r.cpu())).float()
    assert rel_err(got, want) < 2e-2, rel_err(got, want)
    rows_without = (~keep).all(dim=1).cpu()
    assert float(got[rows_without].abs().max()) == 0.0 if bool(rows_without.any()) else True
