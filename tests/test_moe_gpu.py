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
