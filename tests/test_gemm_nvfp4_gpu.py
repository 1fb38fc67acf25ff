"""NVFP4 GEMM (tcgen05 mxf4nvf4 block-scaled MMA) and its activation quantiser against the fp32 statement."""
import pytest
import torch

from ksanallm_b200.ops import native, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def test_quant_nvfp4_matches_reference():
    torch.manual_seed(0)
    x = (torch.randn(300, 1024, device=DEV) * torch.exp2(torch.randint(-4, 5, (300, 1), device=DEV).float())).to(torch.bfloat16)
    ts = (x.float().abs().amax() / (448.0 * 6.0)).reshape(())
    q, bs, _ = native.quant_nvfp4(x, ts)
    q_r, bs_r, _ = ref.quant_nvfp4(x, ts)
    assert (bs.view(torch.uint8) != bs_r.view(torch.uint8)).float().mean() < 1e-3
    assert (q != q_r).float().mean() < 5e-3                       # reciprocal vs division rounding on a few ties
    d, d_r = ref.dequant_nvfp4(q, bs, ts), ref.dequant_nvfp4(q_r, bs_r, ts)
    assert rel_err(d, d_r) < 2e-2 and rel_err(d, x) < 0.15


@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 256, 256), (128, 128, 512, 128), (300, 1000, 768, 0), (77, 264, 1024, 128),
                                      (1000, 7168, 2048, 0), (4096, 4096, 7168, 256)])
def test_gemm_nvfp4(M, N, K, bn):
    g = torch.Generator(device="cpu").manual_seed(M + N + K)
    # rows / 16-blocks of very different magnitude: a scale applied to the wrong row or block shows up grossly
    x = torch.randn(M, K, generator=g) * torch.exp2(torch.randint(-3, 4, (M, 1), generator=g).float())
    x = x * torch.exp2(torch.randint(-2, 3, (1, K // 16), generator=g).float()).repeat_interleave(16, 1)
    w = torch.randn(N, K, generator=g) * 0.05 * torch.exp2(torch.randint(-3, 4, (N, 1), generator=g).float())
    w = w * torch.exp2(torch.randint(-2, 3, (1, K // 16), generator=g).float()).repeat_interleave(16, 1)
    x, w = x.to(DEV, torch.bfloat16), w.to(DEV)
    wq, w_bs, w_ts = ref.quant_nvfp4(w)
    a_ts = (x.float().abs().amax() / (448.0 * 6.0)).reshape(())
    aq, a_bs, _ = native.quant_nvfp4(x, a_ts)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        y = native.gemm_nvfp4(aq, a_bs, a_ts, wq, w_bs, w_ts, bias=bias, residual=res, bn=bn)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    want = ref.gemm_nvfp4(aq, a_bs, a_ts, wq, w_bs, w_ts, bias, res, out_dtype=torch.float32)
    assert rel_err(y, want) < 1e-2, rel_err(y, want)
    yf = torch.empty(M, N, device=DEV, dtype=torch.float32)
    native.gemm_nvfp4(aq, a_bs, a_ts, wq, w_bs, w_ts, out_f32=yf, bn=bn)
    assert rel_err(yf, ref.gemm_nvfp4(aq, a_bs, a_ts, wq, w_bs, w_ts, out_dtype=torch.float32)) < 2e-3
